"""Loads a model folder and assembles model, cache and step function on one GPU."""

from __future__ import annotations

import logging
from pathlib import Path

import torch

from ..cache.device import DeviceCache, plan_groups
from ..cache.manager import CacheManager
from ..config import architecture_of, read_config_json, read_eos_token_ids
from ..models.decoder import DecoderModel
from ..parts.base import Runtime
from ..weights.loader import load_tensors
from .step import StepFunction

logger = logging.getLogger(__name__)

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, "auto": torch.bfloat16}


def resolve_dtype(dtype: str | torch.dtype) -> torch.dtype:
    """``auto`` is bfloat16, the serving dtype (src/tokamak/config.py:167-180); float32
    selects the true 32-bit path."""
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"Unknown dtype spec: {dtype!r}")
        return dtype
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"Unknown dtype spec: {dtype!r}") from None


def require_cuda(device: str | torch.device = "cuda") -> torch.device:
    """The engine runs on a CUDA device only; there is no CPU path to fall back to."""
    dev = torch.device("cuda" if device == "auto" else device)
    if dev.type != "cuda":
        raise RuntimeError(f"tokamak_b200 runs on CUDA devices only, got {dev}")
    if not torch.cuda.is_available():
        raise RuntimeError("tokamak_b200 needs a CUDA device and none is available")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    return dev


class EngineCore:
    """Configuration, model, cache and step function of one model folder.

    Args:
        model: folder with ``config.json`` and ``*.safetensors``.
        dtype: ``bfloat16`` (serving kernels) or ``float32`` (everything in true 32-bit).
        max_seq_len: cap on one request's length; defaults to the model's maximum.
        page_size: positions per cache page (``block_size`` of the reference).
        pool_tokens: positions the page pool of every layer group holds; at least
            ``max_seq_len`` so that any single request can finish alone
            (src/tokamak/engine/llm.py:157-163), which is also the default.  ``"auto"`` sizes
            the pool from the device memory that is free once the weights are loaded:
            ``memory_utilization`` of it, less room for the activations of the largest step.
        memory_utilization: share of the free device memory that ``pool_tokens="auto"`` may use.
        max_slots: most requests that are live at a time.
        max_step_tokens: most tokens of one step.
        tensors, raw_config: weights and configuration given directly instead of read from
            the folder (random weights made on the device, for measurements).
        window: the engine-wide attention window (``None``: what the configuration says); an
            architecture that does not take the option refuses it.
    """

    def __init__(self, model: str | Path, *, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda", max_seq_len: int | None = None,
                 page_size: int = 16, pool_tokens: int | str | None = None, max_slots: int = 16,
                 max_step_tokens: int | None = None, tensors: dict | None = None,
                 raw_config: dict | None = None, window: int | None = None,
                 memory_utilization: float = 0.9):
        self.device = require_cuda(device)
        self.dtype = resolve_dtype(dtype)
        torch.cuda.set_device(self.device)
        if raw_config is None:
            raw_config = read_config_json(model)
            eos = read_eos_token_ids(model, raw_config)
        else:
            eos = None
        self.raw_config = raw_config
        self.architecture = architecture_of(raw_config)
        self.config = self.architecture.parse(raw_config, eos)
        self.spec = self.architecture.build_spec(self.config, window=window)
        rt = Runtime(device=self.device, dtype=self.dtype)
        if tensors is None:
            expected = DecoderModel.expected_tensors(self.spec)
            tensors = load_tensors(model, expected, self.dtype, self.device)
        self.model = DecoderModel(self.spec, tensors, rt)
        del tensors

        model_max = self.config.max_position_embeddings
        self.max_seq_len = min(max_seq_len or model_max, model_max)
        if page_size < 1:
            raise ValueError(f"block_size must be >= 1, got {page_size}")
        self.max_step_tokens = max_step_tokens or max(self.max_seq_len, max_slots)
        if pool_tokens == "auto":
            pool_tokens = self._pool_tokens_from_free_memory(page_size, max_slots, memory_utilization)
        elif isinstance(pool_tokens, str):
            raise ValueError(f"kv_pool_tokens must be a number of tokens or 'auto', got {pool_tokens!r}")
        pool_tokens = pool_tokens or self.max_seq_len
        if pool_tokens < self.max_seq_len:
            raise ValueError(f"kv_pool_tokens ({pool_tokens}) must be >= max_seq_len "
                             f"({self.max_seq_len}) so any single request can complete alone")
        kv_groups, state_groups = plan_groups(self.model.cache_needs(), pool_tokens, page_size)
        self.manager = CacheManager(kv_groups, state_groups, max_slots)
        self.cache = DeviceCache(self.manager, self.dtype, self.device, self.max_seq_len)
        self.page_size = page_size
        self.step = StepFunction(self.model, self.cache, self.max_step_tokens, self.max_seq_len)
        logger.info("Loaded %s (%s) on %s as %s: %d pages of %d tokens per layer group",
                    model, self.config.architecture, self.device, self.dtype,
                    kv_groups[0].num_pages if kv_groups else 0, page_size)


    def _pool_tokens_from_free_memory(self, page_size: int, max_slots: int, utilization: float) -> int:
        """Positions that fit into the free device memory beside the activations of one step.

        The activations are measured, not estimated: a throw-away cache of the smallest allowed
        size carries one step of the largest allowed size, and the allocator's peak during that
        step is what the real pool leaves free (whatever parts the model is made of)."""
        from ..cache.manager import KVPagesNeed
        from .step import StepEntry
        if not 0.0 < utilization <= 1.0:
            raise ValueError(f"memory_utilization must be in (0, 1], got {utilization}")
        elem = 4 if self.dtype == torch.float32 else 2
        per_token = sum(2 * need.n_kv_heads * need.head_dim * elem
                        for need in self.model.cache_needs().values() if isinstance(need, KVPagesNeed))
        smallest = -(-self.max_seq_len // page_size) * page_size
        if per_token == 0:
            return smallest
        kv_groups, state_groups = plan_groups(self.model.cache_needs(), smallest, page_size)
        manager = CacheManager(kv_groups, state_groups, max_slots)
        cache = DeviceCache(manager, self.dtype, self.device, self.max_seq_len)
        step = StepFunction(self.model, cache, self.max_step_tokens, self.max_seq_len, use_graphs=False)
        n = min(self.max_step_tokens, self.max_seq_len)
        torch.cuda.synchronize(self.device)
        torch.cuda.reset_peak_memory_stats(self.device)
        before = torch.cuda.memory_allocated(self.device)
        step.run([StepEntry("probe", [0] * n, [n - 1])])
        torch.cuda.synchronize(self.device)
        peak = torch.cuda.max_memory_allocated(self.device) - before
        del step, cache, manager, kv_groups, state_groups
        torch.cuda.empty_cache()
        # the float32 logits of a full decode batch come on top of what one wanted row needed
        workspace = int(1.25 * peak) + 8 * max_slots * self.config.vocab_size
        free, _ = torch.cuda.mem_get_info(self.device)
        budget = int(free * utilization) - workspace
        tokens = max(budget, 0) // per_token // page_size * page_size
        logger.info("free device memory %.1f GB, step workspace %.2f GB: pool of %d tokens",
                    free / 1e9, workspace / 1e9, max(tokens, smallest))
        return max(tokens, smallest)


def random_core(raw_config: dict, *, seed: int = 0, std: float = 0.02, norm_std: float = 0.1,
                dtype: str | torch.dtype = "bfloat16", device: str | torch.device = "cuda",
                **kwargs) -> EngineCore:
    """An engine with seeded random weights made directly on the device (no folder is written).

    For measurements at sizes whose checkpoint would take minutes to write and read.  The
    values come from the device's generator, so they differ from a folder written with the
    same seed by :func:`tokamak_b200.weights.write_random_model`.
    """
    from ..weights.random_init import random_tensors

    dev = require_cuda(device)
    dt = resolve_dtype(dtype)
    arch = architecture_of(raw_config)
    spec = arch.build_spec(arch.parse(raw_config), window=kwargs.get("window"))
    expected = DecoderModel.expected_tensors(spec)
    tensors = random_tensors(expected, seed, std, norm_std, dt, device=dev)
    for name, req in expected.items():
        if req.role == "vector" and name in tensors:
            tensors[name] = tensors[name].float()
    return EngineCore("<random>", dtype=dt, device=dev, tensors=tensors, raw_config=raw_config, **kwargs)
