"""Writes the golden logits under this folder from WeichunK/tokamak's own model code.

Run on the CPU, once, with the reference's source tree given on the command line:

    python tests/golden/make_golden.py --reference-src <checkout>/src

For tiny configurations A and B it writes seeded random float32 weights with
this repository's writer, loads the folder into the reference's
``TransformerForCausalLM`` with the reference's own ``load_weights``, runs a whole
sequence through ``PrefillContext`` over a ``ContiguousKVCache`` and stores the
float32 logits of every position, the token ids, and a digest of the weights
(so that a change of the random generator is noticed rather than mistaken for a
numerical fault).  ``tests/test_plain.py`` compares the plain implementation
with these files.  The window configuration is not covered: the reference has no
per-layer window.
"""

from __future__ import annotations

import argparse
import hashlib
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))


def weights_digest(tensors: dict) -> str:
    h = hashlib.sha256()
    for name in sorted(tensors):
        h.update(name.encode())
        h.update(tensors[name].to(torch.float32).contiguous().numpy().tobytes())
    return h.hexdigest()


def golden_tokens(vocab: int, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (length,), generator=gen).tolist()


def reference_logits(tag: str):
    """(logits [T, V] float32, token ids, digest of the weights) of tiny configuration ``tag``
    from the reference's own model code, which must be importable (``tokamak`` on ``sys.path``)."""
    from tokamak.config import ModelConfig
    from tokamak.model.kv_cache import ContiguousKVCache
    from tokamak.model.loader import build_model, load_weights
    from tokamak.model.step_context import PrefillContext

    import tiny_configs
    from plain import qwen3_plain as plain
    from tokamak_b200.weights import write_random_model

    raw, init, _page = tiny_configs.ALL[tag]
    with tempfile.TemporaryDirectory() as d:
        write_random_model(d, raw, dtype="float32", **init)
        cfg_json, tensors = plain.load_folder(d)
        cfg = ModelConfig(
            architecture="Qwen3ForCausalLM", vocab_size=raw["vocab_size"],
            hidden_size=raw["hidden_size"], num_layers=raw["num_hidden_layers"],
            num_attention_heads=raw["num_attention_heads"],
            num_kv_heads=raw["num_key_value_heads"], head_dim=raw["head_dim"],
            intermediate_size=raw["intermediate_size"], rms_norm_eps=raw["rms_norm_eps"],
            rope_theta=plain.rope_theta_of(raw),
            max_position_embeddings=raw["max_position_embeddings"],
            tie_word_embeddings=raw["tie_word_embeddings"], attention_bias=False,
            use_qk_norm=True, eos_token_ids=())
        model = build_model(cfg, torch.device("cpu"), torch.float32)
        load_weights(model, Path(d))
        ids = golden_tokens(raw["vocab_size"], 40, init["seed"])
        cache = ContiguousKVCache(cfg, max_seq_len=64, device=torch.device("cpu"),
                                  dtype=torch.float32)
        with torch.no_grad():
            hidden = model(torch.tensor([ids]), torch.arange(len(ids))[None], PrefillContext(cache))
            logits = model.compute_logits(hidden)[0]
        return logits.contiguous(), ids, weights_digest(tensors)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True)
    args = ap.parse_args()
    sys.path.insert(0, args.reference_src)

    from safetensors.torch import save_file

    for tag in ("A", "B"):
        logits, ids, digest = reference_logits(tag)
        save_file({"logits": logits, "token_ids": torch.tensor(ids, dtype=torch.int32)},
                  str(HERE / f"tiny_{tag}.safetensors"), metadata={"weights_sha256": digest})
        print(tag, tuple(logits.shape), digest[:16])


if __name__ == "__main__":
    main()
