"""tokamak_b200: a single-GPU inference engine for the Qwen3 dense decoder on NVIDIA B200."""

from .sampling.params import SamplingParams

__version__ = "0.1.0"

__all__ = ["LLM", "RequestOutput", "SamplingParams", "__version__"]


def __getattr__(name):
    # the engine imports torch and loads the CUDA library; keep `import tokamak_b200` light
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    if name == "RequestOutput":
        from .engine.outputs import RequestOutput
        return RequestOutput
    raise AttributeError(name)
