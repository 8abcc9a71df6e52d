"""dinfer_b200: a small, whole inference engine for one B200 (sm_100a), from a model folder
(config.json + safetensors) to generated tokens."""
__version__ = "0.1.0"

from .sampling.params import SamplingParams  # noqa: F401


def __getattr__(name):
    # LLM pulls in torch and the kernels; import it only when asked for
    if name in ("LLM", "RequestOutput"):
        from .engine import llm
        return getattr(llm, name)
    raise AttributeError(name)
