"""B200-native LLM serving framework (sm_100a kernels, NVLink-fused collectives)."""
__version__ = "0.1.0"

from .sampling_params import SamplingParams  # noqa: F401


def __getattr__(name):
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    if name == "LLMEngine":
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    raise AttributeError(name)
