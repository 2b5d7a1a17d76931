"""mini_llm_b200: a small, whole GPT-2 inference engine for one B200 (sm_100a).

Configuration and registry (``config``), safetensors weights (``weights``), model
parts and their assembly (``parts``, ``models``), paged cache manager (``cache``),
step function, scheduler and entry point (``engine``), sampling (``sampling``),
hand-written CUDA kernels (``csrc``, reached through ``ops``).
"""
from .config.base import (ConfigError, EngineConfig, config_from_dict, load_config, register_architecture,
                          registered_architectures)
from .parts import attention, block, embedding, head, mlp, norm, positions  # noqa: F401  (register the parts)
from .parts.base import register_part
from .models import gpt2  # noqa: F401  (registers GPT2LMHeadModel)
from .weights.random_init import write_random_model
from .sampling.params import SamplingParams
from .engine.request import Request, RequestState, Response


def __getattr__(name):
    if name == "LLM":          # needs CUDA at construction only; imported on demand
        from .engine.llm import LLM
        return LLM
    raise AttributeError(name)


__all__ = ["ConfigError", "EngineConfig", "config_from_dict", "load_config", "register_architecture",
           "registered_architectures", "register_part", "write_random_model", "SamplingParams", "Request",
           "RequestState", "Response", "LLM"]
__version__ = "0.1.0"
