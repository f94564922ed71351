"""photon_infer_b200: a small, whole LLM inference engine for one GPU (NVIDIA B200, sm_100a).

    from photon_infer_b200 import ContinuousBatchEngine, EngineOptions
    engine = ContinuousBatchEngine("model_folder", EngineOptions(dtype="bfloat16"))
    rid = engine.add_request([1, 5, 9], max_new_tokens=32)
    tokens = engine.run_until_complete()[rid]
"""
__version__ = "0.1.0"

from .config import EngineOptions, LlamaConfig, load_config, register_architecture  # noqa: F401
from .errors import ErrorCode, PhotonError  # noqa: F401


def __getattr__(name):
    # the engine pulls in the CUDA side; import it on first use
    if name in ("ContinuousBatchEngine", "generate"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "write_random_model":
        from .weights import write_random_model
        return write_random_model
    raise AttributeError(name)
