"""photon_infer_b200: a small, whole LLM inference engine for one GPU (NVIDIA B200, sm_100a)."""
__version__ = "0.1.0"
