"""gemmallm_b200: GemmaLLM's Mixture-of-Experts feed-forward block as
hand-written CUDA kernels for NVIDIA B200 (sm_100a), behind the C ABI of
include/moe_b200.h. ``MOE`` and ``FeedForward`` are drop-ins for the reference
classes of model.py:154-276."""
from .moe import MOE, FeedForward  # noqa: F401
from ._cabi import MoeB200Error  # noqa: F401

__all__ = ["MOE", "FeedForward", "MoeB200Error"]
