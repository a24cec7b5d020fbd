"""gemmallm_b200: GemmaLLM's Mixture-of-Experts feed-forward block as
hand-written CUDA kernels for NVIDIA B200 (sm_100a), behind the C ABI of
include/moe_b200.h. ``MOE`` and ``FeedForward`` are drop-ins for the reference
classes of model.py:154-276, ``Attention`` for the decoder layer's attention
(model.py:59-152) the block sits behind, ``LLMLayer`` for that layer itself (model.py:278-321).

Attributes are resolved on first use so that ``python -m gemmallm_b200.build``
can (re)build libmoe_b200.so before anything tries to load it.
"""
__all__ = ["MOE", "FeedForward", "Attention", "LLMLayer", "MoeB200Error"]


def __getattr__(name):
    if name in ("MOE", "FeedForward"):
        from . import moe
        return getattr(moe, name)
    if name == "Attention":
        from .attention import Attention
        return Attention
    if name == "LLMLayer":
        from .layer import LLMLayer
        return LLMLayer
    if name == "MoeB200Error":
        from ._cabi import MoeB200Error
        return MoeB200Error
    raise AttributeError(f"module 'gemmallm_b200' has no attribute {name!r}")
