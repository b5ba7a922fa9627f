"""whirl_llm_b200: WHIRL's token-sampling hot path for NVIDIA B200 (sm_100a).

The product is ``libwhirl_b200.so`` (hand-written CUDA kernels behind the C ABI of ``include/whirl_b200.h``).  This
package is the thin Python host side over it: ctypes bindings that take torch tensors for device memory and streams.
There is no CPU or PyTorch fallback: if the library is missing or fails to load, importing ``whirl_llm_b200.api`` raises.
"""
__all__ = ["api", "build"]
