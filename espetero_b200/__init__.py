"""B200-native attention path for Espetero's forest pass (paged-KV GQA decode, causal
prefill, tree verify, split-K merge, FP8 KV): CUDA kernels for sm_100a behind the C ABI of
include/espetero_attn.h. The Python modules here are the test / benchmark harness around
that library; the product is the shared library."""

__all__ = ["capi", "workloads"]
