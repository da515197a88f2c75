"""Python faces of the CUDA kernels under `csrc/`.  Every function takes torch tensors on the
CUDA device, launches on torch's current stream and raises if the launch is refused.  There is
no CPU path: without a device, or without a compiler for the kernels, these functions fail."""
from .ops import (DT, KernelError, add_rmsnorm, decode_clusters16, decode_fusion_ok, dense_binary, argmax, attention_decode, attention_prefill,
                  embedding, fill_normal, gather_i32, into_plan, launch_count, linear, linear_into, linear_into_ok, linear_swiglu, mlp_fused, mlp_fused_ok, prefill_tc_ok, require_head_dim, residual_add, rope_append, sample, scatter_i32, swiglu, tc_error, tc_plan, uniform)

__all__ = ["DT", "KernelError", "add_rmsnorm", "decode_clusters16", "decode_fusion_ok", "dense_binary", "argmax", "attention_decode", "attention_prefill",
           "embedding", "fill_normal", "gather_i32", "into_plan", "launch_count", "linear", "linear_into", "linear_into_ok", "linear_swiglu", "mlp_fused", "mlp_fused_ok", "prefill_tc_ok", "require_head_dim", "residual_add", "rope_append", "sample", "scatter_i32", "swiglu", "tc_error", "tc_plan", "uniform"]
