"""B200-native per-token INT8 quantizer and INT8 flash attention (forward + backward).

Public entry points (same names and conventions as the reference project's modules):

    asymmetric_quant_per_token(x)                      -> (codes, scale, zero_point)
    quant_flash_attn(q, kv_fp16, kv_quant, sm_scale)   -> o        (autograd: dq, dkv)
    quant_attention(q, k, v, causal, sm_scale)         -> o        (autograd: dq, dk, dv)
    quant_attention_host(q, k, v, causal, sm_scale)    -> o        (host tensors in and out, copies overlapped)
    quant_flash_attn_func(q, k, v, causal=...)         -> o        ((B,S,H,D) layout, grouped K/V heads; also
                                                                    _kvpacked_ and _varlen_ forms)

All of them require a CUDA device and the in-tree shared library libqfa_sm100a.so.
"""
from .asymmetric_quant import (  # noqa: F401
    asymmetric_quant_per_token, asymmetric_quant_per_token_ex, dequantize_per_token,
)
from .quant_flash_attn import (  # noqa: F401
    QuantFlashAttention, quant_flash_attn, QuantAttention, quant_attention,
    quantize_qkv, quant_attention_forward, int8_attention_forward, int8_attention_backward, dequantize_16bit,
    HostAttentionPipeline, quant_attention_host, check_kernel_status,
)
from .flash_attn_interface import (  # noqa: F401
    quant_flash_attn_func, quant_flash_attn_kvpacked_func, quant_flash_attn_varlen_func,
)
from .sharding import all_gather_heads, head_slice, shard_bounds  # noqa: F401
from ._lib import launch_count  # noqa: F401

__all__ = [
    "asymmetric_quant_per_token", "asymmetric_quant_per_token_ex", "dequantize_per_token",
    "QuantFlashAttention", "quant_flash_attn", "QuantAttention", "quant_attention",
    "quantize_qkv", "quant_attention_forward", "int8_attention_forward", "int8_attention_backward", "dequantize_16bit",
    "HostAttentionPipeline", "quant_attention_host", "check_kernel_status",
    "quant_flash_attn_func", "quant_flash_attn_kvpacked_func", "quant_flash_attn_varlen_func",
    "all_gather_heads", "head_slice", "shard_bounds", "launch_count",
]
