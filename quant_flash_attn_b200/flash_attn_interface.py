"""`flash_attn_func`-style front end of the int8 attention operator.

The reference compares itself with Dao's FlashAttention through calls of the form
`flash_attn_func(q, k, v, causal=...)` on `(batch, seqlen, heads, head_dim)` tensors
(compute_flops.py:119-122, test_speed.py:85-87).  This module gives the int8 operator the same call
style, so that a model written against that interface can switch over:

    quant_flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False)
    quant_flash_attn_kvpacked_func(q, kv, ...)
    quant_flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, ...)

Layout: the kernels take element strides for every operand, so the `(B, S, H, D)` tensors are handed to
them as transposed VIEWS; nothing is copied on the way in, and the output is written straight into a
`(B, S, H, D)` tensor.  Grouped-query attention (fewer K/V heads than query heads): without gradients the
K/V heads are quantized once and the forward kernel maps the query heads onto them; with gradients the K/V
heads are repeated first, so that autograd sums each group's gradients.  Packed variable-length batches are
one operator call per sequence.  Under the causal mask query i sees keys j <= i (flash_attn_triton.py:50), i.e. the mask
is aligned to the top-left corner when the two lengths differ.
"""
from __future__ import annotations

import math

import torch

from .quant_flash_attn import int8_attention_forward, quant_attention, quantize_qkv


def _scale(softmax_scale, D: int) -> float:
    return 1.0 / math.sqrt(D) if softmax_scale is None else float(softmax_scale)


def _check(q, k, v, dropout_p):
    if dropout_p != 0.0:
        raise NotImplementedError("the quantized operator has no dropout (the reference has none either)")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("expected q (B,Sq,H,D) and k, v (B,Skv,Hkv,D)")
    if k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3]:
        raise ValueError("expected q (B,Sq,H,D) and k, v (B,Skv,Hkv,D)")
    if q.shape[2] % k.shape[2] != 0:
        raise ValueError("the number of query heads must be a multiple of the number of K/V heads")


def _repeat_kv_heads(x: torch.Tensor, groups: int) -> torch.Tensor:
    """(B,S,Hkv,D) -> (B,S,Hkv*groups,D): query head h reads K/V head h // groups."""
    if groups == 1:
        return x
    B, S, Hkv, D = x.shape
    return x[:, :, :, None, :].expand(B, S, Hkv, groups, D).reshape(B, S, Hkv * groups, D)


def quant_flash_attn_func(q, k, v, dropout_p: float = 0.0, softmax_scale=None, causal: bool = False):
    """q (B,Sq,H,D); k, v (B,Skv,Hkv,D) with H a multiple of Hkv; fp16 or bf16 CUDA tensors.
    Returns the attention output (B,Sq,H,D).  Differentiable in q, k, v (straight-through gradients of the
    quantized operands, as `quant_attention`)."""
    _check(q, k, v, dropout_p)
    groups = q.shape[2] // k.shape[2]
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if groups > 1 and not needs_grad:
        # inference: K and V are quantized once per K/V head and the forward kernel maps query heads onto them
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        qq, kq, vq = quantize_qkv(qt, kt, vt)
        o, _ = int8_attention_forward(qq, kq, vq, bool(causal), _scale(softmax_scale, q.shape[3]), q.dtype,
                                      o=torch.empty_like(qt))
        return o.transpose(1, 2).contiguous()
    k, v = _repeat_kv_heads(k, groups), _repeat_kv_heads(v, groups)
    o = quant_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), bool(causal), _scale(softmax_scale, q.shape[3]))
    # the operator wrote its result in q's memory layout, so this view is already contiguous (B,Sq,H,D)
    return o.transpose(1, 2).contiguous()


def quant_flash_attn_kvpacked_func(q, kv, dropout_p: float = 0.0, softmax_scale=None, causal: bool = False):
    """q (B,Sq,H,D), kv (B,Skv,2,Hkv,D)."""
    if kv.dim() != 5 or kv.shape[2] != 2:
        raise ValueError("expected kv (B,Skv,2,Hkv,D)")
    return quant_flash_attn_func(q, kv[:, :, 0], kv[:, :, 1], dropout_p, softmax_scale, causal)


def quant_flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q=None, max_seqlen_k=None,
                                 dropout_p: float = 0.0, softmax_scale=None, causal: bool = False):
    """Packed variable-length batch: q (total_q,H,D); k, v (total_k,Hkv,D); cu_seqlens_* (batch+1,) int32
    prefix sums of the sequence lengths.  Returns (total_q,H,D).  max_seqlen_* are accepted for signature
    compatibility.  One operator call per sequence; sequences of length zero produce no rows."""
    if dropout_p != 0.0:
        raise NotImplementedError("the quantized operator has no dropout (the reference has none either)")
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3 or k.shape != v.shape:
        raise ValueError("expected q (total_q,H,D) and k, v (total_k,Hkv,D)")
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    ck = [int(x) for x in cu_seqlens_k.tolist()]
    if len(cq) != len(ck) or len(cq) < 2 or cq[0] != 0 or ck[0] != 0 or cq[-1] != q.shape[0] or ck[-1] != k.shape[0]:
        raise ValueError("cu_seqlens_q / cu_seqlens_k do not describe q / k")
    outs = []
    for b in range(len(cq) - 1):
        q0, q1, k0, k1 = cq[b], cq[b + 1], ck[b], ck[b + 1]
        if q1 == q0:
            continue
        if k1 == k0:
            outs.append(torch.zeros_like(q[q0:q1]))         # no keys: softmax over nothing
            continue
        outs.append(quant_flash_attn_func(q[None, q0:q1], k[None, k0:k1], v[None, k0:k1], 0.0, softmax_scale, causal)[0])
    if not outs:
        return torch.zeros_like(q)
    return torch.cat(outs, dim=0)
