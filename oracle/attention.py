"""CPU restatement of the quantized flash-attention math (test infrastructure only).

Two numeric modes, matching the two operator entry points of the package:

ref mode  -- what the reference kernels compute (quant_flash_attn.py):
    Q stays in its 16-bit dtype, a single quantized tensor serves as K and V,
    it is dequantized with the stored fp16 scale and rounded to Q's dtype
    (quant_flash_attn.py:65-66), forward pre-scales Q by sm_scale and rounds it
    (quant_flash_attn.py:50-52), natural-exp softmax, LSE = m + log l
    (quant_flash_attn.py:70-79).  Backward follows quant_flash_attn.py:153-164,
    including dKV = dV + sm_scale * dK.

int8 mode -- the int8 x int8 extension: Q, K and V are all quantized per token,
    the logits come from the exact integer identity
        sum_d (q-zq)(k-zk) = q.k - zk*sum(q) - zq*sum(k) + D*zq*zk
    scaled by s_q*s_k*sm_scale, causal masking uses the rule row >= column
    (flash_attn_triton.py:50), V is dequantized and rounded to the 16-bit dtype
    as in quant_flash_attn.py:65-66.  Gradients are those of the same function
    of the dequantized operands (straight-through to q, k, v).

Everything is evaluated in fp32 (fp64 optional) without tiling, so the only
differences to a GPU kernel are the kernel's own 16-bit roundings of P / dS and
fp32 summation order; the tolerances in the tests cover those.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .quantizer import quantize_per_token


def attention_ops(B, H, Sq, Skv, D, causal=False):
    """Forward op count, 4*B*H*D*P (test_speed.py:111-112; causal counts the kept pairs)."""
    if not causal:
        pairs = Sq * Skv
    elif Sq <= Skv:
        pairs = Sq * (Sq + 1) // 2
    else:
        pairs = Skv * (Skv + 1) // 2 + (Sq - Skv) * Skv
    return 4 * B * H * D * pairs


def _dequant_t(codes: torch.Tensor, scale_f16: torch.Tensor, zp: torch.Tensor) -> torch.Tensor:
    # quant_flash_attn.py:65 -- fp32 (code - zp) * scale with the stored fp16 scale
    return (codes.float() - zp.float()) * scale_f16.float()


def _quantize_t(x: torch.Tensor):
    """Oracle quantizer on a torch tensor (..., D); returns torch tensors."""
    codes, _s32, s16, zp, rs = quantize_per_token(x.float().numpy())
    return (torch.from_numpy(codes), torch.from_numpy(s16.astype(np.float32)),
            torch.from_numpy(zp), torch.from_numpy(rs))


# --------------------------------------------------------------------------- ref mode

def ref_mode_forward(q, codes, scale_f16, zp, sm_scale, compute=torch.float32, round_output=True):
    """q (Z,H,NQ,D) fp16/bf16; codes (Z,H,NKV,D) int8; scale/zp (Z,H,NKV,1).
    Returns O (q dtype, or un-rounded when round_output is False) and LSE (Z,H,NQ) fp32.
    quant_flash_attn.py:50-83."""
    kv = _dequant_t(codes, scale_f16, zp).to(q.dtype)                      # :65-66
    qs = (q.float() * sm_scale).to(q.dtype)                               # :52 (fp32 product, rounded)
    s = qs.to(compute) @ kv.to(compute).transpose(-1, -2)                  # :68
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    o = (p @ kv.to(compute)) / l                                           # :75-78
    lse = (m + torch.log(l)).squeeze(-1)                                   # :79
    return (o.to(q.dtype) if round_output else o), lse.float()


def ref_mode_backward(q, codes, scale_f16, zp, sm_scale, o, lse, do, compute=torch.float32, round_output=True):
    """Returns (dq, dkv) in q's dtype (un-rounded when round_output is False).
    quant_flash_attn.py:88-101 and :133-166."""
    kv = _dequant_t(codes, scale_f16, zp).to(q.dtype).to(compute)          # :150-151
    delta = (o.to(compute) * do.to(compute)).sum(-1, keepdim=True)         # :99
    qf, dof = q.to(compute), do.to(compute)
    s = (qf @ kv.transpose(-1, -2)) * sm_scale                             # :153 (q NOT pre-rounded)
    p = torch.exp(s - lse.to(compute).unsqueeze(-1))                       # :155
    dv = p.transpose(-1, -2) @ dof                                         # :156
    dp = dof @ kv.transpose(-1, -2)                                        # :157
    ds = p * (dp - delta)                                                  # :158
    dq = (ds @ kv) * sm_scale                                              # :159,164
    dk = ds.transpose(-1, -2) @ qf                                         # :160
    dkv = dv + dk * sm_scale                                               # :161
    return (dq.to(q.dtype), dkv.to(q.dtype)) if round_output else (dq, dkv)


# --------------------------------------------------------------------------- int8 mode

def int8_mode_logits(qq, kq, sm_scale, causal, compute=torch.float32):
    """qq/kq = (codes, scale, zp, rowsum) torch tensors with leading (B,H,S) dims.
    Returns the scaled logits with -inf where masked."""
    qc, qs, qz, qsum = qq
    kc, ks, kz, ksum = kq
    D = qc.shape[-1]
    # exact integer matmul (|acc| <= 128*128*D fits fp64 and int32)
    acc = (qc.double() @ kc.double().transpose(-1, -2))
    zq = qz.double().unsqueeze(-1)
    zk = kz.double().unsqueeze(-2)
    corr = acc - zk * qsum.double().unsqueeze(-1) - zq * ksum.double().unsqueeze(-2) + D * zq * zk
    s = corr.to(compute) * (qs.to(compute).unsqueeze(-1) * ks.to(compute).unsqueeze(-2)) * sm_scale
    if causal:
        sq, sk = s.shape[-2], s.shape[-1]
        keep = torch.arange(sq).unsqueeze(-1) >= torch.arange(sk).unsqueeze(0)   # flash_attn_triton.py:50
        s = s.masked_fill(~keep, float("-inf"))
    return s


def int8_mode_quantize(x):
    """Per-token quantization of (B,H,S,D) -> (codes, scale(fp32 value of the fp16 scale), zp, rowsum)."""
    return _quantize_t(x)


def int8_mode_forward(q, k, v, causal, sm_scale, compute=torch.float32, quant=None, round_output=True):
    """q,k,v (B,H,S,D) 16-bit.  Returns O (q dtype), LSE (B,H,Sq) fp32 and the
    quantized operands (for the backward).

    `quant` = ((codes, scale, zp, rowsum),)*3 for q, k, v overrides the CPU quantizer, so
    that attention can be judged on exactly the operands a GPU quantizer produced (GPU
    division is not IEEE, see quantizer.py); scale is the fp32 value of the stored fp16
    scale, shapes (B,H,S)."""
    if quant is None:
        qq, kq, vq = _quantize_t(q), _quantize_t(k), _quantize_t(v)
    else:
        qq, kq, vq = quant
    s = int8_mode_logits(qq, kq, sm_scale, causal, compute)
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    vhat = _dequant_t(vq[0], vq[1].unsqueeze(-1), vq[2].unsqueeze(-1)).to(q.dtype).to(compute)
    o = (p @ vhat) / l
    lse = (m + torch.log(l)).squeeze(-1)
    return (o.to(q.dtype) if round_output else o), lse.float(), (qq, kq, vq)


def int8_mode_backward(quant, causal, sm_scale, o, lse, do, dtype, compute=torch.float32, round_output=True):
    """Gradients of int8_mode_forward w.r.t. the dequantized operands
    (straight-through): returns dq, dk, dv in `dtype` (un-rounded when round_output is False)."""
    qq, kq, vq = quant
    s = int8_mode_logits(qq, kq, sm_scale, causal, compute)
    p = torch.exp(s - lse.to(compute).unsqueeze(-1))
    qhat = _dequant_t(qq[0], qq[1].unsqueeze(-1), qq[2].unsqueeze(-1)).to(compute)
    khat = _dequant_t(kq[0], kq[1].unsqueeze(-1), kq[2].unsqueeze(-1)).to(compute)
    vhat = _dequant_t(vq[0], vq[1].unsqueeze(-1), vq[2].unsqueeze(-1)).to(dtype).to(compute)
    dof = do.to(compute)
    delta = (o.to(compute) * dof).sum(-1, keepdim=True)
    dv = p.transpose(-1, -2) @ dof
    dp = dof @ vhat.transpose(-1, -2)
    ds = p * (dp - delta)
    dq = (ds @ khat) * sm_scale
    dk = (ds.transpose(-1, -2) @ qhat) * sm_scale
    return (dq.to(dtype), dk.to(dtype), dv.to(dtype)) if round_output else (dq, dk, dv)


def default_sm_scale(D):
    return 1.0 / math.sqrt(D)
