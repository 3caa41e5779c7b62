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

Everything is evaluated in fp32 (fp64 optional).  Two switches bring the evaluation
closer to what the kernels (and the reference's Triton kernels) do with 16-bit operands:

round_p=<dtype>  the second products take 16-bit left operands, exactly as the reference
    does: `tl.dot(p.to(q_dtype), v)` (quant_flash_attn.py:75; the row sum l keeps the
    un-rounded p, :73), `p.to(do.dtype)`, `ds_block.to(...)` (quant_flash_attn.py:156,
    159-160); in int8 mode Q^ and K^ of the backward are rounded to the dtype as the
    dequantizing kernel writes them (quant_flash_attn.py:150-151 does the same to K^).
    P is taken relative to the exact row maximum (one block covering the row).
row_chunk=<n>    query rows are processed n at a time, so that a 32k x 32k logit
    matrix never exists; results do not depend on it.

With round_p=None the only differences to a GPU kernel are the kernel's own 16-bit
roundings of P / dS and fp32 summation order.
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

def ref_mode_forward(q, codes, scale_f16, zp, sm_scale, compute=torch.float32, round_output=True, round_p=False):
    """q (Z,H,NQ,D) fp16/bf16; codes (Z,H,NKV,D) int8; scale/zp (Z,H,NKV,1).
    Returns O (q dtype, or un-rounded when round_output is False) and LSE (Z,H,NQ) fp32.
    quant_flash_attn.py:50-83."""
    kv = _dequant_t(codes, scale_f16, zp).to(q.dtype)                      # :65-66
    qs = (q.float() * sm_scale).to(q.dtype)                               # :52 (fp32 product, rounded)
    s = qs.to(compute) @ kv.to(compute).transpose(-1, -2)                  # :68
    m = s.max(dim=-1, keepdim=True).values
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)                                        # :73 (un-rounded p)
    if round_p:
        p = p.to(q.dtype).to(compute)                                      # :75
    o = (p @ kv.to(compute)) / l                                           # :75-78
    lse = (m + torch.log(l)).squeeze(-1)                                   # :79
    return (o.to(q.dtype) if round_output else o), lse.float()


def ref_mode_backward(q, codes, scale_f16, zp, sm_scale, o, lse, do, compute=torch.float32, round_output=True,
                      round_p=False):
    """Returns (dq, dkv) in q's dtype (un-rounded when round_output is False).
    quant_flash_attn.py:88-101 and :133-166."""
    kv = _dequant_t(codes, scale_f16, zp).to(q.dtype).to(compute)          # :150-151
    delta = (o.to(compute) * do.to(compute)).sum(-1, keepdim=True)         # :99
    qf, dof = q.to(compute), do.to(compute)
    s = (qf @ kv.transpose(-1, -2)) * sm_scale                             # :153 (q NOT pre-rounded)
    p = torch.exp(s - lse.to(compute).unsqueeze(-1))                       # :155
    rnd = (lambda t: t.to(q.dtype).to(compute)) if round_p else (lambda t: t)
    dv = rnd(p).transpose(-1, -2) @ dof                                    # :156
    dp = dof @ kv.transpose(-1, -2)                                        # :157
    ds = rnd(p * (dp - delta))                                             # :158, rounded at :159-160
    dq = (ds @ kv) * sm_scale                                              # :159,164
    dk = ds.transpose(-1, -2) @ qf                                         # :160
    dkv = dv + dk * sm_scale                                               # :161
    return (dq.to(q.dtype), dkv.to(q.dtype)) if round_output else (dq, dkv)


# --------------------------------------------------------------------------- int8 mode

def int8_mode_logits(qq, kq, sm_scale, causal, compute=torch.float32, rows=None):
    """qq/kq = (codes, scale, zp, rowsum) torch tensors with leading (B,H,S) dims.
    Returns the scaled logits with -inf where masked.  `rows` = (r0, r1) restricts the
    query rows (the causal mask keeps using the absolute row index)."""
    qc, qs, qz, qsum = qq
    kc, ks, kz, ksum = kq
    r0, r1 = (0, qc.shape[-2]) if rows is None else rows
    qc, qs, qz, qsum = qc[..., r0:r1, :], qs[..., r0:r1], qz[..., r0:r1], qsum[..., r0:r1]
    D = qc.shape[-1]
    # exact integer matmul: every partial sum is an integer below 128*128*D <= 2**21, so fp32 holds it exactly
    assert D <= 512
    acc = (qc.float() @ kc.float().transpose(-1, -2)).double()
    zq = qz.double().unsqueeze(-1)
    zk = kz.double().unsqueeze(-2)
    corr = acc - zk * qsum.double().unsqueeze(-1) - zq * ksum.double().unsqueeze(-2) + D * zq * zk
    s = corr.to(compute) * (qs.to(compute).unsqueeze(-1) * ks.to(compute).unsqueeze(-2)) * sm_scale
    if causal:
        sk = s.shape[-1]
        keep = torch.arange(r0, r1).unsqueeze(-1) >= torch.arange(sk).unsqueeze(0)   # flash_attn_triton.py:50
        s = s.masked_fill(~keep, float("-inf"))
    return s


def _chunks(n, step):
    step = n if not step else int(step)
    return [(a, min(n, a + step)) for a in range(0, n, step)]


def int8_mode_quantize(x):
    """Per-token quantization of (B,H,S,D) -> (codes, scale(fp32 value of the fp16 scale), zp, rowsum)."""
    return _quantize_t(x)


def int8_mode_forward(q, k, v, causal, sm_scale, compute=torch.float32, quant=None, round_output=True,
                      round_p=None, row_chunk=None):
    """q,k,v (B,H,S,D) 16-bit.  Returns O (q dtype), LSE (B,H,Sq) fp32 and the
    quantized operands (for the backward).

    `quant` = ((codes, scale, zp, rowsum),)*3 for q, k, v overrides the CPU quantizer, so
    that attention can be judged on exactly the operands a GPU quantizer produced (GPU
    division is not IEEE, see quantizer.py); scale is the fp32 value of the stored fp16
    scale, shapes (B,H,S).  `round_p`, `row_chunk`: see the module docstring."""
    if quant is None:
        qq, kq, vq = _quantize_t(q), _quantize_t(k), _quantize_t(v)
    else:
        qq, kq, vq = quant
    vhat = _dequant_t(vq[0], vq[1].unsqueeze(-1), vq[2].unsqueeze(-1)).to(q.dtype).to(compute)
    Sq = qq[0].shape[-2]
    o_parts, lse_parts = [], []
    for rows in _chunks(Sq, row_chunk):
        s = int8_mode_logits(qq, kq, sm_scale, causal, compute, rows)
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)                                        # quant_flash_attn.py:73
        if round_p is not None:
            p = p.to(round_p).to(compute)                                      # quant_flash_attn.py:75
        o_parts.append((p @ vhat) / l)
        lse_parts.append((m + torch.log(l)).squeeze(-1))
    o = torch.cat(o_parts, dim=-2)
    lse = torch.cat(lse_parts, dim=-1)
    return (o.to(q.dtype) if round_output else o), lse.float(), (qq, kq, vq)


def int8_mode_backward(quant, causal, sm_scale, o, lse, do, dtype, compute=torch.float32, round_output=True,
                       round_p=None, row_chunk=None, return_delta=False):
    """Gradients of int8_mode_forward w.r.t. the dequantized operands
    (straight-through): returns dq, dk, dv in `dtype` (un-rounded when round_output is False),
    plus delta = rowsum(o * do) (B,H,Sq) when `return_delta`.  `round_p`, `row_chunk`: see the
    module docstring."""
    qq, kq, vq = quant
    qhat = _dequant_t(qq[0], qq[1].unsqueeze(-1), qq[2].unsqueeze(-1))
    khat = _dequant_t(kq[0], kq[1].unsqueeze(-1), kq[2].unsqueeze(-1))
    if round_p is not None:
        qhat, khat = qhat.to(round_p), khat.to(round_p)
    qhat, khat = qhat.to(compute), khat.to(compute)
    vhat = _dequant_t(vq[0], vq[1].unsqueeze(-1), vq[2].unsqueeze(-1)).to(dtype).to(compute)
    dof = do.to(compute)
    delta_all = (o.to(compute) * dof).sum(-1, keepdim=True)                    # quant_flash_attn.py:99
    rnd = (lambda t: t.to(round_p).to(compute)) if round_p is not None else (lambda t: t)
    dq_parts = []
    dk = torch.zeros_like(khat)
    dv = torch.zeros_like(vhat)
    for r0, r1 in _chunks(qhat.shape[-2], row_chunk):
        s = int8_mode_logits(qq, kq, sm_scale, causal, compute, (r0, r1))
        p = torch.exp(s - lse[..., r0:r1].to(compute).unsqueeze(-1))           # :155
        dv += rnd(p).transpose(-1, -2) @ dof[..., r0:r1, :]                    # :156
        dp = dof[..., r0:r1, :] @ vhat.transpose(-1, -2)                       # :157
        ds = rnd(p * (dp - delta_all[..., r0:r1, :]))                          # :158, rounded at :159-160
        dq_parts.append((ds @ khat) * sm_scale)                                # :159,164
        dk += ds.transpose(-1, -2) @ qhat[..., r0:r1, :]                       # :160
    dq = torch.cat(dq_parts, dim=-2)
    dk = dk * sm_scale
    out = (dq.to(dtype), dk.to(dtype), dv.to(dtype)) if round_output else (dq, dk, dv)
    return out + (delta_all.squeeze(-1).float(),) if return_delta else out


def default_sm_scale(D):
    return 1.0 / math.sqrt(D)
