"""Per-token asymmetric INT8 quantization (host side).

Mirrors the reference module asymmetric_quant.py: same function name, argument and
return convention (asymmetric_quant.py:109-149); the work is done by the CUDA kernel
behind qfa_quant_per_token.
"""
from __future__ import annotations

import torch

from . import _lib

_DT = {torch.float16: _lib.QFA_F16, torch.bfloat16: _lib.QFA_BF16}


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _quantize(x: torch.Tensor, want_sum: bool, want_dequant: bool):
    if x.dim() != 4:
        raise ValueError("expected a 4-D tensor (Batch, Num_Heads, Seq_Len, Head_Dim)")
    _require_cuda(x, "input_tensor")
    if x.dtype not in _DT:
        raise TypeError(f"expected float16 or bfloat16 input, got {x.dtype}")
    Z, H, M, K = x.shape
    # codes are written with the input's strides (asymmetric_quant.py:64,127)
    codes = torch.empty_like(x, dtype=torch.int8)
    if codes.stride() != x.stride():
        x = x.contiguous()
        codes = torch.empty_like(x, dtype=torch.int8)
    scale = torch.empty(Z, H, M, 1, dtype=torch.float16, device=x.device)
    zp = torch.empty(Z, H, M, 1, dtype=torch.int8, device=x.device)
    rowsum = torch.empty(Z, H, M, dtype=torch.int32, device=x.device) if want_sum else None
    xhat = torch.empty(Z, H, M, K, dtype=x.dtype, device=x.device) if want_dequant else None
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.qfa_quant_dequant_per_token(
            x.data_ptr(), codes.data_ptr(), scale.data_ptr(), zp.data_ptr(),
            rowsum.data_ptr() if want_sum else None, xhat.data_ptr() if want_dequant else None,
            Z, H, M, K, x.stride(0), x.stride(1), x.stride(2), x.stride(3), _DT[x.dtype], _stream(x))
    _lib.check(rc, "qfa_quant_dequant_per_token")
    return codes, scale, zp, rowsum, xhat


def _quantize_batch(tensors, want_dequant, outs=None, want_centered=None):
    """Quantizes several (B,H,S,D) tensors of one dtype on one device with a single library call (one kernel launch
    when they share the head dimension and have 16-byte aligned rows).  `want_dequant[i]` asks for the dequantized
    copy of tensor i, `want_centered[i]` for code - zero_point as fp16 (the K operand of the forward's 16-bit logits
    MMA).  Returns one (codes, scale, zp, rowsum, dequantized-or-None) tuple per tensor -- with the centered tensor
    as a sixth element where it was asked for -- bit-identical to separate `_quantize` calls.  `outs` (optional)
    supplies those tuples pre-allocated: codes with the strides of its input, the others contiguous; nothing is
    allocated then."""
    import ctypes as C
    x0 = tensors[0]
    jobs = (_lib.QfaQuantJob * len(tensors))()
    results, keep = [], []
    if want_centered is None:
        want_centered = (False,) * len(tensors)
    for i, (x, dq, ct) in enumerate(zip(tensors, want_dequant, want_centered)):
        if x.dim() != 4:
            raise ValueError("expected a 4-D tensor (Batch, Num_Heads, Seq_Len, Head_Dim)")
        _require_cuda(x, "input_tensor")
        if x.dtype != x0.dtype or x.dtype not in _DT or x.device != x0.device:
            raise TypeError("expected float16 or bfloat16 tensors of one dtype on one device")
        Z, H, M, K = x.shape
        if outs is not None:
            codes, scale, zp, rowsum, xhat = outs[i][:5]
            ctr = outs[i][5] if len(outs[i]) > 5 else None
            if codes.stride() != x.stride() or (dq and xhat is None) or (ct and ctr is None):
                raise ValueError("pre-allocated quantizer outputs do not match the input")
        else:
            codes = torch.empty_like(x, dtype=torch.int8)    # the input's strides (asymmetric_quant.py:64,127)
            if codes.stride() != x.stride():
                x = x.contiguous()
                codes = torch.empty_like(x, dtype=torch.int8)
            scale = torch.empty(Z, H, M, 1, dtype=torch.float16, device=x.device)
            zp = torch.empty(Z, H, M, 1, dtype=torch.int8, device=x.device)
            rowsum = torch.empty(Z, H, M, dtype=torch.int32, device=x.device)
            xhat = torch.empty(Z, H, M, K, dtype=x.dtype, device=x.device) if dq else None
            ctr = torch.empty(Z, H, M, K, dtype=torch.float16, device=x.device) if ct else None
        jobs[i] = _lib.QfaQuantJob(x.data_ptr(), codes.data_ptr(), scale.data_ptr(), zp.data_ptr(), rowsum.data_ptr(),
                                   xhat.data_ptr() if dq else None, Z, H, M, K, *x.stride(),
                                   ctr.data_ptr() if ct else None)
        keep.append(x)
        results.append((codes, scale, zp, rowsum, xhat) + ((ctr,) if ct else ()))
    with torch.cuda.device(x0.device):
        rc = _lib.load().qfa_quant_batch_per_token(jobs, len(tensors), _DT[x0.dtype], _stream(x0))
    _lib.check(rc, "qfa_quant_batch_per_token")
    return results


def asymmetric_quant_per_token(input_tensor: torch.Tensor):
    """Quantizes a (Batch, Num_Heads, Seq_Len, Head_Dim) fp16/bf16 CUDA tensor to INT8, one
    scale and zero-point per token.

    Returns (quantized int8 tensor with the input's shape and strides,
             scale float16 (B,H,S,1), zero_point int8 (B,H,S,1)) -- asymmetric_quant.py:117-121.
    """
    codes, scale, zp, _, _ = _quantize(input_tensor, False, False)
    return codes, scale, zp


def asymmetric_quant_per_token_ex(input_tensor: torch.Tensor, dequant: bool = False):
    """Same quantizer, also returning the per-token sum of the codes (int32, (B,H,S)) that the
    int8 attention needs, and optionally the dequantized tensor (code - zp) * scale in the
    input dtype.  Returns (codes, scale, zero_point, rowsum[, dequantized])."""
    codes, scale, zp, rowsum, xhat = _quantize(input_tensor, True, dequant)
    return (codes, scale, zp, rowsum, xhat) if dequant else (codes, scale, zp, rowsum)


def dequantize_per_token(quantized_tensor, scale, zero_point):
    """(code - zp) * scale in fp32, as the reference's helper (asymmetric_quant.py:158-160)."""
    return (quantized_tensor.to(torch.float32) - zero_point.to(torch.float32)) * scale.to(torch.float32)
