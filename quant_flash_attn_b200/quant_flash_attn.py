"""Quantized flash attention operators (host side).

`QuantFlashAttention` / `quant_flash_attn` keep the reference's signature and autograd
contract (quant_flash_attn.py:173-240): `quant_flash_attn(q, kv_fp16, kv_quant, sm_scale)`,
positional only, `kv_fp16` is a gradient placeholder whose values are never read, backward
returns `(dq, dkv, None, None)` with `dkv = dV + sm_scale * dK`.

`QuantAttention` / `quant_attention(q, k, v, causal, sm_scale)` is the int8 x int8 operator
with the signature of flash_attn_triton.py:441: it quantizes q, k and v per token itself and
returns gradients `(dq, dk, dv, None, None)` (flash_attn_triton.py:517).

Both run only on CUDA through libqfa_sm100a.so; tensors are allocated here with torch and
handed to the library as raw pointers.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _lib
from .asymmetric_quant import _DT, _require_cuda, _stream, _quantize, _quantize_batch


def _next_power_of_2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def _s3(t: torch.Tensor):
    return _lib.c_i64x3(t.stride(0), t.stride(1), t.stride(2))


def _rows16(t: torch.Tensor) -> torch.Tensor:
    """Kernels read rows with 16-byte vectors: inner stride 1, other strides multiples of 16 bytes."""
    m = 16 // t.element_size()
    if t.stride(3) != 1 or any(t.stride(i) % m for i in range(3)) or t.data_ptr() % 16:
        return t.contiguous()
    return t


def _flat(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _quant_tensor(codes, scale, zp, rowsum=None) -> _lib.QfaQuantTensor:
    return _lib.QfaQuantTensor(codes.data_ptr(), _s3(codes), scale.data_ptr(), zp.data_ptr(),
                               rowsum.data_ptr() if rowsum is not None else None)


def _check_head_dim(D: int):
    if D not in (64, 128):
        raise ValueError(f"head dimension {D} is not supported (64 or 128)")


def _status_ptr(device) -> int:
    """Address of the device's status word (pinned host memory the GPU writes directly).  Before handing it to
    the next launch, report what an EARLIER launch on this device left there: a kernel whose bounded wait ran
    out returns garbage, and the caller must hear about it even though nobody synchronised for it."""
    _lib.raise_if_kernel_status(device)
    return _lib.status_word(device).data_ptr()


def _after_launch(device):
    # QFA_CHECK_STATUS=1 (debugging aid): synchronise after every attention launch and raise at once
    if os.environ.get("QFA_CHECK_STATUS"):
        _lib.raise_if_kernel_status(device, synchronize=True)


def check_kernel_status(device=None, synchronize: bool = True):
    """Raises RuntimeError if any attention kernel launched so far on `device` (default: the current device)
    reported a status, i.e. a bounded barrier wait inside it ran out and its outputs are invalid.  The operators
    run this check (without synchronising) before each of their launches; call it yourself, with the default
    `synchronize=True`, before trusting the results of the LAST launches of a run."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _lib.raise_if_kernel_status(dev, synchronize=synchronize)


class QuantFlashAttention(torch.autograd.Function):
    """Attention of 16-bit queries against one per-token INT8-quantized tensor used as both K and V."""

    @staticmethod
    def forward(ctx, q, kv_fp16, kv_quant, sm_scale):
        _require_cuda(q, "q")
        Z, H, N_CTX_Q, HEAD_DIM = q.shape
        _, _, N_CTX_KV, _ = kv_fp16.shape                      # only the shape is read (quant_flash_attn.py:181)
        if q.dtype not in _DT:
            raise TypeError(f"q must be float16 or bfloat16, got {q.dtype}")
        _check_head_dim(HEAD_DIM)
        kv_codes, kv_scale, kv_zero_point = kv_quant[:3]
        if kv_codes.shape[2] != N_CTX_KV:
            raise ValueError("kv_fp16 and kv_quant disagree on the KV length")
        PADDED_N_CTX_Q = max(_next_power_of_2(N_CTX_Q), 16)   # LSE layout of quant_flash_attn.py:182,185
        qk = _rows16(q)
        kv_codes_k = _rows16(kv_codes)
        kv_scale_k, kv_zp_k = _flat(kv_scale), _flat(kv_zero_point)
        o = torch.empty_like(qk)
        lse = torch.empty((Z, H, PADDED_N_CTX_Q), device=q.device, dtype=torch.float32)

        kvq = _quant_tensor(kv_codes_k, kv_scale_k, kv_zp_k)
        # more than 128 query rows: the tcgen05 kernel takes the K/V tensor dequantized to 16 bit ((code - zp) * scale
        # rounded to q's dtype, quant_flash_attn.py:65-66) as both of its operands; 17 to 128 rows: one query tile per
        # head, every K/V tile is read once and the kernel dequantizes the codes itself; up to 16 rows the
        # short-query kernels read the int8 codes
        kv_hat = dequantize_16bit(kv_codes_k, kv_scale_k, kv_zp_k, q.dtype) if N_CTX_Q > 128 else None
        args = _lib.QfaFwdArgs(
            mode=_lib.QFA_MODE_REF, dtype=_DT[q.dtype], causal=0, sm_scale=float(sm_scale),
            B=Z, H=H, Sq=N_CTX_Q, Skv=N_CTX_KV, D=HEAD_DIM,
            q=qk.data_ptr(), q_stride=_s3(qk), k=kvq, v=kvq, v_hat=kv_hat.data_ptr() if kv_hat is not None else None,
            o=o.data_ptr(), o_stride=_s3(o), lse=lse.data_ptr(), lse_stride=PADDED_N_CTX_Q,
            status=_status_ptr(q.device))
        with torch.cuda.device(q.device):
            rc = _lib.load().qfa_attn_fwd(C.byref(args), _stream(q))
        _lib.check(rc, "qfa_attn_fwd")
        _after_launch(q.device)

        ctx.save_for_backward(qk, o, lse, kv_codes_k, kv_scale_k, kv_zp_k)
        ctx.sm_scale = sm_scale
        ctx.Z, ctx.H, ctx.N_CTX_Q, ctx.HEAD_DIM = Z, H, N_CTX_Q, HEAD_DIM
        ctx.PADDED_N_CTX_Q = PADDED_N_CTX_Q
        return o

    @staticmethod
    def backward(ctx, grad_output):
        q, o, lse, kv_codes, kv_scale, kv_zero_point = ctx.saved_tensors
        Z, H, N_CTX_Q, HEAD_DIM = ctx.Z, ctx.H, ctx.N_CTX_Q, ctx.HEAD_DIM
        N_CTX_KV = kv_codes.shape[2]
        do = _rows16(grad_output)
        dq = torch.empty_like(q)
        dkv = torch.empty(kv_codes.shape, dtype=q.dtype, device=q.device)
        delta = torch.empty_like(lse)
        dq_accum = torch.empty((Z, H, N_CTX_Q, HEAD_DIM), dtype=torch.float32, device=q.device)
        lib = _lib.load()
        stream = _stream(q)
        with torch.cuda.device(q.device):
            so, sdo = _s3(o), _s3(do)
            rc = lib.qfa_attn_bwd_delta(o.data_ptr(), C.byref(so), do.data_ptr(), C.byref(sdo), delta.data_ptr(),
                                        ctx.PADDED_N_CTX_Q, Z, H, N_CTX_Q, HEAD_DIM, _DT[q.dtype], stream)
            _lib.check(rc, "qfa_attn_bwd_delta")
            kvq = _quant_tensor(kv_codes, kv_scale, kv_zero_point)
            # more than 32 query rows: the tcgen05 kernels, which take the dequantized K/V tensor (rebuilt here
            # rather than kept alive between forward and backward: one launch)
            kv_hat = dequantize_16bit(kv_codes, kv_scale, kv_zero_point, q.dtype) if N_CTX_Q > 32 else None
            args = _lib.QfaBwdArgs(
                mode=_lib.QFA_MODE_REF, dtype=_DT[q.dtype], causal=0, dkv_fused=1, sm_scale=float(ctx.sm_scale),
                B=Z, H=H, Sq=N_CTX_Q, Skv=N_CTX_KV, D=HEAD_DIM,
                q=q.data_ptr(), q_stride=_s3(q), k=kvq, v=kvq,
                d_o=do.data_ptr(), do_stride=sdo, lse=lse.data_ptr(), delta=delta.data_ptr(),
                lse_stride=ctx.PADDED_N_CTX_Q,
                dq=dq.data_ptr(), dq_stride=_s3(dq), dk=dkv.data_ptr(), dk_stride=_s3(dkv),
                dv=None, dv_stride=_lib.c_i64x3(0, 0, 0), dq_accum=dq_accum.data_ptr(),
                status=_status_ptr(q.device), v_hat=kv_hat.data_ptr() if kv_hat is not None else None)
            rc = lib.qfa_attn_bwd(C.byref(args), stream)
        _lib.check(rc, "qfa_attn_bwd")
        _after_launch(q.device)
        return dq, dkv, None, None


quant_flash_attn = QuantFlashAttention.apply


def quantize_qkv(q, k, v):
    """Per-token quantization of the three operands of `quant_attention`.

    Returns three tuples (codes, scale, zp, rowsum, dequantized-or-None); only V carries the
    dequantized 16-bit tensor (the P.V operand, quant_flash_attn.py:65-66).  The K tuple has a sixth element, the
    centered codes (code - zero_point as fp16): with it the forward forms its exact integer logits on the 16-bit
    tensor path; `kq[:5]` selects the int8 MMA instead (same results)."""
    if q.dtype == k.dtype == v.dtype and q.device == k.device == v.device:
        # one launch for the three tensors
        return tuple(_quantize_batch((q, k, v), (False, False, True), want_centered=(False, True, False)))
    kq = _quantize(k, True, False)
    return _quantize(q, True, False), kq + (center_codes(kq[0], kq[2]),), _quantize(v, True, True)


def int8_attention_forward(qq, kq, vq, causal: bool, sm_scale: float, dtype: torch.dtype,
                           o: torch.Tensor | None = None, lse: torch.Tensor | None = None):
    """Forward of the int8 operator on already quantized operands (tuples from `quantize_qkv`).
    Returns (o, lse); lse is (B,H,Sq) fp32 natural-log.  k and v may have fewer heads than q (a divisor of
    H): query head h then reads K/V head h // (H / Hkv)."""
    qc, qs, qz, qsum = qq[:4]
    kc, ks, kz, ksum = kq[:4]
    vc, vs, vz = vq[:3]
    vhat = vq[4] if len(vq) > 4 else None
    kctr = kq[5] if len(kq) > 5 else None        # centered K codes (fp16): selects the 16-bit logits MMA
    B, H, Sq, D = qc.shape
    Hkv, Skv = kc.shape[1], kc.shape[2]
    _check_head_dim(D)
    if H % Hkv != 0 or vc.shape[1] != Hkv:
        raise ValueError("the number of query heads must be a multiple of the number of K/V heads")
    if Hkv != H and vhat is None:
        raise ValueError("grouped K/V heads need the dequantized V from quantize_qkv")
    if o is None:
        o = torch.empty((B, H, Sq, D), dtype=dtype, device=qc.device)
    if lse is None:
        lse = torch.empty((B, H, Sq), dtype=torch.float32, device=qc.device)
    args = _lib.QfaFwdArgs(
        mode=_lib.QFA_MODE_INT8, dtype=_DT[dtype], causal=int(bool(causal)), sm_scale=float(sm_scale),
        B=B, H=H, Sq=Sq, Skv=Skv, D=D, q=None, q_stride=_lib.c_i64x3(0, 0, 0),
        qq=_quant_tensor(qc, qs, qz, qsum), k=_quant_tensor(kc, ks, kz, ksum), v=_quant_tensor(vc, vs, vz),
        v_hat=vhat.data_ptr() if vhat is not None else None,
        o=o.data_ptr(), o_stride=_s3(o), lse=lse.data_ptr(), lse_stride=Sq,
        status=_status_ptr(qc.device), Hkv=Hkv,
        k_ctr=kctr.data_ptr() if (kctr is not None and vhat is not None) else None)
    with torch.cuda.device(qc.device):
        rc = _lib.load().qfa_attn_fwd(C.byref(args), _stream(qc))
    _lib.check(rc, "qfa_attn_fwd")
    _after_launch(qc.device)
    return o, lse


_side_streams = {}


def _streams_for(device, n: int):
    """`n` side streams of `device`, created once."""
    key = torch.device(device).index
    have = _side_streams.setdefault(key, [])
    with torch.cuda.device(device):
        while len(have) < n:
            have.append(torch.cuda.Stream())
    return have[:n]


def quant_attention_forward(q, k, v, causal: bool, sm_scale: float, chunks: int = 4):
    """Front half of the int8 operator: quantize q, k, v per token and run the forward.  Returns
    (o, lse, qq, kq, vq) with qq, kq, vq as from `quantize_qkv`.

    Heads are independent units of the path, so the flattened (batch x head) axis is cut into `chunks` slices that
    run on side streams: the quantizer of slice c+1 (bound by HBM) overlaps the attention of slice c (bound by
    the SMs), and the attention launches of all slices queue up behind each other like one launch.  What stays
    exposed of the quantizer is its first slice.  Every output is allocated up front on the caller's stream, the
    side streams only fill slices of it, and the caller's stream waits for them before this function returns.
    Results are bit-identical to `quantize_qkv` followed by `int8_attention_forward`.  Operands that are not
    contiguous (B,H,S,D) tensors of one dtype, or too few heads, take that plain two-call route."""
    from .sharding import shard_bounds
    B, H, Sq, D = q.shape
    Skv = k.shape[2]
    n = B * H
    plain = (chunks <= 1 or n < 2 * chunks or k.shape[:2] != (B, H) or v.shape != k.shape
             or not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous())
             or not (q.dtype == k.dtype == v.dtype) or not (q.device == k.device == v.device))
    if plain:
        qq, kq, vq = quantize_qkv(q, k, v)
        o, lse = int8_attention_forward(qq, kq, vq, causal, sm_scale, q.dtype, o=torch.empty_like(q))
        return o, lse, qq, kq, vq
    _check_head_dim(D)
    dev, dt = q.device, q.dtype

    def alloc(S_, dequant, centered=False):
        return (torch.empty((B, H, S_, D), dtype=torch.int8, device=dev),
                torch.empty((B, H, S_, 1), dtype=torch.float16, device=dev),
                torch.empty((B, H, S_, 1), dtype=torch.int8, device=dev),
                torch.empty((B, H, S_), dtype=torch.int32, device=dev),
                torch.empty((B, H, S_, D), dtype=dt, device=dev) if dequant else None) + \
               ((torch.empty((B, H, S_, D), dtype=torch.float16, device=dev),) if centered else ())

    qq, kq, vq = alloc(Sq, False), alloc(Skv, False, True), alloc(Skv, True)
    o = torch.empty_like(q)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=dev)
    flat = lambda t: None if t is None else t.view(1, n, *t.shape[2:])
    xf = [flat(t) for t in (q, k, v)]
    qf, kf, vf = ([flat(t) for t in tup] for tup in (qq, kq, vq))
    of, lf = flat(o), flat(lse)
    main = torch.cuda.current_stream(dev)
    fork = torch.cuda.Event()
    fork.record(main)
    for c, side in enumerate(_streams_for(dev, chunks)):
        a, b = shard_bounds(n, chunks, c)
        cut = lambda tup: tuple(None if t is None else t[:, a:b] for t in tup)
        side.wait_event(fork)
        with torch.cuda.stream(side):
            outs = [cut(qf), cut(kf), cut(vf)]
            _quantize_batch([t[:, a:b] for t in xf], (False, False, True), outs=outs, want_centered=(False, True, False))
            int8_attention_forward(outs[0], outs[1], outs[2], causal, sm_scale, dt, o=of[:, a:b], lse=lf[:, a:b])
            done = torch.cuda.Event()
            done.record(side)
        main.wait_event(done)
    return o, lse, qq, kq, vq


def center_codes(codes, zp) -> torch.Tensor:
    """code - zero_point as a contiguous fp16 (B,H,S,D) tensor (exact: the difference lies in [-255, 255]): the K
    operand of the forward's 16-bit logits MMA.  No counterpart in the reference."""
    B, H, S, D = codes.shape
    out = torch.empty((B, H, S, D), dtype=torch.float16, device=codes.device)
    if codes.stride(3) != 1:
        raise ValueError("codes must have unit stride along the head dimension")
    with torch.cuda.device(codes.device):
        rc = _lib.load().qfa_center_per_token(codes.data_ptr(), zp.contiguous().data_ptr(), out.data_ptr(), B, H, S, D,
                                              codes.stride(0), codes.stride(1), codes.stride(2), _stream(codes))
    _lib.check(rc, "qfa_center_per_token")
    return out


def dequantize_16bit(codes, scale, zp, dtype: torch.dtype) -> torch.Tensor:
    """(code - zp) * scale rounded to `dtype` as a contiguous (B,H,S,D) tensor (quant_flash_attn.py:65-66)."""
    B, H, S, D = codes.shape
    codes = _rows16(codes)
    out = torch.empty((B, H, S, D), dtype=dtype, device=codes.device)
    with torch.cuda.device(codes.device):
        rc = _lib.load().qfa_dequant_per_token(codes.data_ptr(), _flat(scale).data_ptr(), _flat(zp).data_ptr(),
                                               out.data_ptr(), B, H, S, D, codes.stride(0), codes.stride(1),
                                               codes.stride(2), _DT[dtype], _stream(codes))
    _lib.check(rc, "qfa_dequant_per_token")
    return out


def int8_attention_backward(qq, kq, vq, causal, sm_scale, o, lse, do, use_tc: bool | None = None):
    """Backward of the int8 operator; returns (dq, dk, dv) in o's dtype.  `use_tc=False` withholds the
    dequantized operands, which sends the call to the general (mma.sync) kernels: two independent
    implementations of the same arithmetic, used to cross-check each other at sizes the oracle cannot reach."""
    qc, qs, qz, qsum = qq[:4]
    kc, ks, kz, ksum = kq[:4]
    vc, vs, vz = vq[:3]
    B, H, Sq, D = qc.shape
    Skv = kc.shape[2]
    dev, dtype = qc.device, o.dtype
    do = _rows16(do)
    dq = torch.empty((B, H, Sq, D), dtype=dtype, device=dev)
    dk = torch.empty((B, H, Skv, D), dtype=dtype, device=dev)
    dv = torch.empty((B, H, Skv, D), dtype=dtype, device=dev)
    delta = torch.empty((B, H, Sq), dtype=torch.float32, device=dev)
    # the tcgen05 kernels take the dequantized operands as 16-bit tensors and need no dQ scratch; the
    # general kernel (non-positive sm_scale) accumulates dQ in fp32 scratch instead
    use_tc = float(sm_scale) > 0.0 and (use_tc is None or bool(use_tc))
    q_hat = k_hat = v_hat = dq_accum = None
    if use_tc:
        q_hat = dequantize_16bit(qc, qs, qz, dtype)
        k_hat = dequantize_16bit(kc, ks, kz, dtype)
        v_hat = vq[4] if len(vq) > 4 and vq[4] is not None else dequantize_16bit(vc, vs, vz, dtype)
    else:
        dq_accum = torch.empty((B, H, Sq, D), dtype=torch.float32, device=dev)
    lib = _lib.load()
    stream = _stream(qc)
    with torch.cuda.device(dev):
        so, sdo = _s3(o), _s3(do)
        rc = lib.qfa_attn_bwd_delta(o.data_ptr(), C.byref(so), do.data_ptr(), C.byref(sdo), delta.data_ptr(),
                                    Sq, B, H, Sq, D, _DT[dtype], stream)
        _lib.check(rc, "qfa_attn_bwd_delta")
        args = _lib.QfaBwdArgs(
            mode=_lib.QFA_MODE_INT8, dtype=_DT[dtype], causal=int(bool(causal)), dkv_fused=0,
            sm_scale=float(sm_scale), B=B, H=H, Sq=Sq, Skv=Skv, D=D, q=None, q_stride=_lib.c_i64x3(0, 0, 0),
            qq=_quant_tensor(qc, qs, qz, qsum), k=_quant_tensor(kc, ks, kz, ksum), v=_quant_tensor(vc, vs, vz),
            d_o=do.data_ptr(), do_stride=sdo, lse=lse.data_ptr(), delta=delta.data_ptr(), lse_stride=Sq,
            dq=dq.data_ptr(), dq_stride=_s3(dq), dk=dk.data_ptr(), dk_stride=_s3(dk),
            dv=dv.data_ptr(), dv_stride=_s3(dv),
            dq_accum=dq_accum.data_ptr() if dq_accum is not None else None,
            status=_status_ptr(dev),
            q_hat=q_hat.data_ptr() if use_tc else None, k_hat=k_hat.data_ptr() if use_tc else None,
            v_hat=v_hat.data_ptr() if use_tc else None)
        rc = lib.qfa_attn_bwd(C.byref(args), stream)
    _lib.check(rc, "qfa_attn_bwd")
    _after_launch(dev)
    return dq, dk, dv


class QuantAttention(torch.autograd.Function):
    """softmax(Q^ K^^T * sm_scale [causal]) V^ with Q, K, V quantized per token to INT8; the logits
    come from an int8 x int8 tensor-core product plus zero-point corrections."""

    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale):
        for name, t in (("q", q), ("k", k), ("v", v)):
            _require_cuda(t, name)
            if t.dtype != q.dtype or t.dtype not in _DT:
                raise TypeError("q, k, v must share dtype float16 or bfloat16")
        if k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
            raise ValueError("expected q (B,H,Sq,D) and k, v (B,H,Skv,D)")
        # the output takes q's memory layout (the kernels write through strides), so a (B,S,H,D) caller that
        # passes transposed views gets its result in (B,S,H,D) memory without a copy
        o, lse, qq, kq, vq = quant_attention_forward(q, k, v, causal, sm_scale)
        ctx.save_for_backward(o, lse, *qq[:4], *kq[:4], *vq[:3], vq[4])
        ctx.causal, ctx.sm_scale = bool(causal), float(sm_scale)
        return o

    @staticmethod
    def backward(ctx, grad_output):
        t = ctx.saved_tensors
        o, lse = t[0], t[1]
        qq, kq, vq = t[2:6], t[6:10], (t[10], t[11], t[12], None, t[13])
        dq, dk, dv = int8_attention_backward(qq, kq, vq, ctx.causal, ctx.sm_scale, o, lse, grad_output)
        return dq, dk, dv, None, None


quant_attention = QuantAttention.apply


class HostAttentionPipeline:
    """Inference-time int8 attention for operands that live in HOST memory.

    Heads are independent units of the path, so the (batch x head) axis is cut into slices that move through
    three CUDA streams: while slice i is quantized and attended to, slice i+1 is on its way to the device and
    the output of slice i-1 on its way back.  The host <-> device link carries 3 input bytes for every output
    byte, so with the copies overlapped a call costs about as much as the input copy alone.

    Device buffers for two slices in flight are allocated once per (shape, dtype) and reused.  Host tensors
    should be pinned; pageable memory works but the copies then serialize on the host.
    """

    def __init__(self, device=None, slices: int = 16):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.slices = int(slices)
        with torch.cuda.device(self.device):
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream() for _ in range(3))
        self._key = None
        self._bufs = None

    def _buffers(self, heads, Sq, Skv, D, dtype):
        key = (heads, Sq, Skv, D, dtype)
        if key != self._key:
            mk = lambda S: torch.empty((1, heads, S, D), dtype=dtype, device=self.device)
            self._bufs = [(mk(Sq), mk(Skv), mk(Skv)) for _ in range(2)]
            self._key = key
        return self._bufs

    def __call__(self, q, k, v, causal=False, sm_scale=None, out=None):
        """q (B,H,Sq,D), k, v (B,H,Skv,D): contiguous host tensors, fp16 or bf16.  Returns `out` (host, pinned
        if it is allocated here) after everything has landed in it."""
        for name, t in (("q", q), ("k", k), ("v", v)):
            if t.is_cuda or not t.is_contiguous() or t.dim() != 4 or t.dtype != q.dtype or t.dtype not in _DT:
                raise ValueError(f"{name}: expected a contiguous 4-D host tensor, float16 or bfloat16")
        B, H, Sq, D = q.shape
        Skv = k.shape[2]
        if k.shape != v.shape or k.shape[:2] != (B, H) or k.shape[3] != D:
            raise ValueError("expected q (B,H,Sq,D) and k, v (B,H,Skv,D)")
        _check_head_dim(D)
        sm_scale = 1.0 / (D ** 0.5) if sm_scale is None else float(sm_scale)
        if out is None:
            out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        n = B * H
        per = -(-n // max(1, min(self.slices, n)))
        qf, kf, vf, of = (t.view(1, n, t.shape[2], D) for t in (q, k, v, out))
        bufs = self._buffers(per, Sq, Skv, D, q.dtype)
        free = [None, None]          # event after which a buffer set may be overwritten
        keep = []
        with torch.cuda.device(self.device):
            start = torch.cuda.Event()
            start.record(torch.cuda.current_stream())
            for s_ in (self.s_in, self.s_run, self.s_out):
                s_.wait_event(start)
            for i, h0 in enumerate(range(0, n, per)):
                h1 = min(n, h0 + per)
                dq, dk, dv = (b[:, : h1 - h0] for b in bufs[i & 1])
                if free[i & 1] is not None:
                    self.s_in.wait_event(free[i & 1])
                with torch.cuda.stream(self.s_in):
                    dq.copy_(qf[:, h0:h1], non_blocking=True)
                    dk.copy_(kf[:, h0:h1], non_blocking=True)
                    dv.copy_(vf[:, h0:h1], non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(self.s_in)
                self.s_run.wait_event(landed)
                with torch.cuda.stream(self.s_run):
                    qq, kq, vq = quantize_qkv(dq, dk, dv)
                    o, _ = int8_attention_forward(qq, kq, vq, causal, sm_scale, q.dtype)
                    done = torch.cuda.Event()
                    done.record(self.s_run)
                free[i & 1] = done
                self.s_out.wait_event(done)
                with torch.cuda.stream(self.s_out):
                    of[:, h0:h1].copy_(o, non_blocking=True)
                o.record_stream(self.s_out)
                keep.append((qq, kq, vq, o))
            finish = torch.cuda.Event()
            finish.record(self.s_out)
            torch.cuda.current_stream().wait_event(finish)
            finish.synchronize()
        return out


_host_pipelines = {}


def quant_attention_host(q, k, v, causal=False, sm_scale=None, out=None, device=None, slices: int = 16):
    """`quant_attention` (forward only) for host-resident q, k, v; see HostAttentionPipeline."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev, int(slices))
    if key not in _host_pipelines:
        _host_pipelines[key] = HostAttentionPipeline(dev, slices)
    return _host_pipelines[key](q, k, v, causal, sm_scale, out)

