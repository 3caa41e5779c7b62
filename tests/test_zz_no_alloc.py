"""qfa_attn_bwd_static_scratch against qfa_attn_bwd, through the C ABI.

The entry point exists for hosts that cannot allocate device memory when they call the library
(a plugin hook that must not allocate, a process whose device memory is all owned by a pool).
Its dQ accumulator is a fixed array inside the library, so the test checks (a) two calls in a row
give the gradients of the allocating entry point, i.e. stale contents of the shared array never
leak into a result, and (b) a problem larger than the array is refused before any launch.
This file sorts last so that a run stopping at the first failure has already run the other tests.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bwd_args(lib_mod, qq, kq, vq, o, lse, delta, do, dq, dk, dv, dq_accum, causal, sm):
    from quant_flash_attn_b200.quant_flash_attn import _quant_tensor, _s3, _DT
    B, H, Sq, D = qq[0].shape
    return lib_mod.QfaBwdArgs(
        mode=lib_mod.QFA_MODE_INT8, dtype=_DT[o.dtype], causal=int(causal), dkv_fused=0, sm_scale=sm,
        B=B, H=H, Sq=Sq, Skv=kq[0].shape[2], D=D, q=None, q_stride=lib_mod.c_i64x3(0, 0, 0),
        qq=_quant_tensor(*qq[:4]), k=_quant_tensor(*kq[:4]), v=_quant_tensor(*vq[:3]),
        d_o=do.data_ptr(), do_stride=_s3(do), lse=lse.data_ptr(), delta=delta.data_ptr(), lse_stride=Sq,
        dq=dq.data_ptr(), dq_stride=_s3(dq), dk=dk.data_ptr(), dk_stride=_s3(dk), dv=dv.data_ptr(), dv_stride=_s3(dv),
        dq_accum=dq_accum.data_ptr() if dq_accum is not None else None, status=None)


def _problem(qfa, B, H, S, D, causal, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v, do = (torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(4))
    sm = 1.0 / math.sqrt(D)
    qq, kq, vq = qfa.quantize_qkv(q, k, v)
    o, lse = qfa.int8_attention_forward(qq, kq, vq, causal, sm, torch.bfloat16)
    return qq, kq, vq, o, lse, do, sm


def test_static_scratch_backward_matches_allocating_backward():
    import quant_flash_attn_b200 as qfa
    from quant_flash_attn_b200 import _lib
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.qfa_static_scratch_capacity() == 4 << 20
    # two different problems back to back: the second must not see the first one's accumulator
    for call, (B, H, S, D, causal) in enumerate([(2, 4, 512, 128, True), (1, 3, 700, 64, False)]):
        qq, kq, vq, o, lse, do, sm = _problem(qfa, B, H, S, D, causal, seed=100 + call)
        delta = (o.float() * do.float()).sum(-1).contiguous()
        # existing entry point (qfa_attn_bwd) on the same kernel: caller-allocated fp32 accumulator
        want = tuple(torch.empty(B, H, S, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        accum = torch.empty(B, H, S, D, device="cuda", dtype=torch.float32)
        args0 = _bwd_args(_lib, qq, kq, vq, o, lse, delta, do, *want, accum, causal, sm)
        _lib.check(lib.qfa_attn_bwd(C.byref(args0), stream), "qfa_attn_bwd")
        dq, dk, dv = (torch.full((B, H, S, D), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(3))
        args = _bwd_args(_lib, qq, kq, vq, o, lse, delta, do, dq, dk, dv, None, causal, sm)
        if call == 1:
            # dq_accum and the dequantized operands are documented as ignored: hand over buffers full of NaN and
            # check that nothing of them reaches the result and that the caller's accumulator stays untouched
            junk = torch.full((B, H, S, D), float("nan"), device="cuda", dtype=torch.float32)
            junk16 = torch.full((B, H, S, D), float("nan"), device="cuda", dtype=torch.bfloat16)
            args.dq_accum = junk.data_ptr()
            args.q_hat = args.k_hat = args.v_hat = junk16.data_ptr()
        _lib.check(lib.qfa_attn_bwd_static_scratch(C.byref(args), stream), "qfa_attn_bwd_static_scratch")
        torch.cuda.synchronize()
        for name, got, ref in (("dq", dq, want[0]), ("dk", dk, want[1]), ("dv", dv, want[2])):
            assert torch.isfinite(got).all(), name
            scale = ref.float().abs().max().item()
            err = (got.float() - ref.float()).abs().max().item()
            # same kernels and inputs; dq is accumulated with atomics, whose order is not fixed,
            # and delta is recomputed here in fp32 torch: allow a bf16 ulp (2^-7) of the scale
            assert err <= 2.0 ** -7 * scale, f"call {call}: {name} differs by {err} (scale {scale})"
        if call == 1:
            assert torch.isnan(junk).all()


def test_static_scratch_rejects_oversized_problem():
    import quant_flash_attn_b200 as qfa
    from quant_flash_attn_b200 import _lib
    lib = _lib.load()
    B, H, S, D = 1, 1, 128, 64
    qq, kq, vq, o, lse, do, sm = _problem(qfa, B, H, S, D, False, seed=7)
    delta = torch.zeros(B, H, S, device="cuda")
    dq, dk, dv = (torch.empty(B, H, S, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    args = _bwd_args(_lib, qq, kq, vq, o, lse, delta, do, dq, dk, dv, None, False, sm)
    args.B = 1 << 20            # claims 2^20 * 128 * 64 floats: far beyond the array
    n0 = lib.qfa_launch_count()
    rc = lib.qfa_attn_bwd_static_scratch(C.byref(args), torch.cuda.current_stream().cuda_stream)
    assert rc == -9 and b"capacity" in lib.qfa_strerror(rc)
    assert lib.qfa_launch_count() == n0
