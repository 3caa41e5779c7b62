"""The benchmark configurations at FULL size on the GPU, whole heads of each checked against the CPU oracle
(through the C ABI, like every GPU test).

The oracle cannot evaluate 128 heads of 4096 x 4096 logits in a test, so each configuration runs on the GPU
at its full size and a few complete (batch, head) units are compared: O, LSE, delta, dQ, dK, dV.  Heads are
independent units of the path, so a whole head is a complete sub-problem; the remaining heads are covered by
a cross-check between the tcgen05 kernels and the mma.sync kernels (two implementations of one arithmetic).
The oracle gets the operands exactly as the GPU quantizer produced them (the quantizer has its own bit-exact
tests), is evaluated in row chunks and its result is left un-rounded: exact weights for the forward output,
the kernels' semantics (round_p) for the gradients (see the note at the top of test_gpu_attn.py).
"""
import math

import pytest
import torch

import oracle
from parity_util import HALF_ULP, REL_TOL, close, gen, head_quant

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def qfa():
    import quant_flash_attn_b200 as m
    from quant_flash_attn_b200 import _lib
    _lib.load()
    return m


def _per_head_inputs(B, H, S, D, kind, seed, n=4, dtype=torch.bfloat16):
    """n tensors (B,H,S,D) on the GPU; the heads listed in a test get CPU-seeded data (so the oracle sees the
    same values), the others device-seeded data of the same distribution."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for _ in range(n):
        x = torch.randn(B, H, S, D, device="cuda", dtype=torch.float32, generator=g)
        if kind == "outlier":
            idx = torch.randperm(D, generator=torch.Generator().manual_seed(seed))[: max(1, (D + 99) // 100)]
            x[..., idx.cuda()] *= 20.0
        elif kind == "loguniform":
            mag = torch.empty(B, H, S, 1, device="cuda").uniform_(math.log(0.1), math.log(10.0), generator=g)
            x *= torch.exp(mag)
        out.append(x.to(dtype))
    return out


def _check_heads(qfa, tag, q, k, v, do, causal, heads, fwd_only=False, row_chunk=1024, p_rounding=0.0):
    B, H, S, D = q.shape
    dtype = q.dtype
    sm = 1.0 / math.sqrt(D)
    qq, kq, vq = qfa.quantize_qkv(q, k, v)
    o, lse = qfa.int8_attention_forward(qq, kq, vq, causal, sm, dtype)
    assert torch.isfinite(o).all() and torch.isfinite(lse).all()
    if not fwd_only:
        dq, dk, dv = qfa.int8_attention_backward(qq, kq, vq, causal, sm, o, lse, do)
    for (b, h) in heads:
        sl = (slice(b, b + 1), slice(h, h + 1))
        quant = tuple(head_quant(t, b, h) for t in (qq, kq, vq))
        o_ref, lse_ref, _ = oracle.int8_mode_forward(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), causal, sm, quant=quant,
                                                     round_output=False, row_chunk=row_chunk)
        name = f"{tag} head({b},{h})"
        close(o[sl], o_ref, what=name + " o", p_rounding=p_rounding)
        err = (lse[sl].cpu() - lse_ref).abs().max().item()
        assert err <= 2e-3, f"{name} lse: {err}"
        if fwd_only:
            continue
        dq_ref, dk_ref, dv_ref, delta_ref = oracle.int8_mode_backward(
            quant, causal, sm, o[sl].cpu(), lse[sl].cpu(), do[sl].cpu(), dtype, round_output=False, round_p=dtype,
            row_chunk=row_chunk, return_delta=True)
        close(dq[sl], dq_ref, what=name + " dq", p_rounding=p_rounding)
        close(dk[sl], dk_ref, what=name + " dk", p_rounding=p_rounding)
        close(dv[sl], dv_ref, what=name + " dv", p_rounding=p_rounding)
    return qq, kq, vq, o, lse, (None if fwd_only else (dq, dk, dv))


@pytest.mark.parametrize("causal", [False, True])
def test_config2_headline_B4H32S4096D128(qfa, causal):
    """B4 H32 S4096 D128, bf16 N(0,1) with 1 % of the channels x20: forward AND backward, two whole heads
    against the oracle; all 128 heads of the tcgen05 kernels against the mma.sync kernels."""
    q, k, v, do = _per_head_inputs(4, 32, 4096, 128, "outlier", seed=7)
    do = torch.randn(do.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(8)).to(do.dtype)
    tag = "C2 " + ("causal" if causal else "non-causal")
    # channels scaled x20 put the softmax of most rows on one or two keys, so a single 16-bit rounding of P or dS
    # (or one that falls the other way because kernel and oracle differ in the last fp32 bit) reaches the output
    # undiminished: outputs and gradients of THIS configuration get the extra half ulp of parity_util.close;
    # LSE keeps its plain bound, and every other configuration the plain 2e-3
    qq, kq, vq, o, lse, grads = _check_heads(qfa, tag, q, k, v, do, causal, heads=((0, 0), (3, 17)),
                                             p_rounding=HALF_ULP[torch.bfloat16])
    sm = 1.0 / math.sqrt(128)
    o_mma, lse_mma = qfa.int8_attention_forward(qq, kq, vq[:4], causal, sm, torch.bfloat16)
    assert (lse - lse_mma).abs().max().item() <= 2e-3
    # two implementations that are each within the bound of the oracle may differ by twice the bound
    close(o, o_mma.float(), rel=2 * REL_TOL, what=tag + " o tcgen05 vs mma.sync (128 heads)",
          p_rounding=HALF_ULP[torch.bfloat16])
    grads_mma = qfa.int8_attention_backward(qq, kq, vq, causal, sm, o, lse, do, use_tc=False)
    for name, a, b_ in zip(("dq", "dk", "dv"), grads, grads_mma):
        close(a, b_.float(), rel=2 * REL_TOL, what=f"{tag} {name} tcgen05 vs mma.sync (128 heads)",
              p_rounding=HALF_ULP[torch.bfloat16])


def test_config3_training_B8H16S2048D64_causal(qfa):
    """B8 H16 S2048 D64 causal, bf16 N(0,1): O, LSE, delta, dQ, dK, dV of two whole heads."""
    q, k, v, do = _per_head_inputs(8, 16, 2048, 64, "normal", seed=5)
    _, _, _, o, lse, _ = _check_heads(qfa, "C3", q, k, v, do, True, heads=((0, 0), (5, 11)))
    # delta pre-pass on its own (quant_flash_attn.py:88-101): rowsum(O * dO) in fp32
    import ctypes as C
    from quant_flash_attn_b200 import _lib
    delta = torch.empty(8, 16, 2048, dtype=torch.float32, device="cuda")
    s3 = lambda t: _lib.c_i64x3(t.stride(0), t.stride(1), t.stride(2))
    so, sdo = s3(o), s3(do)
    rc = _lib.load().qfa_attn_bwd_delta(o.data_ptr(), C.byref(so), do.data_ptr(), C.byref(sdo), delta.data_ptr(), 2048,
                                        8, 16, 2048, 64, _lib.QFA_BF16, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    want = (o.float() * do.float()).sum(-1)
    close(delta, want, rel=1e-5, what="C3 delta (all heads)")


def test_config4_long_context_B1H32S32768D128_causal(qfa):
    """B1 H32 S32768 D128 causal, per-token magnitudes log-uniform in [0.1, 10]: forward of all 32 heads on the GPU,
    one whole head (32768 x 32768 logits, evaluated in row chunks) against the oracle."""
    q, k, v = _per_head_inputs(1, 32, 32768, 128, "loguniform", seed=11, n=3)
    _check_heads(qfa, "C4", q, k, v, None, True, heads=((0, 9),), fwd_only=True, row_chunk=1024)


def test_config5_sweep_point_S16384_fwd_bwd(qfa):
    """The sweep's longest point: B2 H16 S16384 D128 causal, forward + backward; one whole head against the oracle."""
    q, k, v, do = _per_head_inputs(2, 16, 16384, 128, "normal", seed=13)
    _check_heads(qfa, "C5 S16384", q, k, v, do, True, heads=((1, 3),), row_chunk=1024)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Sq,Skv,D,causal,kind", [
    (1, 2, 256, 256, 128, False, "outlier"), (2, 2, 384, 384, 64, True, "normal"),
    (1, 2, 300, 300, 128, True, "loguniform"), (1, 2, 77, 333, 64, False, "normal"),
])
def test_int8_mode_mma_sync_backward_vs_oracle(qfa, dtype, B, H, Sq, Skv, D, causal, kind):
    """The general (mma.sync) int8-mode backward, the kernel that accumulates dQ in fp32 scratch memory, against
    the oracle directly (the dispatcher prefers the tcgen05 kernels, so it is reached with use_tc=False)."""
    q, k, v = (gen((B, H, S_, D), dtype, s, kind) for S_, s in ((Sq, 51), (Skv, 52), (Skv, 53)))
    do = gen((B, H, Sq, D), dtype, 54)
    sm = 1.0 / math.sqrt(D)
    qq, kq, vq = qfa.quantize_qkv(q.cuda(), k.cuda(), v.cuda())
    o, lse = qfa.int8_attention_forward(qq, kq, vq[:4], causal, sm, dtype)        # mma.sync forward as well
    dq, dk, dv = qfa.int8_attention_backward(qq, kq, vq, causal, sm, o, lse, do.cuda(), use_tc=False)
    from parity_util import cpu_quant
    quant = tuple(cpu_quant(t) for t in (qq, kq, vq))
    o_ref, lse_ref, _ = oracle.int8_mode_forward(q, k, v, causal, sm, quant=quant, round_output=False)
    tag = f"mma.sync int8 Sq{Sq} Skv{Skv} D{D} {'causal ' if causal else ''}{kind} {dtype}".replace("torch.", "")
    close(o, o_ref, what=tag + " o")
    assert (lse.cpu() - lse_ref).abs().max().item() <= 2e-3
    dq_ref, dk_ref, dv_ref = oracle.int8_mode_backward(quant, causal, sm, o.cpu(), lse.cpu(), do, dtype,
                                                       round_output=False, round_p=dtype)
    close(dq, dq_ref, what=tag + " dq")
    close(dk, dk_ref, what=tag + " dk")
    close(dv, dv_ref, what=tag + " dv")
