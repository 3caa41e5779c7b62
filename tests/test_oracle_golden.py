"""The CPU oracle against the fixtures produced by the reference's own kernels
(tests/golden/make_golden.py).  Pins the oracle before it is used to judge CUDA."""
import glob
import os

import numpy as np
import pytest
import torch

import oracle
from oracle.quantizer import quantize_per_token, dequantize_per_token, round_half_away

HERE = os.path.dirname(os.path.abspath(__file__))
QUANT_CASES = sorted(glob.glob(os.path.join(HERE, "golden", "q_*.npz")))
ATTN_CASES = sorted(glob.glob(os.path.join(HERE, "golden", "a_*.npz")))


def test_fixtures_present():
    assert len(QUANT_CASES) >= 7 and len(ATTN_CASES) >= 4


@pytest.mark.parametrize("path", QUANT_CASES, ids=[os.path.basename(p)[:-4] for p in QUANT_CASES])
def test_quantizer_oracle_bit_exact_vs_reference(path):
    g = np.load(path)
    codes, _s32, s16, zp, rowsum = quantize_per_token(g["x"])
    # the interpreter divides with IEEE fp32 like the oracle: equality is exact here
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(s16.view(np.uint16), g["scale"][..., 0].view(np.uint16))
    assert np.array_equal(zp, g["zp"][..., 0])
    assert np.array_equal(rowsum, g["codes"].astype(np.int64).sum(-1))


def test_round_half_away():
    x = np.array([0.5, -0.5, 1.5, 2.5, -2.5, 0.49999997, -0.49999997, 126.5, -128.5, 3.0, 1e9],
                 dtype=np.float32)
    want = np.array([1, -1, 2, 3, -3, 0, 0, 127, -129, 3, 1e9], dtype=np.float32)
    assert np.array_equal(round_half_away(x), want)


def test_quantizer_oracle_edge_rows():
    # constant row -> scale 1 (asymmetric_quant.py:87), zp = clamp(round(-128 - c))
    x = np.full((1, 64), 3.25, np.float32)
    codes, s32, s16, zp, rs = quantize_per_token(x)
    assert s32[0] == 1.0 and zp[0] == -128 and (codes == -125).all() and rs[0] == -125 * 64
    # dequantized error bounded by scale/2 (+ fp16 scale rounding) on random rows
    rng = np.random.default_rng(0)
    x = rng.standard_normal((257, 128)).astype(np.float16).astype(np.float32)
    codes, s32, s16, zp, rs = quantize_per_token(x)
    err = np.abs(dequantize_per_token(codes, s16, zp) - x)
    assert (err <= 0.5 * s32[:, None] * 1.02 + 1e-3 * np.abs(x)).all()
    assert codes.min() == -128 and codes.max() == 127


@pytest.mark.parametrize("path", ATTN_CASES, ids=[os.path.basename(p)[:-4] for p in ATTN_CASES])
def test_ref_mode_oracle_vs_reference(path):
    g = np.load(path)
    q = torch.from_numpy(g["q"])
    go = torch.from_numpy(g["go"])
    codes, scale, zp = (torch.from_numpy(g[k]) for k in ("codes", "scale", "zp"))
    sm = float(g["sm_scale"])
    o, lse = oracle.ref_mode_forward(q, codes, scale, zp, sm)
    o_ref, lse_ref = torch.from_numpy(g["o"]), torch.from_numpy(g["lse"])
    assert (o.float() - o_ref.float()).abs().max() <= 1e-3 * o_ref.float().abs().max() + 1e-3
    assert (lse - lse_ref).abs().max() <= 1e-3
    dq, dkv = oracle.ref_mode_backward(q, codes, scale, zp, sm, o_ref, lse_ref, go)
    for got, want in ((dq, g["dq"]), (dkv, g["dkv"])):
        want = torch.from_numpy(want).float()
        assert (got.float() - want).abs().max() <= 2e-3 * want.abs().max()
    delta = (o_ref.float() * go.float()).sum(-1)
    assert (delta - torch.from_numpy(g["delta"])).abs().max() <= 2e-3


@pytest.mark.parametrize("path", ATTN_CASES, ids=[os.path.basename(p)[:-4] for p in ATTN_CASES])
def test_ref_mode_oracle_with_kernel_semantics_vs_reference(path):
    """round_p: P and dS rounded to the 16-bit dtype before the second products, as the reference's kernels do
    (quant_flash_attn.py:75,156,159-160).  The fixtures come from those kernels, so this evaluation must sit at
    least as close to them as the un-rounded one, and within 1e-3 of the output scale."""
    g = np.load(path)
    q, go = torch.from_numpy(g["q"]), torch.from_numpy(g["go"])
    codes, scale, zp = (torch.from_numpy(g[k]) for k in ("codes", "scale", "zp"))
    sm = float(g["sm_scale"])
    o_ref, lse_ref = torch.from_numpy(g["o"]), torch.from_numpy(g["lse"])

    def rel(a, b):
        b = torch.from_numpy(b).float() if isinstance(b, np.ndarray) else b.float()
        return ((a.float() - b).abs().max() / b.abs().max()).item()

    o, lse = oracle.ref_mode_forward(q, codes, scale, zp, sm, round_output=False, round_p=True)
    dq, dkv = oracle.ref_mode_backward(q, codes, scale, zp, sm, o_ref, lse_ref, go, round_output=False, round_p=True)
    dq0, dkv0 = oracle.ref_mode_backward(q, codes, scale, zp, sm, o_ref, lse_ref, go, round_output=False)
    assert rel(o, o_ref) <= 1e-3 and (lse - lse_ref).abs().max() <= 1e-3
    assert rel(dq, g["dq"]) <= 1e-3 and rel(dkv, g["dkv"]) <= 1e-3
    # the fixtures' own fp16 storage rounding (2^-11) is the floor both evaluations sit on
    assert rel(dq, g["dq"]) <= rel(dq0, g["dq"]) + 2.0 ** -11 and rel(dkv, g["dkv"]) <= rel(dkv0, g["dkv"]) + 2.0 ** -11


def test_int8_mode_round_p_and_row_chunks():
    """int8 mode: row chunks do not change the result; round_p moves it by no more than the 16-bit rounding of the
    weights; the backward's delta equals rowsum(o * do)."""
    torch.manual_seed(3)
    B, H, S, D = 1, 2, 160, 64
    q, k, v, do = (torch.randn(B, H, S, D).bfloat16() for _ in range(4))
    for causal in (False, True):
        o, lse, quant = oracle.int8_mode_forward(q, k, v, causal, 0.125, round_output=False)
        o_c, lse_c, _ = oracle.int8_mode_forward(q, k, v, causal, 0.125, round_output=False, quant=quant, row_chunk=48)
        assert (o - o_c).abs().max() <= 1e-6 and (lse - lse_c).abs().max() <= 1e-6
        o_r, _, _ = oracle.int8_mode_forward(q, k, v, causal, 0.125, round_output=False, quant=quant,
                                             round_p=torch.bfloat16)
        assert 0 < (o - o_r).abs().max() <= 2.0 ** -8 * v.float().abs().max()
        g = oracle.int8_mode_backward(quant, causal, 0.125, o, lse, do, torch.bfloat16, round_output=False)
        g_c = oracle.int8_mode_backward(quant, causal, 0.125, o, lse, do, torch.bfloat16, round_output=False,
                                        row_chunk=48, return_delta=True)
        for a, b in zip(g, g_c[:3]):
            assert (a - b).abs().max() <= 1e-4 * a.abs().max()
        assert (g_c[3] - (o.float() * do.float()).sum(-1)).abs().max() <= 1e-5


def test_int8_identity_matches_dequantized_matmul():
    torch.manual_seed(0)
    q = torch.randn(1, 2, 64, 64).half()
    k = torch.randn(1, 2, 96, 64).half()
    qq, kq = oracle.attention.int8_mode_quantize(q), oracle.attention.int8_mode_quantize(k)
    s = oracle.attention.int8_mode_logits(qq, kq, 0.125, False, torch.float64)
    qh = (qq[0].double() - qq[2].double().unsqueeze(-1)) * qq[1].double().unsqueeze(-1)
    kh = (kq[0].double() - kq[2].double().unsqueeze(-1)) * kq[1].double().unsqueeze(-1)
    want = qh @ kh.transpose(-1, -2) * 0.125
    assert (s - want).abs().max() < 1e-9


def test_int8_mode_backward_matches_autograd():
    torch.manual_seed(1)
    B, H, S, D = 1, 2, 48, 64
    q, k, v = (torch.randn(B, H, S, D).bfloat16() for _ in range(3))
    do = torch.randn(B, H, S, D).bfloat16()
    for causal in (False, True):
        o, lse, quant = oracle.int8_mode_forward(q, k, v, causal, 0.125, torch.float64)
        dq, dk, dv = oracle.int8_mode_backward(quant, causal, 0.125, o, lse, do, torch.float32, torch.float64)
        deq = lambda t: ((t[0].double() - t[2].double().unsqueeze(-1)) * t[1].double().unsqueeze(-1))
        qh, kh = deq(quant[0]).requires_grad_(), deq(quant[1]).requires_grad_()
        vh = deq(quant[2]).bfloat16().double().requires_grad_()
        o2 = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=0.125)
        o2.backward(do.double())
        # o passed to the backward is bf16-rounded, so delta carries ~1e-3 relative noise
        for got, want in ((dq, qh.grad), (dk, kh.grad), (dv, vh.grad)):
            assert (got.double() - want).abs().max() <= 5e-3 * want.abs().max()
        assert (o.double() - o2).abs().max() <= 1e-2 * o2.abs().max()


def test_attention_ops():
    assert oracle.attention_ops(4, 32, 4096, 4096, 128) == 4 * 4 * 32 * 128 * 4096 * 4096
    assert oracle.attention_ops(1, 1, 4, 4, 1, causal=True) == 4 * 10
