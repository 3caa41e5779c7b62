"""CUDA attention kernels (both numeric modes, forward and backward) against the reference
fixtures and the CPU oracle, through the C ABI."""
import glob
import math
import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ATTN_CASES = sorted(glob.glob(os.path.join(HERE, "golden", "a_*.npz")))

from parity_util import HALF_ULP, close as _close, cpu_quant as _cpu_quant, gen as _gen  # noqa: E402

# The bound is 2e-3 of the output scale plus the storage rounding of the result (parity_util.close), for both
# dtypes, outputs and gradients alike; the oracle's result is left un-rounded.
#   Gradients are compared with the oracle evaluated with the kernels' semantics (round_p: P and dS rounded to the
# 16-bit dtype before the gradient products, quant_flash_attn.py:156,159-160): kernel and oracle exponentiate
# against the same reference (the saved LSE), so their roundings coincide.
#   Forward outputs are compared with the oracle's EXACT weights: the forward kernels round P against their own
# running reference (the reference's kernel against its running maximum, quant_flash_attn.py:70-75), the oracle
# would round it against the row maximum, and two roundings of P against different reference points are
# independent noise of the same size: rounding in the oracle too makes the comparison noisier, not tighter.


@pytest.fixture(scope="module")
def qfa():
    import quant_flash_attn_b200 as m
    from quant_flash_attn_b200 import _lib
    _lib.load()
    return m


# ------------------------------------------------------------------ ref mode (the reference's operator)

@pytest.mark.parametrize("path", ATTN_CASES, ids=[os.path.basename(p)[:-4] for p in ATTN_CASES])
def test_ref_mode_vs_reference_fixtures(qfa, path):
    g = np.load(path)
    q = torch.from_numpy(g["q"]).cuda().requires_grad_()
    kv = torch.from_numpy(g["kv"]).cuda().requires_grad_()
    go = torch.from_numpy(g["go"]).cuda()
    sm = float(g["sm_scale"])
    kvq = qfa.asymmetric_quant_per_token(kv.detach())
    # feed the fixture's own codes so that attention is compared on identical quantized inputs
    kvq = (torch.from_numpy(g["codes"]).cuda(), torch.from_numpy(g["scale"]).cuda(), torch.from_numpy(g["zp"]).cuda())
    o = qfa.quant_flash_attn(q, kv, kvq, sm)
    o.backward(go)
    _close(o, torch.from_numpy(g["o"]), what="o")
    _close(q.grad, torch.from_numpy(g["dq"]), what="dq")
    _close(kv.grad, torch.from_numpy(g["dkv"]), what="dkv")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 2, 17, 1023, 128), (2, 3, 18, 512, 64), (1, 2, 97, 689, 128),
                                   (1, 1, 200, 130, 64), (1, 2, 1, 64, 128), (1, 1, 64, 1, 64),
                                   # 17 to 32 query rows (dedicated converter warps, three K/V stages): one, two and
                                   # many K/V tiles, ragged last tile; 33 to 128 rows with exactly two and three tiles
                                   (1, 1, 32, 1, 64), (1, 2, 20, 130, 128), (2, 2, 31, 257, 64), (1, 2, 25, 640, 128),
                                   (1, 2, 128, 256, 128), (1, 1, 33, 384, 64)])
def test_ref_mode_vs_oracle_ragged(qfa, dtype, shape):
    Z, H, NQ, NKV, D = shape
    q = _gen((Z, H, NQ, D), dtype, 1)
    kv = _gen((Z, H, NKV, D), dtype, 2)
    go = _gen((Z, H, NQ, D), dtype, 3)
    sm = 1.0 / math.sqrt(D)
    qc, kvc = q.cuda().requires_grad_(), kv.cuda().requires_grad_()
    kvq = qfa.asymmetric_quant_per_token(kvc.detach())
    o = qfa.quant_flash_attn(qc, kvc, kvq, sm)
    o.backward(go.cuda())
    codes, scale, zp = (t.cpu() for t in kvq)
    o_ref, lse_ref = oracle.ref_mode_forward(q, codes, scale, zp, sm, round_output=False)
    tag = f"ref-mode {shape} {dtype}".replace("torch.", "")
    _close(o, o_ref, what=tag + " o")
    dq_ref, dkv_ref = oracle.ref_mode_backward(q, codes, scale, zp, sm, o.detach().cpu(), lse_ref, go,
                                               round_output=False, round_p=True)
    _close(qc.grad, dq_ref, what=tag + " dq")
    _close(kvc.grad, dkv_ref, what=tag + " dkv")


# the reference's own accuracy test (shapes and tolerances of test_accuracy.py:35-45,115,123,131)
@pytest.mark.parametrize("Z,H,NQ,NKV,D", [(2, 4, 18, 512, 64), (2, 8, 32, 1024, 128), (4, 16, 16, 2048, 64),
                                          (1, 2, 17, 1023, 128), (99, 53, 97, 689, 128)])
def test_reference_accuracy_test_shapes(qfa, Z, H, NQ, NKV, D):
    torch.manual_seed(20)
    dtype, device = torch.float16, "cuda"
    q_ref = torch.randn((Z, H, NQ, D), dtype=dtype, device=device, requires_grad=True)
    kv_ref = torch.randn((Z, H, NKV, D), dtype=dtype, device=device, requires_grad=True)
    q_t = q_ref.clone().detach().requires_grad_(True)
    kv_t = kv_ref.clone().detach().requires_grad_(True)
    sm_scale = 1.0 / (D ** 0.5)
    grad_output = torch.randn_like(q_ref)
    ref_out = torch.nn.functional.scaled_dot_product_attention(q_ref, kv_ref, kv_ref, is_causal=False, scale=sm_scale)
    ref_out.backward(grad_output)
    kv_quant = qfa.asymmetric_quant_per_token(kv_t)
    out = qfa.quant_flash_attn(q_t, kv_t, kv_quant, sm_scale)
    out.backward(grad_output)
    assert torch.allclose(ref_out, out, atol=1e-1, rtol=0)
    assert torch.allclose(q_ref.grad, q_t.grad, atol=1e-2, rtol=0.01)
    assert torch.allclose(kv_ref.grad, kv_t.grad, atol=1e-2, rtol=0.02)


# ------------------------------------------------------------------ int8 mode

INT8_SHAPES = [
    # B, H, Sq, Skv, D, causal, kind
    (1, 4, 512, 512, 64, False, "normal"),          # BASELINE config 1 shape
    (1, 2, 256, 256, 128, False, "outlier"),
    (1, 2, 256, 256, 128, True, "outlier"),
    (2, 2, 384, 384, 64, True, "normal"),
    (1, 2, 300, 300, 128, True, "loguniform"),      # ragged tiles
    (1, 2, 77, 333, 64, False, "normal"),           # Sq != Skv
    (1, 1, 130, 70, 128, True, "normal"),           # causal with Sq > Skv
    (1, 3, 1024, 1024, 128, True, "normal"),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Sq,Skv,D,causal,kind", INT8_SHAPES)
def test_int8_mode_forward_backward_vs_oracle(qfa, dtype, B, H, Sq, Skv, D, causal, kind):
    q = _gen((B, H, Sq, D), dtype, 11, kind)
    k = _gen((B, H, Skv, D), dtype, 12, kind)
    v = _gen((B, H, Skv, D), dtype, 13, kind)
    do = _gen((B, H, Sq, D), dtype, 14)
    sm = 1.0 / math.sqrt(D)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = qfa.quant_attention(qc, kc, vc, causal, sm)
    o.backward(do.cuda())
    # the oracle gets the operands exactly as the GPU quantizer produced them (the quantizer has
    # its own bit-exact tests; CPU division would move ~0.4 % of the codes by one)
    quant = tuple(_cpu_quant(t) for t in qfa.quantize_qkv(qc.detach(), kc.detach(), vc.detach()))
    o_ref, lse_ref, quant = oracle.int8_mode_forward(q, k, v, causal, sm, quant=quant, round_output=False)
    tag = f"int8 B{B} H{H} Sq{Sq} Skv{Skv} D{D} {'causal ' if causal else ''}{kind} {dtype}".replace("torch.", "")
    _close(o, o_ref, what=tag + " o")
    dq_ref, dk_ref, dv_ref = oracle.int8_mode_backward(quant, causal, sm, o.detach().cpu(), lse_ref, do, dtype,
                                                       round_output=False, round_p=dtype)
    _close(qc.grad, dq_ref, what=tag + " dq")
    _close(kc.grad, dk_ref, what=tag + " dk")
    _close(vc.grad, dv_ref, what=tag + " dv")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Hkv,Sq,Skv,D,causal,kind", [
    (1, 2, 2, 1000, 1000, 128, False, "outlier"), (1, 2, 2, 1000, 1000, 128, True, "normal"),
    (1, 2, 2, 700, 700, 64, True, "loguniform"), (2, 4, 2, 300, 517, 128, False, "normal"),
    (1, 1, 1, 77, 1290, 64, False, "outlier"), (1, 2, 1, 130, 70, 128, True, "normal"), (1, 1, 1, 1, 1, 64, False, "normal")])
def test_two_logit_routes_give_the_same_bits(qfa, dtype, B, H, Hkv, Sq, Skv, D, causal, kind):
    """The tcgen05 forward forms sum((q - z_q)(k - z_k)) either with the int8 MMA plus zero-point terms (K tuple
    without the centered codes) or with the 16-bit MMA over centered operands (K tuple as quantize_qkv returns it).
    Both are exact integer arithmetic followed by the same fp32 operations: O and LSE must be bit-identical, also
    with grouped K/V heads, ragged tiles and the causal mask; and both must match the oracle."""
    q = _gen((B, H, Sq, D), dtype, 51, kind)
    k = _gen((B, Hkv, Skv, D), dtype, 52, kind)
    v = _gen((B, Hkv, Skv, D), dtype, 53, kind)
    sm = 1.0 / math.sqrt(D)
    qq, kq, vq = qfa.quantize_qkv(q.cuda(), k.cuda(), v.cuda())
    assert len(kq) == 6 and kq[5].dtype == torch.float16
    o_c, lse_c = qfa.int8_attention_forward(qq, kq, vq, causal, sm, dtype)
    o_i, lse_i = qfa.int8_attention_forward(qq, kq[:5], vq, causal, sm, dtype)
    qfa.check_kernel_status()
    assert torch.equal(o_c, o_i) and torch.equal(lse_c, lse_i)
    if Hkv == H:
        o_ref, lse_ref, _ = oracle.int8_mode_forward(q, k, v, causal, sm, round_output=False,
                                                     quant=tuple(_cpu_quant(t) for t in (qq, kq, vq)))
        _close(o_c, o_ref, what=f"int8 centered route B{B} H{H} Sq{Sq} Skv{Skv} D{D} {kind} {dtype} o".replace("torch.", ""))
        assert (lse_c.cpu() - lse_ref).abs().max() <= 2e-3


def test_int8_mode_lse_and_quantized_operands(qfa):
    B, H, S, D = 1, 2, 320, 128
    q, k, v = (_gen((B, H, S, D), torch.bfloat16, s, "outlier") for s in (21, 22, 23))
    qq, kq, vq = qfa.quantize_qkv(q.cuda(), k.cuda(), v.cuda())
    for causal in (False, True):
        o, lse = qfa.int8_attention_forward(qq, kq, vq, causal, 0.1, torch.bfloat16)
        o_ref, lse_ref, _ = oracle.int8_mode_forward(q, k, v, causal, 0.1, round_output=False,
                                                     quant=tuple(_cpu_quant(t) for t in (qq, kq, vq)))
        assert (lse.cpu() - lse_ref).abs().max() <= 2e-3
        _close(o, o_ref, what=f"int8 lse-case causal={causal} o")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("slope", [0.02, 0.2])
def test_int8_mode_growing_logits(qfa, dtype, causal, slope):
    """Logits that keep growing along the key axis: every 128-key tile exceeds the running maximum of a row
    by tens (slope 0.02) or by more than a hundred powers of two (slope 0.2), so the forward kernel's
    reference has to be raised on every tile: rescale of O, l and the packed P, and (large slope, or fp16
    with either slope) the recompute-from-S branch.  Output and LSE must still match the oracle."""
    B, H, S, D = 1, 2, 1024, 128
    g = torch.Generator().manual_seed(31)
    q = (0.5 + 0.05 * torch.randn((B, H, S, D), generator=g)).to(dtype)
    ramp = (slope * torch.arange(S, dtype=torch.float32)).view(1, 1, S, 1)
    k = ((0.2 + ramp) * (1.0 + 0.1 * torch.randn((B, H, S, D), generator=g))).to(dtype)
    v = torch.randn((B, H, S, D), generator=g).to(dtype)
    sm = 1.0 / math.sqrt(D)
    qq, kq, vq = qfa.quantize_qkv(q.cuda(), k.cuda(), v.cuda())
    o, lse = qfa.int8_attention_forward(qq, kq, vq, causal, sm, dtype)
    o_ref, lse_ref, _ = oracle.int8_mode_forward(q, k, v, causal, sm, round_output=False,
                                                 quant=tuple(_cpu_quant(t) for t in (qq, kq, vq)))
    assert torch.isfinite(lse).all()
    assert ((lse.cpu() - lse_ref).abs() <= 2e-3 + 1e-5 * lse_ref.abs()).all()
    # the rows built here sit on their last few keys: the one case (with outlier channels at the headline size) that
    # gets the extra half ulp of parity_util.close
    _close(o, o_ref, what=f"int8 growing-logits slope {slope} causal={causal} {dtype} o".replace("torch.", ""),
           p_rounding=HALF_ULP[dtype])


@pytest.mark.parametrize("causal", [False, True])
def test_host_pipeline_matches_device_operator(qfa, causal):
    """quant_attention_host (heads sliced over three streams, host tensors in and out) returns exactly what
    quant_attention returns for the same operands; 7 heads over 3 slices leaves a ragged last slice."""
    B, H, S, D = 1, 7, 200, 128
    q, k, v = (_gen((B, H, S, D), torch.bfloat16, s) for s in (41, 42, 43))
    sm = 1.0 / math.sqrt(D)
    want = qfa.quant_attention(q.cuda(), k.cuda(), v.cuda(), causal, sm).cpu()
    got = qfa.quant_attention_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), causal, sm, slices=3)
    assert not got.is_cuda and torch.equal(got, want)
    # a second call reuses the pipeline's buffers
    got2 = qfa.quant_attention_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), causal, sm, slices=3)
    assert torch.equal(got2, want)


@pytest.mark.parametrize("causal", [False, True])
def test_pipelined_front_half_equals_two_calls(qfa, causal):
    """quant_attention_forward (heads cut into slices on side streams, quantizer of a slice overlapping the
    attention of the previous one) returns the bits of quantize_qkv + int8_attention_forward: 11 heads over 4
    slices is ragged; a (B,S,H,D) view and a 3-head problem take the plain route."""
    B, H, S, D = 1, 11, 300, 128
    q, k, v = (_gen((B, H, S, D), torch.bfloat16, s, "outlier").cuda() for s in (61, 62, 63))
    sm = 1.0 / math.sqrt(D)
    o, lse, qq, kq, vq = qfa.quant_attention_forward(q, k, v, causal, sm)
    torch.cuda.synchronize()
    qq2, kq2, vq2 = qfa.quantize_qkv(q, k, v)
    o2, lse2 = qfa.int8_attention_forward(qq2, kq2, vq2, causal, sm, torch.bfloat16)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    for a, b in zip(qq + kq + vq, qq2 + kq2 + vq2):
        assert (a is None and b is None) or (a.shape == b.shape and torch.equal(a, b))
    # twice in a row on the same side streams, then the autograd operator on top of it
    o3 = qfa.quant_attention_forward(q, k, v, causal, sm)[0]
    assert torch.equal(o3, o2)
    assert torch.equal(qfa.quant_attention(q, k, v, causal, sm), o2)
    qt = q.transpose(1, 2).contiguous().transpose(1, 2)            # (B,S,H,D) memory
    assert torch.equal(qfa.quant_attention_forward(qt, k, v, causal, sm)[0], o2)
    assert torch.equal(qfa.quant_attention_forward(q[:, :3], k[:, :3], v[:, :3], causal, sm)[0], o2[:, :3])


def test_training_shape_properties(qfa):
    """BASELINE config 3 (B8 H16 S2048 D64 causal) at full size: the oracle is too slow there, so
    check size-independent properties: finite outputs, row 0 attends only to token 0, gradient
    of a head does not depend on the other heads (partition invariance)."""
    B, H, S, D = 8, 16, 2048, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v, do = (torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(4))
    sm = 1.0 / math.sqrt(D)
    qa, ka, va = (t.clone().requires_grad_() for t in (q, k, v))
    o = qfa.quant_attention(qa, ka, va, True, sm)
    o.backward(do)
    for t in (o, qa.grad, ka.grad, va.grad):
        assert torch.isfinite(t).all()
    # causal row 0 sees only column 0: O[0] = V^[0]
    qq, kq, vq = qfa.quantize_qkv(q, k, v)
    assert torch.equal(o[:, :, 0], vq[4][:, :, 0])
    # one head alone gives the same numbers as inside the batch
    sl = (slice(3, 4), slice(5, 6))
    qb, kb, vb = (t[sl].clone().requires_grad_() for t in (q, k, v))
    ob = qfa.quant_attention(qb, kb, vb, True, sm)
    ob.backward(do[sl])
    assert torch.equal(ob, o[sl])
    assert torch.equal(kb.grad, ka.grad[sl]) and torch.equal(vb.grad, va.grad[sl])
    _close(qb.grad, qa.grad[sl], rel=1e-3, what="dq (atomic order)")


def test_attention_rejects_bad_arguments(qfa):
    q = torch.randn(1, 1, 16, 96, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError):
        qfa.quant_attention(q, q, q, False, 0.1)               # head dim 96
    q = torch.randn(1, 1, 16, 64, device="cuda", dtype=torch.float32)
    with pytest.raises(TypeError):
        qfa.quant_attention(q, q, q, False, 0.1)
    with pytest.raises(RuntimeError):
        qfa.quant_attention(q.cpu().half(), q.cpu().half(), q.cpu().half(), False, 0.1)
