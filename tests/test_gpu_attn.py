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

# north-star tolerance for results that share the kernel's semantics: max-abs error <= 2e-3 of
# the output scale, cosine similarity >= 0.9999.  The kernel's result is STORED in a 16-bit dtype,
# which alone moves an element by up to half an ulp of its own magnitude (2^-8 relative for
# bf16, 2^-11 for fp16); the comparison is against the oracle's un-rounded fp32 result and adds
# exactly that storage term.
# Gradients computed from bf16 operands get twice the bound: the kernels (like the reference,
# quant_flash_attn.py:156,159-160) round P and dS to the input dtype before the gradient
# products, and with 8 significant bits that alone is ~3e-3 of the gradient scale; fp16 meets 2e-3.
REL_TOL = 2e-3
REL_TOL_GRAD = {torch.bfloat16: 4e-3, torch.float16: 2e-3}
COS_TOL = 0.9999
HALF_ULP = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


@pytest.fixture(scope="module")
def qfa():
    import quant_flash_attn_b200 as m
    from quant_flash_attn_b200 import _lib
    _lib.load()
    return m


def _close(got, want, rel=REL_TOL, cos=COS_TOL, what=""):
    storage = HALF_ULP.get(got.dtype, 0.0)
    got, want = got.detach().float().cpu().flatten(), want.detach().float().cpu().flatten()
    assert torch.isfinite(got).all(), what
    scale = want.abs().max().item()
    excess = ((got - want).abs() - storage * want.abs()).max().item()
    c = torch.nn.functional.cosine_similarity(got.double(), want.double(), dim=0).item()
    assert excess <= rel * scale + 1e-5, f"{what}: max-abs excess {excess:.3e} > {rel} * {scale:.3e}"
    if scale > 1e-4:
        assert c >= cos, f"{what}: cosine {c}"


def _cpu_quant(t):
    """GPU quantizer output tuple -> the oracle's (codes, scale fp32, zp, rowsum) on CPU."""
    codes, scale, zp, rowsum = t[:4]
    return (codes.cpu(), scale.float().cpu().squeeze(-1), zp.cpu().squeeze(-1), rowsum.cpu())


def _gen(shape, dtype, seed, kind="normal"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    if kind == "outlier":
        D = shape[-1]
        idx = torch.randperm(D, generator=g)[: max(1, (D + 99) // 100)]
        x[..., idx] *= 20.0
    elif kind == "loguniform":
        x = x * torch.exp(torch.empty(shape[:-1] + (1,)).uniform_(math.log(0.1), math.log(10.0), generator=g))
    return x.to(dtype)


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
                                   (1, 1, 200, 130, 64), (1, 2, 1, 64, 128), (1, 1, 64, 1, 64)])
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
    _close(o, o_ref, what="o")
    dq_ref, dkv_ref = oracle.ref_mode_backward(q, codes, scale, zp, sm, o.detach().cpu(), lse_ref, go,
                                               round_output=False)
    _close(qc.grad, dq_ref, rel=REL_TOL_GRAD[dtype], what="dq")
    _close(kvc.grad, dkv_ref, rel=REL_TOL_GRAD[dtype], what="dkv")


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
    _close(o, o_ref, what="o")
    dq_ref, dk_ref, dv_ref = oracle.int8_mode_backward(quant, causal, sm, o.detach().cpu(), lse_ref, do, dtype,
                                                       round_output=False)
    _close(qc.grad, dq_ref, rel=REL_TOL_GRAD[dtype], what="dq")
    _close(kc.grad, dk_ref, rel=REL_TOL_GRAD[dtype], what="dk")
    _close(vc.grad, dv_ref, rel=REL_TOL_GRAD[dtype], what="dv")


def test_int8_mode_lse_and_quantized_operands(qfa):
    B, H, S, D = 1, 2, 320, 128
    q, k, v = (_gen((B, H, S, D), torch.bfloat16, s, "outlier") for s in (21, 22, 23))
    qq, kq, vq = qfa.quantize_qkv(q.cuda(), k.cuda(), v.cuda())
    for causal in (False, True):
        o, lse = qfa.int8_attention_forward(qq, kq, vq, causal, 0.1, torch.bfloat16)
        o_ref, lse_ref, _ = oracle.int8_mode_forward(q, k, v, causal, 0.1, round_output=False,
                                                     quant=tuple(_cpu_quant(t) for t in (qq, kq, vq)))
        assert (lse.cpu() - lse_ref).abs().max() <= 2e-3
        _close(o, o_ref, what="o")


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
    # a row's weight sits on a handful of keys here, so the rounding of P to the 16-bit dtype before P.V (the
    # reference's own semantics, quant_flash_attn.py:75; the oracle keeps P in fp32) does not average out: allow
    # half an ulp of that dtype on top of the usual bound
    _close(o, o_ref, rel=REL_TOL + HALF_ULP[dtype], what="o")


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


def test_headline_size_cross_checks(qfa):
    """The benchmark's full size (B4 H32 S4096 D128, outlier channels).  The oracle is too slow for 128 heads, so:
    two whole heads against the oracle, and every head of the tcgen05 forward against the mma.sync forward (an
    independent implementation of the same arithmetic, reached by withholding the dequantized V)."""
    B, H, S, D = 4, 32, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(7)
    q, k, v = (torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(3))
    idx = torch.tensor([5, 77], device="cuda")
    for t in (q, k, v):
        t[..., idx] *= 20.0
    sm = 1.0 / math.sqrt(D)
    qq, kq, vq = qfa.quantize_qkv(q, k, v)
    o_tc, lse_tc = qfa.int8_attention_forward(qq, kq, vq, False, sm, torch.bfloat16)
    o_mma, lse_mma = qfa.int8_attention_forward(qq, kq, vq[:4], False, sm, torch.bfloat16)
    assert torch.isfinite(o_tc).all() and torch.isfinite(lse_tc).all()
    assert (lse_tc - lse_mma).abs().max().item() <= 2e-3
    _close(o_tc, o_mma.float(), rel=REL_TOL + HALF_ULP[torch.bfloat16], what="tc vs mma")
    for b, h in ((0, 0), (3, 17)):
        sl = (slice(b, b + 1), slice(h, h + 1))
        quant = tuple(tuple(x[sl].cpu() for x in _cpu_quant_dev(t)) for t in (qq, kq, vq))
        o_ref, lse_ref, _ = oracle.int8_mode_forward(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), False, sm, quant=quant,
                                                     round_output=False)
        assert (lse_tc[sl].cpu() - lse_ref).abs().max().item() <= 2e-3
        # outlier channels make the softmax of many rows sit on a few keys, so the 16-bit rounding of P before P.V
        # (the reference's semantics, quant_flash_attn.py:75; the oracle keeps P in fp32) does not average out:
        # allow half an ulp of the dtype on top of the usual bound, as in test_int8_mode_growing_logits
        _close(o_tc[sl], o_ref, rel=REL_TOL + HALF_ULP[torch.bfloat16], what=f"head ({b},{h})")
    # backward: tcgen05 kernels against the mma.sync kernels on all 128 heads
    do = torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16, generator=g)
    grads_tc = qfa.int8_attention_backward(qq, kq, vq, False, sm, o_tc, lse_tc, do)
    grads_mma = qfa.int8_attention_backward(qq, kq, vq, False, sm, o_tc, lse_tc, do, use_tc=False)
    for name, a, b_ in zip(("dq", "dk", "dv"), grads_tc, grads_mma):
        _close(a, b_.float(), rel=REL_TOL_GRAD[torch.bfloat16], what=name + " tc vs mma")


def _cpu_quant_dev(t):
    """Like _cpu_quant but keeps the tensors on the device and 4-D / 3-D sliceable: (codes, scale, zp, rowsum)."""
    codes, scale, zp, rowsum = t[:4]
    return (codes, scale.float().squeeze(-1), zp.squeeze(-1), rowsum)


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
