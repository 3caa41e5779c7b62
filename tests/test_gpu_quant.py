"""CUDA quantizer against the golden fixtures and the CPU oracle (through the C ABI)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle.quantizer import quantize_per_token

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
QUANT_CASES = sorted(glob.glob(os.path.join(HERE, "golden", "q_*.npz")))
GPU_CASES = sorted(glob.glob(os.path.join(HERE, "golden", "gpuref_q_*.npz")))


@pytest.fixture(scope="module")
def qfa():
    import quant_flash_attn_b200 as m
    from quant_flash_attn_b200 import _lib
    _lib.load()
    return m


def _compare_with_ieee_oracle(x_cpu_f32, codes, scale, zp, rowsum=None):
    """CPU oracle divides with IEEE fp32, the GPU with div.full.f32: exact .5 ties of
    x/scale+zp (frequent for short-mantissa inputs) can land on either side.  Allow one code
    (two where the zero-point moved too) on <= 2 % of the elements; exact equality is gated by
    the GPU-written reference fixtures instead."""
    oc, _s32, os16, ozp, orow = quantize_per_token(x_cpu_f32)
    codes, zp = codes.cpu().numpy(), zp.cpu().numpy().reshape(ozp.shape)
    scale_bits = scale.cpu().numpy().reshape(os16.shape).view(np.uint16).astype(np.int32)
    d = np.abs(codes.astype(np.int32) - oc.astype(np.int32))
    dz = np.abs(zp.astype(np.int32) - ozp.astype(np.int32))
    assert dz.max() <= 1 and (dz != 0).mean() <= 1e-2 + 2.0 / dz.size
    assert (d <= 1 + dz[..., None]).all()
    assert (d != 0).mean() <= 2e-2 + 4.0 / d.size
    ds = np.abs(scale_bits - os16.view(np.uint16).astype(np.int32))
    assert ds.max() <= 1 and (ds != 0).mean() <= 1e-2 + 2.0 / ds.size
    if rowsum is not None:
        assert np.array_equal(rowsum.cpu().numpy(), codes.astype(np.int64).sum(-1))
    return int((d != 0).sum()), int((dz != 0).sum()), int((ds != 0).sum())


@pytest.mark.parametrize("path", QUANT_CASES, ids=[os.path.basename(p)[:-4] for p in QUANT_CASES])
def test_quantizer_vs_reference_fixtures(qfa, path):
    g = np.load(path)
    # rebuild the fixture's strided view (one case is (B,S,H,D) data seen as (B,H,S,D))
    base = torch.empty(g["x"].size, dtype=torch.float16, device="cuda")
    x = torch.as_strided(base, tuple(g["x"].shape), [int(s) for s in g["x_stride"]])
    x.copy_(torch.from_numpy(g["x"]).cuda())
    codes, scale, zp, rowsum = qfa.asymmetric_quant_per_token_ex(x)
    assert codes.stride() == x.stride()
    assert scale.shape == (*x.shape[:3], 1) and scale.dtype == torch.float16 and zp.dtype == torch.int8
    # the fixtures come from the reference kernels run with IEEE division (CPU interpreter)
    dc = (codes.cpu().numpy().astype(np.int32) - g["codes"].astype(np.int32))
    assert np.abs(dc).max() <= 2 and (dc != 0).mean() <= 2e-2
    assert np.abs(zp.cpu().numpy().astype(np.int32) - g["zp"].astype(np.int32)).max() <= 1
    assert np.abs(scale.cpu().numpy().view(np.uint16).astype(np.int32) -
                  g["scale"].view(np.uint16).astype(np.int32)).max() <= 1
    assert np.array_equal(rowsum.cpu().numpy(), codes.cpu().numpy().astype(np.int64).sum(-1))


@pytest.mark.parametrize("path", GPU_CASES, ids=[os.path.basename(p)[:-4] for p in GPU_CASES])
def test_quantizer_bit_exact_vs_reference_on_gpu(qfa, path):
    """Fixtures written by the reference's Triton kernel on a B200: equality must be exact."""
    g = np.load(path)
    dt = torch.bfloat16 if str(g["dtype"]) == "bfloat16" else torch.float16
    x = torch.from_numpy(g["x_bits"]).cuda().view(dt)
    codes, scale, zp = qfa.asymmetric_quant_per_token(x)
    assert np.array_equal(codes.cpu().numpy(), g["codes"])
    assert np.array_equal(scale.cpu().numpy().view(np.uint16), g["scale"].view(np.uint16))
    assert np.array_equal(zp.cpu().numpy(), g["zp"])


def _inputs(kind, shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    if kind == "outlier":
        D = shape[-1]
        idx = torch.randperm(D, generator=g)[: max(1, (D + 99) // 100)]
        x[..., idx] *= 20.0
    elif kind == "loguniform":
        mag = torch.exp(torch.empty(shape[:-1] + (1,)).uniform_(np.log(0.1), np.log(10.0), generator=g))
        x = x * mag
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind,shape", [
    ("normal", (1, 4, 512, 64)), ("normal", (2, 8, 1023, 128)), ("outlier", (2, 3, 257, 128)),
    ("loguniform", (1, 2, 999, 128)), ("normal", (1, 1, 1, 64)), ("normal", (3, 2, 65, 256)),
    ("normal", (1, 2, 33, 8)), ("normal", (2, 2, 40, 32)), ("normal", (1, 3, 50, 96)),
    ("normal", (1, 2, 31, 40)), ("normal", (1, 1, 7, 1)),
])
def test_quantizer_vs_oracle(qfa, dtype, kind, shape):
    x = _inputs(kind, shape, dtype, seed=sum(shape) + len(kind))
    codes, scale, zp, rowsum, xhat = qfa.asymmetric_quant_per_token_ex(x.cuda(), dequant=True)
    _compare_with_ieee_oracle(x.float().numpy(), codes, scale, zp, rowsum)
    want = ((codes.float() - zp.float()) * scale.float()).to(dtype)
    assert torch.equal(xhat, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quantizer_strided_inputs(qfa, dtype):
    # (B,S,H,D)-contiguous data viewed as (B,H,S,D) -- codes must inherit the strides
    base = _inputs("normal", (2, 37, 5, 128), dtype, 3).cuda()
    x = base.transpose(1, 2)
    codes, scale, zp = qfa.asymmetric_quant_per_token(x)
    assert codes.stride() == x.stride()
    c2, s2, z2 = qfa.asymmetric_quant_per_token(x.contiguous())
    assert torch.equal(codes, c2) and torch.equal(scale, s2) and torch.equal(zp, z2)
    # inner stride != 1 goes through the general kernel
    y = _inputs("normal", (1, 2, 19, 128), dtype, 4).cuda()[..., ::2]
    c3, s3, z3 = qfa.asymmetric_quant_per_token(y)
    c4, s4, z4 = qfa.asymmetric_quant_per_token(y.contiguous())
    assert torch.equal(c3, c4) and torch.equal(s3, s4) and torch.equal(z3, z4)


def test_quantizer_edge_rows(qfa):
    D = 128
    rows = torch.stack([
        torch.zeros(D), torch.full((D,), -7.5), torch.linspace(0, 255, D), torch.linspace(-127.5, 127.5, D),
        torch.cat([torch.full((D - 1,), float("nan")), torch.tensor([1.0])]),
        torch.cat([torch.ones(D - 1), torch.tensor([float("inf")])]),
    ]).to(torch.bfloat16)[None, None].cuda()
    codes, scale, zp, rowsum = qfa.asymmetric_quant_per_token_ex(rows)
    torch.cuda.synchronize()
    assert scale[0, 0, 0, 0] == 1.0 and zp[0, 0, 0, 0] == -128 and (codes[0, 0, 0] == -128).all()
    assert scale[0, 0, 1, 0] == 1.0 and (codes[0, 0, 1] == -128).all()      # -128 + 7.5 - 7.5 -> clamp
    oc, _, os16, ozp, _ = quantize_per_token(rows[0, 0, :4].float().cpu().numpy())
    assert np.abs(codes[0, 0, :4].cpu().numpy().astype(np.int32) - oc).max() <= 1
    # NaN elements encode as 127 (min/max drop the NaN operand), inf rows stay finite codes
    assert (codes[0, 0, 4, :-1] == 127).all()
    assert np.array_equal(rowsum.cpu().numpy(), codes.cpu().numpy().astype(np.int64).sum(-1))


def test_quantizer_is_idempotent_on_its_own_output(qfa):
    """Size-independent property at a full benchmark size: quantizing the dequantized tensor
    reproduces codes whose dequantization is (nearly) a fixed point, and row sums match."""
    x = torch.randn(4, 32, 4096, 128, device="cuda", dtype=torch.bfloat16)
    codes, scale, zp, rowsum = qfa.asymmetric_quant_per_token_ex(x)
    assert int(codes.min()) == -128 and int(codes.max()) == 127
    assert torch.equal(rowsum, codes.sum(-1, dtype=torch.int32))
    xh = (codes.float() - zp.float()) * scale.float()
    err = (xh - x.float()).abs()
    assert bool((err <= 0.51 * scale.float() + 0.01 * x.float().abs()).all())


def test_quantizer_above_2_31_elements(qfa):
    """The reference's own large case, (512, 32, 2041, 128) = 4.28e9 elements (asymmetric_quant.py:163-188; its
    kernel needs 64-bit offsets, asymmetric_quant.py:55-61).  Checked at full size: three windows of rows (the
    first, the one around element offset 2^31, the last) against the oracle in the documented band; the same
    windows bit for bit against a separate launch on just that slice (small offsets); code sums and the
    dequantization bound on every row."""
    Z, H, M, D = 512, 32, 2041, 128
    x = torch.empty(Z, H, M, D, device="cuda", dtype=torch.bfloat16)
    g = torch.Generator(device="cuda").manual_seed(17)
    for z in range(0, Z, 64):
        x[z:z + 64].normal_(generator=g)
    assert x.numel() > 2 ** 31
    codes, scale, zp, rowsum = qfa.asymmetric_quant_per_token_ex(x)
    rows_per_z = H * M
    z_mid = (2 ** 31 // D) // rows_per_z            # the batch index whose rows straddle element offset 2^31
    for z in (0, z_mid, Z - 1):
        c2, s2, z2, r2 = qfa.asymmetric_quant_per_token_ex(x[z:z + 1])
        assert torch.equal(codes[z:z + 1], c2) and torch.equal(scale[z:z + 1], s2)
        assert torch.equal(zp[z:z + 1], z2) and torch.equal(rowsum[z:z + 1], r2)
        sl = (slice(z, z + 1), slice(0, 2))         # 2 heads x 2041 rows per window for the CPU oracle
        _compare_with_ieee_oracle(x[sl].float().cpu().numpy(), codes[sl], scale[sl], zp[sl], rowsum[sl])
    for z in range(0, Z, 32):
        sl = slice(z, z + 32)
        c = codes[sl]
        assert torch.equal(rowsum[sl], c.sum(-1, dtype=torch.int32))
        sc, xf = scale[sl].float(), x[sl].float()
        err = ((c.float() - zp[sl].float()) * sc - xf).abs()
        assert bool((err <= 0.51 * sc + 0.01 * xf.abs()).all())
        del c, sc, xf, err


def test_batched_quantizer_equals_separate_calls(qfa):
    """qfa_quant_batch_per_token (Q, K, V in one launch; V also dequantized) against three separate calls: same bits.
    Covers the one-launch path (same head dim, aligned), ragged token counts, a transposed view, and the fallback
    (different head dims -> one launch per job)."""
    from quant_flash_attn_b200 import _lib
    from quant_flash_attn_b200.asymmetric_quant import _quantize, _quantize_batch
    for dtype in (torch.bfloat16, torch.float16):
        q = _inputs("outlier", (2, 3, 301, 128), dtype, 1).cuda()
        k = _inputs("normal", (2, 3, 77, 128), dtype, 2).cuda()
        v = _inputs("loguniform", (2, 77, 3, 128), dtype, 3).cuda().transpose(1, 2)      # (B,S,H,D) memory
        n0 = _lib.launch_count()
        got = _quantize_batch((q, k, v), (False, False, True))
        assert _lib.launch_count() - n0 == 1
        want = (_quantize(q, True, False), _quantize(k, True, False), _quantize(v, True, True))
        for g, w in zip(got, want):
            assert g[0].stride() == w[0].stride()
            for a, b in zip(g, w):
                assert (a is None and b is None) or torch.equal(a, b)
        # different head dims: falls back to one launch per job, still the same bits
        k64 = _inputs("normal", (2, 3, 77, 64), dtype, 4).cuda()
        n0 = _lib.launch_count()
        got = _quantize_batch((q, k64), (True, False))
        assert _lib.launch_count() - n0 == 2
        for g, w in zip(got, (_quantize(q, True, True), _quantize(k64, True, False))):
            for a, b in zip(g, w):
                assert (a is None and b is None) or torch.equal(a, b)
    lib = _lib.load()
    assert lib.qfa_quant_batch_per_token(None, 1, 1, None) == -1
    jobs = (_lib.QfaQuantJob * 5)()
    assert lib.qfa_quant_batch_per_token(jobs, 5, 1, None) == -3
    assert lib.qfa_quant_batch_per_token(jobs, 1, 9, None) == -2


def test_centered_codes_are_exact(qfa):
    """The centered output (code - zero_point as fp16) of the batched quantizer -- fused into the one-launch path,
    a second launch in the per-job fallback -- and of the standalone qfa_center_per_token all equal the integer
    difference exactly, together with a dequantized output of the same job and for a (B,S,H,D) view."""
    from quant_flash_attn_b200 import _lib
    from quant_flash_attn_b200.asymmetric_quant import _quantize, _quantize_batch
    from quant_flash_attn_b200.quant_flash_attn import center_codes
    for dtype in (torch.bfloat16, torch.float16):
        q = _inputs("outlier", (2, 3, 301, 128), dtype, 1).cuda()
        k = _inputs("loguniform", (2, 77, 3, 128), dtype, 2).cuda().transpose(1, 2)
        n0 = _lib.launch_count()
        got = _quantize_batch((q, k, q), (False, False, True), want_centered=(False, True, True))
        assert _lib.launch_count() - n0 == 1
        assert len(got[0]) == 5 and len(got[1]) == 6 and len(got[2]) == 6
        for g, x, dq in ((got[1], k, False), (got[2], q, True)):
            w = _quantize(x, True, dq)
            for a, b in zip(g[:5], w):
                assert (a is None and b is None) or torch.equal(a, b)
            want = g[0].to(torch.int32) - g[2].to(torch.int32)
            assert g[5].dtype == torch.float16 and g[5].is_contiguous()
            assert torch.equal(g[5].to(torch.int32), want)
            assert torch.equal(center_codes(g[0], g[2]), g[5])
        # per-job fallback (different head dims): quantize, then the centering kernel
        k64 = _inputs("normal", (2, 3, 77, 64), dtype, 4).cuda()
        n0 = _lib.launch_count()
        got = _quantize_batch((q, k64), (False, False), want_centered=(False, True))
        assert _lib.launch_count() - n0 == 3
        assert torch.equal(got[1][5].to(torch.int32), got[1][0].to(torch.int32) - got[1][2].to(torch.int32))
    # extreme codes and zero points: -128 - 127 and 127 - (-128)
    codes = torch.tensor([-128, 127] * 32, dtype=torch.int8, device="cuda").view(1, 1, 2, 32)
    zp = torch.tensor([127, -128], dtype=torch.int8, device="cuda").view(1, 1, 2, 1)
    c = center_codes(codes, zp)
    assert torch.equal(c.to(torch.int32), codes.to(torch.int32) - zp.to(torch.int32))
    lib = _lib.load()
    assert lib.qfa_center_per_token(None, None, None, 1, 1, 1, 16, 16, 16, 16, None) == -1
    assert lib.qfa_center_per_token(codes.data_ptr(), zp.data_ptr(), c.data_ptr(), 1, 1, 2, 24, 48, 48, 24, None) == -4
    assert lib.qfa_center_per_token(codes.data_ptr() + 1, zp.data_ptr(), c.data_ptr(), 1, 1, 2, 32, 64, 64, 32, None) == -6


def test_quantizer_rejects_bad_arguments(qfa):
    with pytest.raises(RuntimeError):
        qfa.asymmetric_quant_per_token(torch.zeros(1, 1, 2, 64, dtype=torch.float16))       # CPU tensor
    with pytest.raises(TypeError):
        qfa.asymmetric_quant_per_token(torch.zeros(1, 1, 2, 64, device="cuda"))             # fp32
    with pytest.raises(ValueError):
        qfa.asymmetric_quant_per_token(torch.zeros(2, 64, device="cuda", dtype=torch.float16))
    # empty input is a no-op
    c, s, z = qfa.asymmetric_quant_per_token(torch.zeros(1, 2, 0, 64, device="cuda", dtype=torch.float16))
    assert c.numel() == 0 and s.numel() == 0
