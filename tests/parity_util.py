"""Shared pieces of the GPU parity tests: seeded inputs with the value distributions of the
benchmark configurations, the tolerance check, and a record of what was measured."""
import math

import torch

# Tolerance for results that share the kernel's semantics: max-abs error <= 2e-3 of the output
# scale, cosine similarity >= 0.9999.  The kernel's result is STORED in a 16-bit dtype, which
# alone moves an element by up to half an ulp of its own magnitude (2^-8 relative for bf16,
# 2^-11 for fp16); the comparison is against the oracle's un-rounded result and allows exactly
# that storage term per element on top of the bound.
REL_TOL = 2e-3
COS_TOL = 0.9999
HALF_ULP = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}

# every comparison made by close(): (label, max-abs / scale, max-abs beyond storage rounding / scale, cosine)
REPORT = []


def gen(shape, dtype, seed, kind="normal"):
    """Seeded stand-ins for the benchmark inputs: N(0,1); N(0,1) with 1 % of the channels x20
    ("outlier"); N(0,1) times a per-token magnitude log-uniform in [0.1, 10] ("loguniform")."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    if kind == "outlier":
        D = shape[-1]
        idx = torch.randperm(D, generator=g)[: max(1, (D + 99) // 100)]
        x[..., idx] *= 20.0
    elif kind == "loguniform":
        x = x * torch.exp(torch.empty(shape[:-1] + (1,)).uniform_(math.log(0.1), math.log(10.0), generator=g))
    return x.to(dtype)


def measure(got, want):
    """(scale of `want`, max-abs error, max-abs error beyond the storage rounding of got's dtype, cosine)."""
    storage = HALF_ULP.get(got.dtype, 0.0)
    got, want = got.detach().float().cpu().flatten(), want.detach().float().cpu().flatten()
    scale = want.abs().max().item()
    diff = (got - want).abs()
    excess = (diff - storage * want.abs()).max().item()
    c = torch.nn.functional.cosine_similarity(got.double(), want.double(), dim=0).item()
    return scale, diff.max().item(), excess, c


def close(got, want, rel=REL_TOL, cos=COS_TOL, what="", p_rounding=0.0):
    """`p_rounding` (half an ulp of the 16-bit dtype, or 0) is added to `rel` for results whose rows hang on ONE
    rounded weight.  The kernels, like the reference (quant_flash_attn.py:75,156,159-160), round P and dS to the
    16-bit dtype before the second products.  Where the softmax of a row sits on one or two keys, that single
    rounding (or one that falls the other way because two evaluations differ in the last fp32 bit) reaches the
    output undiminished instead of averaging out over many keys, and with two dominant keys of opposite dS the
    affected output element can be far smaller than the term that moved: the error is bounded by half an ulp of
    the OUTPUT SCALE, not of the element.  Only the tests that build such rows (logits growing along the key
    axis; channels scaled x20) pass it; everything else is held to the plain bound."""
    assert torch.isfinite(got).all(), what
    scale, raw, excess, c = measure(got, want)
    if scale > 1e-4:        # a result that is zero by construction has no scale to report against
        REPORT.append({"what": what, "dtype": str(got.dtype).replace("torch.", ""), "scale": scale,
                       "max_abs_over_scale": raw / scale, "beyond_storage_over_scale": max(excess, 0.0) / scale,
                       "cosine": c, "bound": rel + p_rounding})
    assert excess <= (rel + p_rounding) * scale + 1e-5, \
        f"{what}: max-abs excess {excess:.3e} > {rel + p_rounding} * {scale:.3e}"
    if scale > 1e-4:
        assert c >= cos, f"{what}: cosine {c}"


def cpu_quant(t):
    """GPU quantizer output tuple -> the oracle's (codes, scale fp32, zp, rowsum) on CPU."""
    codes, scale, zp, rowsum = t[:4]
    return (codes.cpu(), scale.float().cpu().squeeze(-1), zp.cpu().squeeze(-1), rowsum.cpu())


def head_quant(t, b, h):
    """One (batch, head) of a GPU quantizer output tuple as the oracle's CPU operands, leading dims (1,1)."""
    codes, scale, zp, rowsum = t[:4]
    sl = (slice(b, b + 1), slice(h, h + 1))
    return (codes[sl].cpu(), scale[sl].float().cpu().squeeze(-1), zp[sl].cpu().squeeze(-1), rowsum[sl].cpu())
