"""`flash_attn_func`-style front end ((B,S,H,D) layout, grouped K/V heads, packed variable-length batches)
against the CPU oracle and against the (B,H,S,D) operator it wraps."""
import math

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

from parity_util import close as _close, cpu_quant as _cpu_quant, gen as _gen  # noqa: E402


@pytest.fixture(scope="module")
def qfa():
    import quant_flash_attn_b200 as m
    from quant_flash_attn_b200 import _lib
    _lib.load()
    return m


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,Sq,Skv,H,D,causal", [(2, 200, 200, 3, 128, True), (1, 77, 333, 2, 64, False)])
def test_bshd_layout_vs_oracle(qfa, dtype, B, Sq, Skv, H, D, causal):
    # N(0,1) operands: this test is about the layout; heavy-tailed logits (where the 16-bit rounding of P shows)
    # have their own cases in test_gpu_attn.py
    q = _gen((B, Sq, H, D), dtype, 51)
    k = _gen((B, Skv, H, D), dtype, 52)
    v = _gen((B, Skv, H, D), dtype, 53)
    do = _gen((B, Sq, H, D), dtype, 54)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = qfa.quant_flash_attn_func(qc, kc, vc, causal=causal)
    assert o.shape == (B, Sq, H, D) and o.is_contiguous()
    o.backward(do.cuda())
    sm = 1.0 / math.sqrt(D)
    # the oracle works in (B,H,S,D); hand it the operands exactly as the GPU quantizer produced them
    qt, kt, vt = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    quant = tuple(_cpu_quant(t) for t in qfa.quantize_qkv(qt.cuda(), kt.cuda(), vt.cuda()))
    o_ref, lse_ref, quant = oracle.int8_mode_forward(qt, kt, vt, causal, sm, quant=quant, round_output=False)
    _close(o.transpose(1, 2), o_ref, what="bshd o")
    dq_ref, dk_ref, dv_ref = oracle.int8_mode_backward(quant, causal, sm, o.detach().transpose(1, 2).cpu(), lse_ref,
                                                       do.transpose(1, 2), dtype, round_output=False, round_p=dtype)
    _close(qc.grad.transpose(1, 2), dq_ref, what="bshd dq")
    _close(kc.grad.transpose(1, 2), dk_ref, what="bshd dk")
    _close(vc.grad.transpose(1, 2), dv_ref, what="bshd dv")


def test_bshd_equals_bhsd_operator(qfa):
    """Same numbers as the (B,H,S,D) operator on the transposed tensors, bit for bit: only the strides differ."""
    B, S, H, D = 2, 256, 4, 128
    q, k, v = (_gen((B, S, H, D), torch.bfloat16, s).cuda() for s in (61, 62, 63))
    got = qfa.quant_flash_attn_func(q, k, v, causal=True)
    want = qfa.quant_attention(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(),
                               v.transpose(1, 2).contiguous(), True, 1.0 / math.sqrt(D))
    assert torch.equal(got, want.transpose(1, 2))


def test_grouped_kv_heads(qfa):
    """H = 6 query heads on Hkv = 2 K/V heads: equals the call with the K/V heads repeated, and the K/V gradients
    are the sums over each group."""
    B, S, H, Hkv, D = 1, 192, 6, 2, 64
    q = _gen((B, S, H, D), torch.float16, 71).cuda().requires_grad_()
    k = _gen((B, S, Hkv, D), torch.float16, 72).cuda().requires_grad_()
    v = _gen((B, S, Hkv, D), torch.float16, 73).cuda().requires_grad_()
    do = _gen((B, S, H, D), torch.float16, 74).cuda()
    o = qfa.quant_flash_attn_func(q, k, v, causal=True)
    o.backward(do)
    kr = k.detach().repeat_interleave(H // Hkv, dim=2).requires_grad_()
    vr = v.detach().repeat_interleave(H // Hkv, dim=2).requires_grad_()
    qr = q.detach().clone().requires_grad_()
    o2 = qfa.quant_flash_attn_func(qr, kr, vr, causal=True)
    o2.backward(do)
    assert torch.equal(o, o2) and torch.equal(q.grad, qr.grad)
    want_dk = kr.grad.float().view(B, S, Hkv, H // Hkv, D).sum(3)
    want_dv = vr.grad.float().view(B, S, Hkv, H // Hkv, D).sum(3)
    _close(k.grad, want_dk, what="dk")
    _close(v.grad, want_dv, what="dv")
    # packed K/V form; without gradients the forward kernel reads the two K/V heads directly (no repetition):
    # same operands, same arithmetic, same bits
    o3 = qfa.quant_flash_attn_kvpacked_func(q.detach(), torch.stack([k.detach(), v.detach()], dim=2), causal=True)
    assert torch.equal(o3, o)
    with torch.no_grad():
        o4 = qfa.quant_flash_attn_func(q, k, v, causal=True)
    assert torch.equal(o4, o)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_grouped_kv_heads_native_forward(qfa, dtype):
    """(B,H,S,D) operator with 8 query heads on 2 K/V heads at D=128, ragged lengths, against the oracle fed with
    the repeated heads."""
    B, H, Hkv, Sq, Skv, D = 2, 8, 2, 150, 300, 128
    q = _gen((B, H, Sq, D), dtype, 91)
    k = _gen((B, Hkv, Skv, D), dtype, 92)
    v = _gen((B, Hkv, Skv, D), dtype, 93)
    sm = 1.0 / math.sqrt(D)
    qq, kq, vq = qfa.quantize_qkv(q.cuda(), k.cuda(), v.cuda())
    o, lse = qfa.int8_attention_forward(qq, kq, vq, False, sm, dtype)
    rep = lambda t: tuple(x.repeat_interleave(H // Hkv, dim=1) for x in _cpu_quant(t))
    o_ref, lse_ref, _ = oracle.int8_mode_forward(q, k.repeat_interleave(H // Hkv, dim=1), v.repeat_interleave(H // Hkv, dim=1),
                                                 False, sm, quant=(_cpu_quant(qq), rep(kq), rep(vq)), round_output=False)
    assert (lse.cpu() - lse_ref).abs().max() <= 2e-3
    _close(o, o_ref, what="o")


def test_varlen_batch(qfa):
    """Three sequences of different lengths (one empty) packed along the token axis: every sequence equals its own
    dense call, gradients included."""
    H, D = 2, 128
    lens_q, lens_k = [130, 0, 65], [130, 7, 200]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32).cuda()
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32).cuda()
    q = _gen((sum(lens_q), H, D), torch.bfloat16, 81).cuda().requires_grad_()
    k = _gen((sum(lens_k), H, D), torch.bfloat16, 82).cuda().requires_grad_()
    v = _gen((sum(lens_k), H, D), torch.bfloat16, 83).cuda().requires_grad_()
    do = _gen((sum(lens_q), H, D), torch.bfloat16, 84).cuda()
    o = qfa.quant_flash_attn_varlen_func(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), causal=False)
    assert o.shape == q.shape
    o.backward(do)
    q0 = k0 = 0
    for lq, lk in zip(lens_q, lens_k):
        if lq:
            qs = q.detach()[None, q0:q0 + lq].clone().requires_grad_()
            ks = k.detach()[None, k0:k0 + lk].clone().requires_grad_()
            vs = v.detach()[None, k0:k0 + lk].clone().requires_grad_()
            os_ = qfa.quant_flash_attn_func(qs, ks, vs)
            os_.backward(do[None, q0:q0 + lq])
            assert torch.equal(o[q0:q0 + lq], os_[0])
            assert torch.equal(q.grad[q0:q0 + lq], qs.grad[0])
            assert torch.equal(k.grad[k0:k0 + lk], ks.grad[0]) and torch.equal(v.grad[k0:k0 + lk], vs.grad[0])
        else:
            assert float(k.grad[k0:k0 + lk].abs().max()) == 0.0      # keys nobody attends to
        q0 += lq
        k0 += lk


def test_frontend_rejects_what_it_cannot_do(qfa):
    q = torch.zeros(1, 16, 4, 64, dtype=torch.float16, device="cuda")
    k = torch.zeros(1, 16, 3, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        qfa.quant_flash_attn_func(q, k, k)                     # 4 query heads on 3 K/V heads
    with pytest.raises(NotImplementedError):
        qfa.quant_flash_attn_func(q, q, q, dropout_p=0.1)
