"""Generates the golden fixtures in this directory from the REFERENCE implementation.

Run once, in a container that has the reference checkout and Triton but no GPU:

    QFA_REFERENCE_DIR=/path/to/quant_flash_attn python tests/golden/make_golden.py

The reference kernels are executed unmodified on the CPU through Triton's
interpreter (TRITON_INTERPRET=1).  Two harness-side adaptations are needed and
neither touches the kernels' arithmetic:

* the autotuner needs a GPU driver, so the kernels are launched through `.fn`
  with an explicit block size (results do not depend on it: min/max are exact,
  and the attention cases use KV lengths that are multiples of the block);
* the interpreter cannot call `libdevice.round`; it is replaced by the same
  function written with floor/ceil (round half away from zero).

The interpreter has no bf16, so all fixtures are fp16.  Outputs are stored as
compressed .npz next to this script; inputs are stored too so the tests do not
depend on any RNG implementation.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
if "QFA_REFERENCE_DIR" not in os.environ:
    sys.exit("set QFA_REFERENCE_DIR to a checkout of the reference project (yisunlp/quant_flash_attn)")
REF = os.environ["QFA_REFERENCE_DIR"]
sys.path.insert(0, REF)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402
from triton.language.extra.cuda import libdevice  # noqa: E402


@triton.jit
def _round_half_away(x):
    return tl.where(x >= 0, tl.floor(x + 0.5), tl.ceil(x - 0.5))


libdevice.round = _round_half_away
tl.extra.cuda.libdevice.round = _round_half_away

import asymmetric_quant as ref_aq  # noqa: E402
import quant_flash_attn as ref_qfa  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def ref_quantize(x: torch.Tensor, block_k: int = 64):
    """The body of the reference's asymmetric_quant_per_token (asymmetric_quant.py:123-149)
    with the autotuner bypassed."""
    Z, H, M, K = x.shape
    codes = torch.empty_like(x, dtype=torch.int8)
    scale = torch.empty(Z, H, M, 1, dtype=torch.float16)
    zp = torch.empty(Z, H, M, 1, dtype=torch.int8)
    ref_aq._asymmetric_quant_kernel.fn[(Z * H * M,)](
        x, codes, scale.view(-1), zp.view(-1),
        x.stride(0), x.stride(1), x.stride(2), x.stride(3),
        Z, H, M, HEAD_DIM=K, BLOCK_SIZE_K=block_k)
    return codes, scale, zp


def ref_attention(q, kv_quant, sm_scale, grad_out, block_n=64):
    """QuantFlashAttention.forward/backward (quant_flash_attn.py:179-237), autotuner bypassed."""
    codes, scale, zp = kv_quant
    Z, H, NQ, D = q.shape
    NKV = codes.shape[2]
    PQ = max(triton.next_power_of_2(NQ), 16)
    o = torch.empty_like(q)
    lse = torch.zeros((Z, H, PQ), dtype=torch.float32)
    ref_qfa._attn_fwd_kernel_quantized.fn[(Z * H,)](
        q, codes, scale, zp, lse, o,
        *q.stride(), *codes.stride(), *scale.stride()[:3], *zp.stride()[:3], *o.stride(),
        Z, H, NQ, NKV, sm_scale, HEAD_DIM=D, PADDED_N_CTX_Q=PQ, BLOCK_N=block_n)
    dq = torch.empty_like(q)
    dkv = torch.empty(codes.shape, dtype=q.dtype)
    delta = torch.zeros_like(lse)
    ref_qfa._bwd_preprocess_kernel[(Z * H,)](
        o, grad_out, delta, *o.stride(), Z, H, NQ, HEAD_DIM=D, PADDED_N_CTX_Q=PQ)
    ref_qfa._bwd_kernel_quantized.fn[(Z * H,)](
        q, codes, scale, zp, lse, grad_out, delta, dq, dkv,
        *q.stride(), *codes.stride(), *scale.stride()[:3], *zp.stride()[:3], *grad_out.stride(),
        Z, H, NQ, NKV, sm_scale, HEAD_DIM=D, PADDED_N_CTX_Q=PQ, BLOCK_N=block_n)
    return o, lse[..., :NQ].contiguous(), delta[..., :NQ].contiguous(), dq, dkv


def edge_rows(D):
    """Rows that exercise the quantizer's branches (asymmetric_quant.py:84-91,103-104)."""
    g = torch.Generator().manual_seed(7)
    rows = [
        torch.zeros(D),                                   # constant row -> scale 1
        torch.full((D,), 3.25),                           # constant non-zero
        -torch.rand(D, generator=g) - 0.5,                # all negative -> zp clamps high
        torch.rand(D, generator=g) + 0.5,                 # all positive -> zp clamps low
        torch.linspace(-1, 1, D),                         # evenly spread: many .5 ties
        torch.linspace(0, 255, D),                        # scale exactly 1, integer values
        torch.linspace(-127.5, 127.5, D),                 # scale 1, every value on a .5 tie
        torch.randn(D, generator=g) * 1e-4,               # tiny magnitudes
        torch.randn(D, generator=g) * 300.0,              # large magnitudes (fp16 scale still finite)
        torch.cat([torch.full((D - 1,), 1.0), torch.tensor([-1.0])]),  # one outlier
        torch.cat([torch.zeros(D - 1), torch.tensor([6.1e-5])]),       # near-denormal range
    ]
    return torch.stack(rows).to(torch.float16)


def main():
    torch.manual_seed(20)  # the reference test's seed (test_accuracy.py:58)
    out = {}

    # ---- quantizer cases
    cases = {
        "q_z1h2m40d64": torch.randn(1, 2, 40, 64).half(),
        "q_z2h1m33d128": torch.randn(2, 1, 33, 128).half(),
        "q_outlier_d128": None,
        "q_edge_d64": edge_rows(64)[None, None],
        "q_edge_d128": edge_rows(128)[None, None],
        # (B,S,H,D)-contiguous data viewed as (B,H,S,D): codes inherit these strides
        "q_transposed_d64": torch.randn(2, 9, 3, 64).half().transpose(1, 2),
        "q_d96": torch.randn(1, 1, 19, 96).half(),          # head dim that is not a power of two
    }
    x = torch.randn(1, 2, 24, 128)
    x[..., 5] *= 20.0
    x[..., 77] *= 20.0
    cases["q_outlier_d128"] = x.half()
    for name, x in cases.items():
        blk = 32 if x.shape[-1] % 64 else 64
        codes, scale, zp = ref_quantize(x, block_k=blk)
        assert codes.stride() == x.stride()
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            x=x.contiguous().numpy(), x_stride=np.array(x.stride()),
                            codes=codes.contiguous().numpy(), scale=scale.numpy(), zp=zp.numpy())
        print("wrote", name, tuple(x.shape))

    # ---- attention (forward + backward), KV lengths multiples of the block
    att = {
        "a_z1h2q18kv512d64": (1, 2, 18, 512, 64),      # test_accuracy.py:37 shape, fewer heads
        "a_z1h1q17kv256d128": (1, 1, 17, 256, 128),
        "a_z2h2q32kv128d128": (2, 2, 32, 128, 128),
        "a_z1h2q97kv192d64": (1, 2, 97, 192, 64),
    }
    for name, (Z, H, NQ, NKV, D) in att.items():
        q = torch.randn(Z, H, NQ, D).half()
        kv = torch.randn(Z, H, NKV, D).half()
        go = torch.randn(Z, H, NQ, D).half()
        sm = 1.0 / D ** 0.5
        kvq = ref_quantize(kv)
        o, lse, delta, dq, dkv = ref_attention(q, kvq, sm, go)
        np.savez_compressed(os.path.join(HERE, name + ".npz"),
                            q=q.numpy(), kv=kv.numpy(), go=go.numpy(), sm_scale=np.float64(sm),
                            codes=kvq[0].numpy(), scale=kvq[1].numpy(), zp=kvq[2].numpy(),
                            o=o.numpy(), lse=lse.numpy(), delta=delta.numpy(),
                            dq=dq.numpy(), dkv=dkv.numpy())
        print("wrote", name)


if __name__ == "__main__":
    main()
