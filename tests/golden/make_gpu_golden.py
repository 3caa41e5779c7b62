"""Generates the gpuref_q_*.npz fixtures: outputs of the REFERENCE quantizer kernel
(asymmetric_quant.py, unmodified, Triton-compiled) running on a B200.

    QFA_REFERENCE_DIR=/path/to/quant_flash_attn python tests/golden/make_gpu_golden.py [out_dir]

Needs a GPU and the reference checkout.  These fixtures pin the bit pattern of the GPU
arithmetic (PTX div.full.f32, libdevice round) that a CPU restatement cannot reproduce; the
-m gpu tests require the CUDA quantizer to match them exactly.  The reference kernel cannot be
compiled for a batch or head count of 1 (Triton specialises the value 1 to a constant and the
kernel calls .to() on it), hence the (2,2,...) shapes of the small cases.
"""
import importlib.util
import math
import os
import sys

import numpy as np
import torch

if "QFA_REFERENCE_DIR" not in os.environ:
    sys.exit("set QFA_REFERENCE_DIR to a checkout of the reference project (yisunlp/quant_flash_attn)")
REF = os.environ["QFA_REFERENCE_DIR"]
OUT = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    m = importlib.util.module_from_spec(spec)
    sys.modules[name] = m
    spec.loader.exec_module(m)
    return m


def gen(kind, shape, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    if kind == "outlier":
        D = shape[-1]
        idx = torch.randperm(D, generator=g)[: max(1, (D + 99) // 100)]
        x[..., idx] *= 20.0
    elif kind == "loguniform":
        x = x * torch.exp(torch.empty(shape[:-1] + (1,)).uniform_(math.log(0.1), math.log(10.0), generator=g))
    elif kind == "edge":
        D, n = shape[-1], shape[2]
        rows = [torch.zeros(D), torch.full((D,), 3.25), -torch.rand(D, generator=g) - 0.5,
                torch.rand(D, generator=g) + 0.5, torch.linspace(-1, 1, D), torch.linspace(0, 255, D),
                torch.linspace(-127.5, 127.5, D), torch.randn(D, generator=g) * 1e-4,
                torch.randn(D, generator=g) * 300, torch.cat([torch.ones(D - 1), torch.tensor([-1.0])])]
        while len(rows) < n:
            rows.append(torch.randn(D, generator=g) * float(torch.rand(1, generator=g) * 50)
                        + float(torch.randn(1, generator=g) * 10))
        x = torch.stack(rows[:n])[None, None].expand(shape).clone()
    return x.to(dtype)


CASES = [
    ("normal", (1, 2, 1024, 128), torch.bfloat16, 1), ("outlier", (1, 2, 1024, 128), torch.bfloat16, 2),
    ("loguniform", (1, 2, 1024, 128), torch.bfloat16, 3), ("normal", (2, 2, 500, 64), torch.bfloat16, 4),
    ("normal", (1, 2, 1024, 128), torch.float16, 5), ("outlier", (2, 2, 500, 64), torch.float16, 6),
    ("edge", (2, 2, 64, 128), torch.bfloat16, 7), ("edge", (2, 2, 64, 64), torch.float16, 8),
    ("normal", (2, 2, 100, 96), torch.bfloat16, 9), ("normal", (2, 2, 100, 256), torch.float16, 10),
]


def main():
    ref = _load("ref_asymmetric_quant", os.path.join(REF, "asymmetric_quant.py"))
    for kind, shape, dtype, seed in CASES:
        x = gen(kind, shape, dtype, seed).cuda()
        c, s, z = ref.asymmetric_quant_per_token(x)
        tag = "bf16" if dtype == torch.bfloat16 else "f16"
        name = f"gpuref_q_{kind}_{'x'.join(map(str, shape))}_{tag}"
        np.savez_compressed(os.path.join(OUT, name + ".npz"), x_bits=x.view(torch.int16).cpu().numpy(),
                            dtype=np.array("bfloat16" if dtype == torch.bfloat16 else "float16"),
                            codes=c.cpu().numpy(), scale=s.cpu().numpy(), zp=z.cpu().numpy())
        print("wrote", name)


if __name__ == "__main__":
    main()
