"""CPU oracle for the quantized flash-attention hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
it exists so that the tests, the smoke check and the CPU-baseline leg of the
benchmark have an independent restatement of the reference algorithm to check
the CUDA kernels against.

Parity status: pinned.  `tests/golden/` holds outputs of the reference's own
Triton kernels (run on CPU through the Triton interpreter, fp16 inputs) and the
not-gpu test-suite checks this oracle against them: quantizer codes, scales and
zero-points bit for bit, attention forward/backward to ~1e-3.
"""
from .quantizer import quantize_per_token, dequantize_per_token, round_half_away  # noqa: F401
from .attention import (  # noqa: F401
    ref_mode_forward, ref_mode_backward, int8_mode_forward, int8_mode_backward,
    attention_ops,
)
