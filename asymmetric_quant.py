"""Drop-in module name of the reference project (asymmetric_quant.py): re-exports the
B200 implementation so `from asymmetric_quant import asymmetric_quant_per_token` keeps working."""
from quant_flash_attn_b200.asymmetric_quant import (  # noqa: F401
    asymmetric_quant_per_token, asymmetric_quant_per_token_ex, dequantize_per_token,
)
