"""Drop-in module name of the reference project (quant_flash_attn.py): re-exports the
B200 implementation so `from quant_flash_attn import quant_flash_attn` keeps working."""
from quant_flash_attn_b200.quant_flash_attn import (  # noqa: F401
    QuantFlashAttention, quant_flash_attn, QuantAttention, quant_attention,
)
