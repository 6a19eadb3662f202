"""Host-side mirror of the reference's ``compact_attn/modules`` operator interface for the path."""
from .attention_forward_chunked_dense import (  # noqa: F401
    COMPACTATTN_VERSION,
    chunked_prefill_column_dense_attention_forward,
    chunked_prefill_column_dense_attention_from_keep_block,
)
from .flashprefill_prefill import flashprefill_compactattn_prefill_full_kv  # noqa: F401
