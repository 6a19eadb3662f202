"""Llama integration of the path: attention modules with the reference's forward signatures."""
from .modeling_llama_compactattn import (  # noqa: F401
    CompactAttnCache,
    CompactAttnLlamaConfig,
    LlamaFlashPrefillCompactAttnAttention,
    LlamaSeerAttentionChunkedDense,
)
