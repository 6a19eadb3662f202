"""Host-side mirror of the reference's ``compact_attn/prefill_sparse`` interface for the path."""
