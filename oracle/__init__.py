"""CPU oracle for the CompactAttention chunked-prefill path.  Test infrastructure only: it is the
checker for the CUDA library, never a fallback for it (see ``compact_oracle``'s module docstring)."""
