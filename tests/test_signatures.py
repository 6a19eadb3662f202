"""The mirror's call signatures against the reference's, frozen in ``tests/golden/signatures.json``
by ``tests/golden/make_signatures.py`` (parameter names, order, kinds and defaults read from the
reference's source).  A mirror callable must accept every reference parameter under the same name,
in the same position, of the same kind and with the same default; it may add parameters after the
reference's positional ones and extra keyword-only ones.  Runs without a GPU.
"""
import inspect
import json
from pathlib import Path

import pytest

FROZEN = json.loads((Path(__file__).resolve().parent / "golden" / "signatures.json").read_text())


def mirror(key):
    from compactattention_b200 import load_attention_replacement as lar
    from compactattention_b200 import modules
    from compactattention_b200.prefill_sparse import attn_gate
    from compactattention_b200.prefill_sparse.llama import modeling_llama_compactattn as mm
    table = {
        "chunked_prefill_column_dense_attention_forward": modules.chunked_prefill_column_dense_attention_forward,
        "chunked_prefill_column_dense_attention_from_keep_block": modules.chunked_prefill_column_dense_attention_from_keep_block,
        "flashprefill_compactattn_prefill_full_kv": modules.flashprefill_compactattn_prefill_full_kv,
        "AttnGate.__init__": attn_gate.AttnGate.__init__,
        "AttnGate.forward": attn_gate.AttnGate.forward,
        "AttnGate.score_compressed_blocks": attn_gate.AttnGate.score_compressed_blocks,
        "AttnGate.apply_block_position_embeddings": attn_gate.AttnGate.apply_block_position_embeddings,
        "MultiHeadLinear.__init__": attn_gate.MultiHeadLinear.__init__,
        "LlamaSeerAttentionChunkedDense.forward": mm.LlamaSeerAttentionChunkedDense.forward,
        "LlamaSeerAttentionChunkedDense._do_kv_cache_update": mm.LlamaSeerAttentionChunkedDense._do_kv_cache_update,
        "LlamaSeerAttentionChunkedDense._do_chunked_compactattn_attention":
            mm.LlamaSeerAttentionChunkedDense._do_chunked_compactattn_attention,
        "LlamaFlashPrefillCompactAttnAttention.forward": mm.LlamaFlashPrefillCompactAttnAttention.forward,
        "load_llama_attention_replacement_model": lar.load_llama_attention_replacement_model,
        "_adapt_attention_return_contract": lar._adapt_attention_return_contract,
        "_reuse_attention_projections": lar._reuse_attention_projections,
    }
    return table[key]


def default_source(param):
    if param.default is inspect.Parameter.empty:
        return None
    return repr(param.default)


@pytest.mark.parametrize("key", sorted(FROZEN))
def test_mirror_keeps_the_reference_signature(key):
    want = FROZEN[key]["params"]
    got = list(inspect.signature(mirror(key)).parameters.values())
    got_by_name = {p.name: p for p in got}
    positional = [w for w in want if w[1] in ("POSITIONAL_ONLY", "POSITIONAL_OR_KEYWORD")]
    for i, (name, kind, default) in enumerate(positional):
        p = got[i]
        assert p.name == name, f"{key}: positional parameter {i} is {p.name!r}, the reference has {name!r}"
        assert p.kind.name == kind, f"{key}: {name} is {p.kind.name}, the reference has {kind}"
        assert default_source(p) == default, f"{key}: {name} defaults to {default_source(p)}, the reference to {default}"
    for name, kind, default in want:
        if kind == "KEYWORD_ONLY":
            p = got_by_name.get(name)
            assert p is not None and p.kind.name == "KEYWORD_ONLY", f"{key}: keyword-only parameter {name} is missing"
            assert default_source(p) == default, f"{key}: {name} defaults to {default_source(p)}, the reference to {default}"
        elif kind in ("VAR_KEYWORD", "VAR_POSITIONAL"):
            assert any(p.kind.name == kind for p in got), f"{key}: the reference accepts {kind}"
    # anything the mirror adds has a default, so every reference call site still binds
    known = {w[0] for w in want}
    for p in got:
        if p.name not in known and p.kind.name in ("POSITIONAL_OR_KEYWORD", "KEYWORD_ONLY"):
            assert p.default is not inspect.Parameter.empty, f"{key}: added parameter {p.name} has no default"
