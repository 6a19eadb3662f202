"""Freezes the call signatures of the reference's interface for the path into ``signatures.json``.

The reference's operator functions, gate class and attention-module forwards are what a caller binds
to; the mirror in ``compactattention_b200`` must keep their parameter names, order, kinds and
defaults.  This script reads them from a checkout of the reference with ``ast`` (no import, so the
model files that need an older transformers release are covered too) and writes one list of
``[name, kind, default-source-or-null]`` per callable; ``tests/test_signatures.py`` compares the
mirror against the committed file.

    python tests/golden/make_signatures.py            # needs COMPACTATTN_REFERENCE_ROOT or ../reference
"""
from __future__ import annotations

import ast
import json
import os
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = Path(os.environ.get("COMPACTATTN_REFERENCE_ROOT", str(HERE.parent.parent.parent / "reference")))

# (key, file relative to the reference root, class or None, function)
TARGETS = [
    ("chunked_prefill_column_dense_attention_forward", "compact_attn/modules/attention_forward_chunked_dense.py", None,
     "chunked_prefill_column_dense_attention_forward"),
    ("chunked_prefill_column_dense_attention_from_keep_block", "compact_attn/modules/attention_forward_chunked_dense.py", None,
     "chunked_prefill_column_dense_attention_from_keep_block"),
    ("flashprefill_compactattn_prefill_full_kv", "compact_attn/modules/flashprefill_prefill.py", None,
     "flashprefill_compactattn_prefill_full_kv"),
    ("AttnGate.__init__", "compact_attn/prefill_sparse/attn_gate.py", "AttnGate", "__init__"),
    ("AttnGate.forward", "compact_attn/prefill_sparse/attn_gate.py", "AttnGate", "forward"),
    ("AttnGate.score_compressed_blocks", "compact_attn/prefill_sparse/attn_gate.py", "AttnGate", "score_compressed_blocks"),
    ("AttnGate.apply_block_position_embeddings", "compact_attn/prefill_sparse/attn_gate.py", "AttnGate",
     "apply_block_position_embeddings"),
    ("MultiHeadLinear.__init__", "compact_attn/prefill_sparse/attn_gate.py", "MultiHeadLinear", "__init__"),
    ("LlamaSeerAttentionChunkedDense.forward", "compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py",
     "LlamaSeerAttentionChunkedDense", "forward"),
    ("LlamaSeerAttentionChunkedDense._do_kv_cache_update", "compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py",
     "LlamaSeerAttentionChunkedDense", "_do_kv_cache_update"),
    ("LlamaSeerAttentionChunkedDense._do_chunked_compactattn_attention",
     "compact_attn/prefill_sparse/llama/modeling_llama_seerattn_chunked_dense.py", "LlamaSeerAttentionChunkedDense",
     "_do_chunked_compactattn_attention"),
    ("LlamaFlashPrefillCompactAttnAttention.forward", "compact_attn/prefill_sparse/llama/modeling_llama_flashprefill_compactattn.py",
     "LlamaFlashPrefillCompactAttnAttention", "forward"),
    ("load_llama_attention_replacement_model", "compact_attn/load_attention_replacement.py", None,
     "load_llama_attention_replacement_model"),
    ("_adapt_attention_return_contract", "compact_attn/load_attention_replacement.py", None, "_adapt_attention_return_contract"),
    ("_reuse_attention_projections", "compact_attn/load_attention_replacement.py", None, "_reuse_attention_projections"),
]


def find_function(tree: ast.Module, cls, fn):
    body = tree.body
    if cls is not None:
        for node in body:
            if isinstance(node, ast.ClassDef) and node.name == cls:
                body = node.body
                break
        else:
            return None
    for node in body:
        if isinstance(node, (ast.FunctionDef, ast.AsyncFunctionDef)) and node.name == fn:
            return node
    return None


def describe(fn: ast.FunctionDef):
    a = fn.args
    out = []
    pos = list(a.posonlyargs) + list(a.args)
    defaults = [None] * (len(pos) - len(a.defaults)) + list(a.defaults)
    for i, (arg, d) in enumerate(zip(pos, defaults)):
        kind = "POSITIONAL_ONLY" if i < len(a.posonlyargs) else "POSITIONAL_OR_KEYWORD"
        out.append([arg.arg, kind, None if d is None else ast.unparse(d)])
    if a.vararg:
        out.append([a.vararg.arg, "VAR_POSITIONAL", None])
    for arg, d in zip(a.kwonlyargs, a.kw_defaults):
        out.append([arg.arg, "KEYWORD_ONLY", None if d is None else ast.unparse(d)])
    if a.kwarg:
        out.append([a.kwarg.arg, "VAR_KEYWORD", None])
    return out


def main() -> None:
    result = {}
    for key, rel, cls, fn in TARGETS:
        path = ROOT / rel
        node = find_function(ast.parse(path.read_text()), cls, fn) if path.exists() else None
        if node is None:
            print(f"not found in the reference: {key} ({rel})")
            continue
        result[key] = {"file": rel, "line": node.lineno, "params": describe(node)}
    out = HERE / "signatures.json"
    lines = []
    for key, entry in result.items():
        params = ",\n   ".join(json.dumps(p) for p in entry["params"])
        lines.append(f' {json.dumps(key)}: {{"file": {json.dumps(entry["file"])}, "line": {entry["line"]}, "params": [\n   {params}\n  ]}}')
    out.write_text("{\n" + ",\n".join(lines) + "\n}\n")
    print(f"wrote {out} ({len(result)} callables)")


if __name__ == "__main__":
    main()
