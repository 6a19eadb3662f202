"""CPU checks of the C-ABI boundary: the library builds/loads without a GPU driver and exports
every function that include/compactattn_b200.h declares (no compute calls here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "compactattn_b200.h"


@pytest.fixture(scope="module")
def lib():
    from compactattention_b200 import _lib, build

    build.build()
    return _lib.load()


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ca_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported(lib):
    names = declared_functions()
    assert "ca_attn_compact" in names and "ca_union_table" in names and len(names) >= 13
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_matches_header(lib):
    from compactattention_b200 import _lib

    assert set(_lib.exported_names()) == set(declared_functions())


def test_abi_version_and_error_string(lib):
    assert lib.ca_abi_version() == 2
    assert isinstance(lib.ca_last_error(), bytes)
    assert lib.ca_launch_count() >= 0


def test_contract_violations_return_codes_without_gpu(lib):
    from compactattention_b200 import _lib

    p = _lib.AttnParams()  # all zero: null pointers
    rc = lib.ca_attn_compact(ctypes.byref(p), None)
    assert rc == -1 and b"non-null" in lib.ca_last_error()
    u = _lib.UnionParams()
    assert lib.ca_union_table(ctypes.byref(u), None) == -1
    s = _lib.SelectParams()
    assert lib.ca_select_rows(ctypes.byref(s), None) == -1
    g = _lib.GatherParams()
    assert lib.ca_gather_kv(ctypes.byref(g), None) == -1


def test_struct_sizes_match_c_layout():
    """ctypes mirrors must have the size the C compiler gives the header's structs."""
    import subprocess, tempfile, textwrap
    from compactattention_b200 import _lib

    src = textwrap.dedent("""
        #include <stdio.h>
        #include "compactattn_b200.h"
        int main(void) {
          printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(ca_gate_prepare_params), sizeof(ca_kv_layout), sizeof(ca_attn_params),
                 sizeof(ca_select_params), sizeof(ca_union_params), sizeof(ca_pool_params),
                 sizeof(ca_project_params), sizeof(ca_gate_score_params), sizeof(ca_flashprefill_score_params),
                 sizeof(ca_gather_params), sizeof(ca_rope_append_params), sizeof(ca_chunk_step_params));
          return 0;
        }""")
    with tempfile.TemporaryDirectory() as d:
        c = Path(d) / "sz.c"
        c.write_text(src)
        exe = Path(d) / "sz"
        subprocess.run(["gcc", "-I", str(ROOT / "include"), str(c), "-o", str(exe)], check=True)
        sizes = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    mirrors = [_lib.GatePrepareParams, _lib.KvLayout, _lib.AttnParams, _lib.SelectParams, _lib.UnionParams, _lib.PoolParams,
               _lib.ProjectParams, _lib.GateScoreParams, _lib.FlashPrefillScoreParams, _lib.GatherParams,
               _lib.RopeAppendParams, _lib.ChunkStepParams]
    assert sizes == [ctypes.sizeof(m) for m in mirrors]


def test_ops_refuse_cpu_tensors():
    import torch
    from compactattention_b200 import ops

    with pytest.raises(ValueError, match="CUDA tensors only"):
        ops.union_table(mask=torch.zeros((1, 4, 8), dtype=torch.bool), num_kv_heads=1, kv_blocks=8, past_blocks=4)


def test_programmatic_launch_toggle_is_host_state_only():
    """The launch-mode switch is a process-wide flag; flipping it needs no device."""
    from compactattention_b200 import _lib

    was = _lib.set_programmatic_launch(True)
    assert was is False           # plain launches by default
    assert _lib.set_programmatic_launch(False) is True
    assert _lib.set_programmatic_launch(False) is False


def test_measurement_drivers_import_without_a_gpu():
    """The drivers quoted in profiles/ must at least import and parse their arguments on a CPU box."""
    import importlib
    for name in ("sweep", "kernel_case", "cycle_accounting", "select_accounting", "tp_check", "chunk_driver",
                 "prefill_sparse.llama.run_prefill"):
        importlib.import_module(f"compactattention_b200.{name}")


def test_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs the oracle port on the host cores and prints one JSON line with
    the keys the benchmark contract names (no GPU needed)."""
    import json
    import subprocess
    import sys

    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr[-500:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "us" and line["higher_is_better"] is False
    assert line["metric"].startswith("per-chunk attn latency") and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_recorded_calls_are_reissued_as_they_were(lib):
    """`_lib.record()` keeps the enqueuing calls of its body; `CallList.run()` re-issues them and raises on a
    failing return code.  (Null parameter blocks: the calls fail validation before touching a device.)"""
    from compactattention_b200 import _lib

    u = _lib.UnionParams()
    with _lib.record() as calls:
        assert lib.ca_union_table(ctypes.byref(u), None) == -1
        assert lib.ca_abi_version() == 2          # not an enqueuing call: not recorded
    assert [c[0] for c in calls.calls] == ["ca_union_table"]
    with pytest.raises(RuntimeError, match="ca_union_table"):
        calls.run()
    assert lib.ca_union_table(ctypes.byref(u), None) == -1 and len(calls.calls) == 1   # nothing is recorded outside the block
    with pytest.raises(RuntimeError):
        with _lib.record():
            with _lib.record():
                pass
