"""The attention entry point for hosts that cannot allocate device memory.

Some hosts of this library may not call cudaMalloc at all: an inference engine that reserved the
whole of HBM for its own pool at start-up (a later allocation simply fails), or a latency-critical
loop where allocation and the synchronisation it implies are forbidden.  They cannot hand
``ca_attn_compact`` a workspace, so ``ca_attn_compact_static_scratch`` keeps the kernel's scratch
(the partial accumulators of work units that are cut across SMs) in a buffer compiled into the
library.  This test drives that entry point through the C ABI on shapes that do cut units, twice
in a row (the buffer keeps the first call's contents), and compares with the ordinary entry point.
It is named to be collected last, and it passes on its own in a fresh process as well.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

# the tolerance of the attention parity tests (bf16 vs an fp32 reference); the two entry points run
# the same kernels, so they are also required to agree far more tightly than that
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from compactattention_b200 import _lib, ops

    return _lib, ops


def make_case(ops, seed, B, Q, K, Hq, Hkv, density, bs=64):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, Q, Hq, 128), generator=g).to(torch.bfloat16).cuda()
    k = torch.randn((B, K, Hkv, 128), generator=g).to(torch.bfloat16).cuda()
    v = torch.randn((B, K, Hkv, 128), generator=g).to(torch.bfloat16).cuda()
    Pb = (K - Q) // bs
    keep = torch.rand((B * Hkv, Pb), generator=g) < density
    idx = torch.full((B * Hkv, Pb), -1, dtype=torch.int32)
    counts = keep.sum(-1).to(torch.int32)
    for r in range(B * Hkv):
        sel = torch.nonzero(keep[r]).flatten().to(torch.int32)
        idx[r, : sel.numel()] = sel
    return q, ops.KvCacheView.from_seq_first(k, v), idx.cuda(), counts.cuda()


def raw_static_call(_lib, ops, q, kv, K, Hkv, idx, counts, out, status):
    """Fills ca_attn_params by hand and calls the C entry point directly (no workspace fields)."""
    p = _lib.AttnParams()
    p.q, p.q_stride_b, p.q_stride_t, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    p.out, p.o_stride_b, p.o_stride_t, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    p.kv = kv.to_c()
    p.block_idx, p.counts, p.block_idx_stride = idx.data_ptr(), counts.data_ptr(), idx.shape[-1]
    p.B, p.Q, p.Hq, p.Hkv, p.D = q.shape[0], q.shape[1], q.shape[2], Hkv, 128
    p.kv_len, p.block_size, p.dtype = K, 64, _lib.CA_DTYPE_BF16
    p.softmax_scale = 1.0 / math.sqrt(128)
    p.status = status.data_ptr()
    rc = _lib.load().ca_attn_compact_static_scratch(C.byref(p), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.load().ca_last_error()


def test_static_scratch_matches_workspace_entry_point_twice(mods):
    _lib, ops = mods
    # two different shapes, both with few and long work units, so that units are cut across SMs and the
    # pieces merged through the scratch; the second call finds the first call's partials in the buffer
    cases = [dict(seed=1, B=1, Q=256, K=32768, Hq=8, Hkv=2, density=0.5),
             dict(seed=2, B=2, Q=128, K=16384, Hq=4, Hkv=1, density=0.6)]
    for c in cases:
        q, kv, idx, counts = make_case(ops, **c)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        want = ops.attn_compact(q, kv, c["K"], c["Hkv"], idx, counts, status=status)
        whole = ops.attn_compact(q, kv, c["K"], c["Hkv"], idx, counts, status=status, use_workspace=False)
        got = torch.full_like(want, float("nan"))
        launches = _lib.launch_count()
        raw_static_call(_lib, ops, q, kv, c["K"], c["Hkv"], idx, counts, got, status)
        torch.cuda.synchronize()
        assert _lib.launch_count() - launches == 2  # attention + the merge of cut units
        assert int(status.item()) == 0
        assert not torch.isnan(got.float()).any()
        # same kernels, same cut, same merge order as the workspace route: identical bits
        assert torch.equal(got, want)
        # and the cut route really ran: units kept whole sum their KV steps in another order
        assert not torch.equal(got, whole)
        err = (got.float() - whole.float()).abs()
        assert err.max().item() < MAX_ABS and err.mean().item() < MEAN_ABS


def test_static_scratch_wrapper_and_errors(mods):
    _lib, ops = mods
    q, kv, idx, counts = make_case(ops, seed=3, B=1, Q=128, K=2048, Hq=4, Hkv=1, density=0.5)
    want = ops.attn_compact(q, kv, 2048, 1, idx, counts)
    out = torch.empty_like(want)
    ops.attn_compact_static_scratch(q, kv, 2048, 1, idx, counts, out)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    # contract violations are reported, not executed
    p = _lib.AttnParams()
    assert _lib.load().ca_attn_compact_static_scratch(C.byref(p), None) == -1
