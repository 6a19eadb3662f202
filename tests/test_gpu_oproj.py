"""The output projection fused with the tensor-parallel reduction (``ca_oproj_allreduce``) on one GPU:
the tcgen05 GEMM alone (world 1) against torch, and the whole three-kernel protocol with two and four ranks
emulated on one device - every "rank" has its own staging, counters and output on the same GPU and the
launches go out rank after rank on one stream, so no kernel ever waits for one that has not run - against the
fp32 sum of the ranks' products.  A wait that nothing satisfies must end with the status bit, not hang."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from compactattention_b200 import _lib
    _lib.load()
    return _lib


def arr(ptrs):
    a = (C.c_void_p * len(ptrs))(*ptrs)
    return a, C.cast(a, C.POINTER(C.c_void_p))


def call(lib, a, w, rank, world, bufs, epoch, status, limit_ns=0, phases=0, mode=0, row_epochs=None, done_tiles_total=0):
    from compactattention_b200 import ops
    p = lib.OprojParams()
    if w is None:   # a is the partial [M, N] itself: the exchange without the GEMM
        p.a, p.a_stride_m, p.w, p.w_stride_n = a.data_ptr(), a.stride(0), None, 0
        p.M, p.N, p.K, p.dtype = a.shape[0], a.shape[1], 0, ops._DTYPES[a.dtype]
    else:
        p.a, p.a_stride_m, p.w, p.w_stride_n = a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0)
        p.M, p.N, p.K, p.dtype = a.shape[0], w.shape[0], a.shape[1], ops._DTYPES[a.dtype]
    p.world, p.rank = world, rank
    keep = []
    for name in ("out", "stage", "tile_counters", "done_counters"):
        if bufs.get(name) is None:
            continue
        k, ptr = arr(bufs[name])
        keep.append(k)
        setattr(p, name, ptr)
    p.out_stride_m, p.epoch, p.phases, p.wait_limit_ns, p.status = p.N, epoch, phases, limit_ns, status.data_ptr()
    p.mode, p.stage_bytes, p.done_tiles_total = mode, bufs.get("stage_bytes", 0), done_tiles_total
    if row_epochs is not None:
        re_arr = (C.c_uint32 * len(row_epochs))(*row_epochs)
        p.row_epochs = C.cast(re_arr, C.POINTER(C.c_uint32))
    rc = lib.load().ca_oproj_allreduce(C.byref(p), ops._stream())
    assert rc == 0, lib.load().ca_last_error()


@pytest.mark.parametrize("M,N,K,dtype", [(1024, 4096, 512, torch.bfloat16), (232, 512, 4096, torch.bfloat16), (1, 256, 64, torch.float16),
                                         (2048, 4096, 1024, torch.bfloat16)])
def test_projection_gemm_alone(lib, M, N, K, dtype):
    g = torch.Generator(device="cuda").manual_seed(M + K)
    a = torch.randn((M, K), device="cuda", generator=g).to(dtype)
    w = (torch.randn((N, K), device="cuda", generator=g) * 0.05).to(dtype)
    out = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    call(lib, a, w, 0, 1, {"out": [out.data_ptr()]}, 1, status)
    want = a.float() @ w.float().T
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    err = (out.float() - want).abs()
    assert not torch.isnan(out.float()).any()
    assert (err / (want.abs() + 1.0)).max().item() < 1e-2, err.max().item()


def make_world(lib, world, M_max, N, dtype):
    stage_b, cnt_b = C.c_size_t(0), C.c_size_t(0)
    assert lib.load().ca_oproj_scratch_bytes(M_max, N, world, C.byref(stage_b), C.byref(cnt_b)) == 0
    esize = torch.empty((), dtype=dtype).element_size()
    outs = [torch.full((M_max, N), float("nan"), dtype=dtype, device="cuda") for _ in range(world)]
    stages = [torch.empty(int(stage_b.value) // esize, dtype=dtype, device="cuda") for _ in range(world)]
    counters = [torch.zeros(int(cnt_b.value) // 4, dtype=torch.int32, device="cuda") for _ in range(world)]
    n_tc = int(cnt_b.value) // 4 - 1
    bufs = {"out": [t.data_ptr() for t in outs], "stage": [t.data_ptr() for t in stages],
            "tile_counters": [t.data_ptr() for t in counters], "done_counters": [t.data_ptr() + 4 * n_tc for t in counters],
            "stage_bytes": int(stage_b.value)}
    return outs, stages, counters, bufs


@pytest.mark.parametrize("world,M,N,K,mode", [(2, 1024, 4096, 2048, 0), (2, 1024, 4096, 2048, 1), (4, 1024, 4096, 1024, 0),
                                              (8, 1000, 4096, 512, 0), (2, 232, 1024, 256, 0), (2, 232, 1024, 256, 1)])
def test_reduction_protocol_with_emulated_ranks(lib, world, M, N, K, mode):
    one_shot = world == 2 and mode != 1   # auto picks the one-shot exchange on two ranks
    dtype = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(world * 100 + M)
    outs, stages, counters, bufs = make_world(lib, world, 1024, N, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):   # the buffers are reused: counters only grow
        xs = [torch.randn((M, K), device="cuda", generator=g).to(dtype) for _ in range(world)]
        ws = [(torch.randn((N, K), device="cuda", generator=g) * 0.05).to(dtype) for _ in range(world)]
        for o in outs:
            o.fill_(float("nan"))
        # the launch order of a real run seen from one device: every rank's GEMM, then every rank's reduction
        # and wait; a reduction finds all partials already there, a wait finds all tiles delivered after the last
        import compactattention_b200._lib as L
        n0 = L.launch_count()
        for phase in (1, 2, 4):
            for r in range(world):
                call(lib, xs[r], ws[r], r, world, bufs, epoch, status, phases=phase, mode=mode)
        assert L.launch_count() - n0 == (2 if one_shot else 3) * world   # one-shot has no final wait
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        parts = [x.float() @ w.float().T for x, w in zip(xs, ws)]
        want = sum(parts)
        # each partial is rounded to 16 bit once before the fp32 sum and the sum once after: the error is
        # bounded by half a unit in the last place (2^-9 for bf16) of every partial and of the result
        tol = 2.0 ** -8 * (sum(p.abs() for p in parts) + want.abs()) + 1e-3
        for r in range(world):
            got = outs[r][:M].float()
            assert not torch.isnan(got).any(), (epoch, r)
            assert ((got - want).abs() <= tol).all(), (epoch, r, (got - want).abs().max().item())
        for r in range(1, world):
            assert torch.equal(outs[r][:M], outs[0][:M])  # every rank holds the same bits


@pytest.mark.parametrize("world,mode", [(2, 0), (2, 1), (4, 0)])
def test_row_counts_may_change_between_calls(lib, world, mode):
    """Chunked prefill ends with a ragged chunk and goes on with single-row decode steps: the per-row-block call
    counts and the running tile total keep the counters' targets right when M shrinks and grows again."""
    N, K, dtype = 1024, 256, torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(7 + world)
    outs, stages, counters, bufs = make_world(lib, world, 1024, N, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    row_calls, tiles_total = [0] * 8, 0
    for epoch, M in enumerate((1024, 232, 1, 1024, 129), start=1):
        blocks = (M + 127) // 128
        for tm in range(blocks):
            row_calls[tm] += 1
        tiles_total += lib.load().ca_oproj_tile_count(M, N)
        xs = [torch.randn((M, K), device="cuda", generator=g).to(dtype) for _ in range(world)]
        ws = [(torch.randn((N, K), device="cuda", generator=g) * 0.05).to(dtype) for _ in range(world)]
        for phase in (1, 2, 4):
            for r in range(world):
                call(lib, xs[r], ws[r], r, world, bufs, epoch, status, phases=phase, mode=mode, row_epochs=row_calls[:blocks],
                     done_tiles_total=tiles_total, limit_ns=50_000_000)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, (epoch, M)
        parts = [x.float() @ w.float().T for x, w in zip(xs, ws)]
        want = sum(parts)
        tol = 2.0 ** -8 * (sum(p.abs() for p in parts) + want.abs()) + 1e-3
        for r in range(world):
            assert ((outs[r][:M].float() - want).abs() <= tol).all(), (epoch, M, r)


@pytest.mark.parametrize("world,M,N,mode", [(2, 1024, 4096, 0), (2, 1000, 512, 1), (4, 1024, 4096, 0), (8, 130, 1024, 0)])
def test_all_reduce_of_existing_partials(lib, world, M, N, mode):
    """w == NULL: the ranks' [M, N] partials are summed through the same exchange without the GEMM - the library's
    own all-reduce.  Emulated ranks on one device; the result must be the fp32 sum rounded once, on every rank."""
    dtype = torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(world + M)
    outs, stages, counters, bufs = make_world(lib, world, 1024, N, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for epoch in (1, 2):
        parts = [torch.randn((M, N), device="cuda", generator=g).to(dtype) for _ in range(world)]
        for o in outs:
            o.fill_(float("nan"))
        for phase in (1, 2, 4):
            for r in range(world):
                call(lib, parts[r], None, r, world, bufs, epoch, status, phases=phase, mode=mode)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        want = sum(p.float() for p in parts).to(dtype)   # exact partials, one rounding of the fp32 sum
        for r in range(world):
            assert torch.equal(outs[r][:M], want), (epoch, r)


def test_a_wait_that_nothing_satisfies_ends_with_the_status_bit(lib):
    """World of two, but only rank 0 ever runs: its reduction waits for rank 1's partial tiles, gives up after the
    (short) limit, sets CA_STATUS_TIMEOUT and returns; the context stays usable and a complete run then passes."""
    world, M, N, K = 2, 256, 512, 128
    dtype = torch.bfloat16
    outs, stages, counters, bufs = make_world(lib, world, 256, N, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.randn((M, K), device="cuda").to(dtype)
    w = (torch.randn((N, K), device="cuda") * 0.05).to(dtype)
    call(lib, x, w, 0, world, bufs, 1, status, limit_ns=2_000_000)   # 2 ms
    torch.cuda.synchronize()
    assert int(status.item()) & lib.CA_STATUS_TIMEOUT
    # fresh buffers, both ranks: fine
    outs, stages, counters, bufs = make_world(lib, world, 256, N, dtype)
    status.zero_()
    for phase in (1, 2, 4):
        for r in range(world):
            call(lib, x, w, r, world, bufs, 1, status, phases=phase)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = 2 * (x.float() @ w.float().T)
    assert ((outs[0][:M].float() - want).abs() <= 2.0 ** -7 * want.abs() + 1e-3).all()
