"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): every rank computes the path for
its own KV heads with the CPU oracle, the row-parallel output projection is summed with the path's
one collective, and the result equals the single-rank computation.  Also the failure path: a rank
that raises before the collective is seen by the others as a time-out, not a hang."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from compactattention_b200 import tp
from oracle import compact_oracle as co


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make(seed=5):
    g = torch.Generator().manual_seed(seed)
    B, Q, K, Hq, Hkv, D, bs, hidden = 1, 128, 640, 8, 4, 128, 64, 96
    q = torch.randn((B, Q, Hq, D), generator=g)
    k = torch.randn((B, K, Hkv, D), generator=g)
    v = torch.randn((B, K, Hkv, D), generator=g)
    keep = torch.rand((B, Hq, K // bs), generator=g) < 0.3
    w_o = torch.randn((hidden, Hq * D), generator=g) * 0.05
    return q, k, v, keep, w_o, (B, Q, K, Hq, Hkv, D, bs, hidden)


def _rank_output(shard, q, k, v, keep, w_o, dims):
    B, Q, K, Hq, Hkv, D, bs, hidden = dims
    q_r, k_r, v_r = shard.slice_q(q), shard.slice_kv(k), shard.slice_kv(v)
    keep_r = shard.slice_q(keep, 1)
    idx, counts = co.block_union_table(keep_r, Q, K, bs, shard.group)
    attn = co.compact_attention(q_r, k_r, v_r, idx, counts, bs)  # [B, Q, Hq/world, D]
    return attn.reshape(B, Q, -1) @ shard.slice_o_proj(w_o, D).T


def _worker(rank, world, port, fail_rank, result_dict):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        q, k, v, keep, w_o, dims = _make()
        shard = tp.HeadShard(world, rank, dims[3], dims[4])
        if rank == fail_rank:
            raise RuntimeError("injected failure before the collective")
        partial = _rank_output(shard, q, k, v, keep, w_o, dims)
        tp.reduce_layer_output(partial)
        t = tp.max_over_ranks([float(rank + 1), 10.0 - rank], "cpu")
        if rank == 0:
            result_dict["out"] = partial
            result_dict["max"] = t
    except Exception as exc:  # reported to the parent
        result_dict[f"error{rank}"] = f"{type(exc).__name__}: {exc}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(world, fail_rank=-1):
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, port, fail_rank, results), nprocs=world, join=True)
        return dict(results)


def test_head_shard_arithmetic():
    s = tp.HeadShard(4, 2, 32, 8)
    assert list(s.kv_heads) == [4, 5] and list(s.q_heads) == list(range(16, 24)) and s.group == 4
    w = torch.arange(32 * 2 * 3).view(32, 2, 3)
    assert torch.equal(s.slice_gate_weight(w), w[16:24])
    assert torch.equal(s.slice_gate_weight(w[:8]), w[4:6])
    with pytest.raises(ValueError):
        tp.HeadShard(3, 0, 32, 8)
    with pytest.raises(ValueError):
        s.slice_gate_weight(w[:5])
    # the shards of all ranks tile the heads exactly once
    seen = sorted(h for r in range(4) for h in tp.HeadShard(4, r, 32, 8).q_heads)
    assert seen == list(range(32))


@pytest.mark.timeout(120)
def test_two_rank_path_matches_single_rank():
    res = _run(2)
    assert not [k for k in res if k.startswith("error")], res
    q, k, v, keep, w_o, dims = _make()
    single = _rank_output(tp.HeadShard(1, 0, dims[3], dims[4]), q, k, v, keep, w_o, dims)
    assert torch.allclose(res["out"], single, rtol=1e-4, atol=1e-4)
    assert res["max"] == [2.0, 10.0]


@pytest.mark.timeout(120)
def test_rank_failure_before_collective_times_out_not_hangs():
    res = _run(2, fail_rank=1)
    assert "injected failure" in res.get("error1", "")
    # rank 0 entered the all-reduce alone and got an error from the process-group time-out
    assert "error0" in res, res


def _ledger_worker(rank, world, port, result_dict):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        from compactattention_b200 import _lib
        ledger = tp.ProjectionCallLedger(1024, 4096)
        states = []
        for rows in (1024, 232, 1, 1024, 129):   # full chunks, a ragged last chunk, a decode step
            epoch, row_epochs, tiles = ledger.next_call(rows)
            assert tiles == sum(_lib.load().ca_oproj_tile_count(r, 4096) for r in (1024, 232, 1, 1024, 129)[:epoch])
            states.append([epoch, tiles] + row_epochs + [0] * (8 - len(row_epochs)))
        mine = torch.tensor(states, dtype=torch.int64)
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        # CPU tensors never take the fused kernels: the library GEMM + all-reduce route stays in charge
        g = torch.Generator().manual_seed(3)
        x_all = torch.randn((world, 4, 64), generator=g)
        w_all = torch.randn((world, 256, 64), generator=g)
        assert not tp.fused_projection_applies(x_all[rank], w_all[rank], None, 1024)
        y = torch.nn.functional.linear(x_all[rank], w_all[rank])
        tp.reduce_layer_output(y)
        if rank == 0:
            result_dict["same_ledgers"] = all(torch.equal(gathered[0], t) for t in gathered)
            result_dict["last_state"] = states[-1]
            result_dict["sum_ok"] = bool(torch.allclose(y, sum(x_all[r] @ w_all[r].T for r in range(world)), atol=1e-4))
    except Exception as exc:
        result_dict[f"error{rank}"] = f"{type(exc).__name__}: {exc}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_projection_ledgers_agree_across_ranks_and_cpu_tensors_take_the_library_route():
    """The counters of the fused output projection only grow; their targets come from a ledger every rank keeps
    by itself.  Two gloo ranks issue the same calls (row counts that shrink and grow) and must hold identical
    ledgers; a block of 128 rows that a short call did not cover keeps its old target."""
    port = _free_port()
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_ledger_worker, args=(2, port, results), nprocs=2, join=True)
        res = dict(results)
    assert not [k for k in res if k.startswith("error")], res
    assert res["same_ledgers"] and res["sum_ok"]
    # after 1024, 232, 1, 1024, 129 rows: call 5; row block 0 covered 5 times, block 1 four times (not by the
    # decode step), blocks 2..7 twice
    assert res["last_state"][0] == 5 and res["last_state"][2:4] == [5, 4]
    ledger = tp.ProjectionCallLedger(256, 512)
    with pytest.raises(ValueError):
        ledger.next_call(257)
