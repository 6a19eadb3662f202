"""Chunk append fused with RoPE and mean-K pooling (``ca_rope_append``) against the CPU oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from compactattention_b200 import ops as _ops
    return _ops


def rope_tables(positions: torch.Tensor, D: int, theta: float = 500000.0):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = positions.to(torch.float32)[:, None] * inv[None]
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos()[None], emb.sin()[None]   # [1, Q, D]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("table_dtype", ["same", "f32"])
@pytest.mark.parametrize("B,Q,position,page_size", [(2, 256, 512, 64), (1, 200, 72, 128), (1, 1024, 3072, 64)])
def test_rope_append_matches_oracle(ops, dtype, table_dtype, B, Q, position, page_size):
    from oracle import compact_oracle as oc
    g = torch.Generator().manual_seed(1234 + Q)
    Hq, Hkv, D, bs = 8, 2, 128, 64
    max_tokens = 4096
    pps = max_tokens // page_size
    q = torch.randn((B, Q, Hq, D), generator=g).to(dtype)
    k = torch.randn((B, Q, Hkv, D), generator=g).to(dtype)
    v = torch.randn((B, Q, Hkv, D), generator=g).to(dtype)
    cos, sin = rope_tables(torch.arange(position, position + Q), D)
    if table_dtype == "same":
        cos, sin = cos.to(dtype), sin.to(dtype)
    table = torch.randperm(B * pps, generator=g).to(torch.int32).view(B, pps)
    k_pages = torch.randn((B * pps, page_size, Hkv, D), generator=g).to(dtype)
    v_pages = torch.randn((B * pps, page_size, Hkv, D), generator=g).to(dtype)
    with_mean = position % bs == 0
    mean_k = torch.zeros((B, max_tokens // bs, Hkv, D), dtype=dtype)

    kp_ref, vp_ref = k_pages.clone(), v_pages.clone()
    q_ref, mk_ref = oc.rope_append(q, k, v, cos, sin, kp_ref, vp_ref, table, position, bs)

    kp, vp, mk = k_pages.cuda(), v_pages.cuda(), mean_k.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    view = ops.KvCacheView.from_paged(kp, vp, table.cuda())
    q_out = ops.rope_append(q.cuda(), k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), view, position,
                            mean_k=mk if with_mean else None, block_size=bs, status=status)
    assert int(status.item()) == 0
    # bit-exact: RoPE with torch's rounding, and the paged placement (pages outside the chunk untouched)
    assert torch.equal(q_out.cpu(), q_ref)
    assert torch.equal(kp.cpu(), kp_ref)
    assert torch.equal(vp.cpu(), vp_ref)
    if with_mean:
        nb = -(-Q // bs)
        got = mk[:, position // bs: position // bs + nb].cpu().float()
        # fp32 sums in a different order, one rounding to 16 bit: within one unit in the last place
        tol = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
        assert (got - mk_ref.float()).abs().max().item() <= tol * max(1.0, mk_ref.float().abs().max().item())
        assert torch.count_nonzero(mk[:, : position // bs]).item() == 0   # earlier blocks untouched


def test_rope_append_in_place_and_without_q(ops):
    from oracle import compact_oracle as oc
    g = torch.Generator().manual_seed(5)
    B, Q, Hq, Hkv, D = 1, 128, 4, 4, 64
    q = torch.randn((B, Q, Hq, D), generator=g).to(torch.bfloat16)
    k = torch.randn((B, Q, Hkv, D), generator=g).to(torch.bfloat16)
    v = torch.randn((B, Q, Hkv, D), generator=g).to(torch.bfloat16)
    cos, sin = rope_tables(torch.arange(Q), D)
    cos, sin = cos.to(torch.bfloat16), sin.to(torch.bfloat16)
    from compactattention_b200.paged_cache import PagedKVCache
    cache = PagedKVCache(B, 256, Hkv, D, "cuda")
    qc = q.cuda()
    q_rot, n = cache.append_rope(qc, k.cuda(), v.cuda(), cos.cuda(), sin.cuda(), q_out=qc)   # rotates q in place
    assert n == Q and q_rot.data_ptr() == qc.data_ptr()
    assert torch.equal(qc.cpu(), oc.apply_rope(q, cos, sin))
    assert torch.equal(cache.k_pages[:2].cpu().reshape(1, Q, Hkv, D), oc.apply_rope(k, cos, sin))
    # keys/values only
    cache2 = PagedKVCache(B, 256, Hkv, D, "cuda")
    assert cache2.append_rope(None, k.cuda(), v.cuda(), cos.cuda(), sin.cuda())[0] is None
    assert torch.equal(cache2.k_pages[:2], cache.k_pages[:2]) and torch.equal(cache2.v_pages[:2], cache.v_pages[:2])


def test_rope_append_rejects_bad_arguments(ops):
    k = torch.zeros((1, 64, 2, 128), dtype=torch.bfloat16, device="cuda")
    cos = torch.zeros((1, 64, 128), dtype=torch.bfloat16, device="cuda")
    pages = torch.zeros((4, 64, 2, 128), dtype=torch.bfloat16, device="cuda")
    view = ops.KvCacheView.from_paged(pages, pages.clone(), torch.arange(4, dtype=torch.int32, device="cuda").view(1, 4))
    with pytest.raises(RuntimeError, match="does not fit"):
        ops.rope_append(None, k, k, cos, cos, view, 256)
    with pytest.raises(ValueError, match="full head dimension"):
        ops.rope_append(None, k, k, cos[..., :64], cos[..., :64], view, 0)
    bad = torch.full((1, 4), 99, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.rope_append(None, k, k, cos, cos, ops.KvCacheView.from_paged(pages, pages.clone(), bad), 0, status=status)
    assert int(status.item()) & 2   # CA_STATUS_BAD_INDEX, nothing written out of range
