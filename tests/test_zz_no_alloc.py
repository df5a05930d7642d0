"""The allocation-free attention entry point (scratch inside the library image)
against the regular one.  Collected last on purpose: a run that stops at the
first failure has already executed every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


def _case(seed, bs, ctx_max, hq=16, hkv=8, block=32):
    g = torch.Generator(device=DEV).manual_seed(seed)
    ctx = torch.randint(block, ctx_max + 1, (bs,), generator=g, device=DEV, dtype=torch.int32)
    need = (ctx + 255) // 256
    pages = int(need.sum()) + 2
    perm = torch.randperm(pages, generator=g, device=DEV).int()
    table = torch.full((bs, int(need.max())), -1, dtype=torch.int32, device=DEV)
    at = 0
    for r in range(bs):
        n = int(need[r])
        table[r, :n] = perm[at:at + n]
        at += n
    kc = torch.randn(pages, 256, hkv, 128, generator=g, device=DEV).to(BF)
    vc = torch.randn(pages, 256, hkv, 128, generator=g, device=DEV).to(BF)
    q = torch.randn(bs, block, hq, 128, generator=g, device=DEV).to(BF)
    return q, kc, vc, ctx, table


def test_noalloc_attention_matches_regular_entry_twice(mdb):
    """Two calls in a row through the C ABI, different inputs each time: what
    the first call leaves in the shared scratch array must not leak into the
    second, and both must equal the workspace-taking entry point."""
    limit = mdb._lib.lib().mdb_attn_block_paged_noalloc_limit()
    assert limit == 8 << 20
    for seed, bs, nsplit in ((1, 2, 8), (2, 3, 5)):
        q, kc, vc, ctx, table = _case(seed, bs, 1500)
        want = mdb.ops.block_attn_with_kvcache(q, kc, vc, ctx, table, nsplit=nsplit)
        got = torch.full_like(q, float("nan"))
        before = torch.cuda.memory_allocated()
        mdb.ops.block_attn_with_kvcache_noalloc(q, kc, vc, ctx, table, got, nsplit=nsplit)
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max()
        assert err <= 2e-2, float(err)          # the tolerance of the attention tests
        assert torch.equal(got, want)           # same kernels, same order of operations
    assert mdb._lib.device_status(clear=True) == 0


def test_noalloc_attention_refuses_oversize(mdb):
    q, kc, vc, ctx, table = _case(3, 8, 600)
    out = torch.empty_like(q)
    # 8 requests x 32 splits x 16 heads x 32 rows x 520 B = 68 MB of partials: beyond the fixed array
    with pytest.raises(mdb._lib.MdbError, match="fixed scratch"):
        mdb.ops.block_attn_with_kvcache_noalloc(q, kc, vc, ctx, table, out, nsplit=32)
    # the same request with one split needs no scratch at all and goes through
    mdb.ops.block_attn_with_kvcache_noalloc(q, kc, vc, ctx, table, out, nsplit=1)
    want = mdb.ops.block_attn_with_kvcache(q, kc, vc, ctx, table, nsplit=1)
    assert torch.equal(out, want)


def test_noalloc_wrapper_checks_shapes_before_the_call(mdb):
    """The kernels hard-code head size 128, 256-token pages and a densely packed
    page-table row; a wrong ``out`` or head size has to stop on the host."""
    q, kc, vc, ctx, table = _case(4, 2, 600)
    with pytest.raises(ValueError, match="shape of q"):
        mdb.ops.block_attn_with_kvcache_noalloc(q, kc, vc, ctx, table, torch.empty_like(q)[:, :16].contiguous())
    with pytest.raises(ValueError, match="head_dim"):
        mdb.ops.block_attn_with_kvcache_noalloc(q[..., :64].contiguous(), kc, vc, ctx, table,
                                                torch.empty_like(q[..., :64].contiguous()))
    wide = torch.full((table.shape[0], 2 * table.shape[1]), -1, dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError, match="unit stride"):
        mdb.ops.block_attn_with_kvcache_noalloc(q, kc, vc, ctx, wide[:, ::2], torch.empty_like(q))
    with pytest.raises(ValueError, match="unit stride"):
        mdb.ops.block_attn_with_kvcache(q, kc, vc, ctx, wide[:, ::2])
