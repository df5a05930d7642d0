"""Per-kernel parity of the sm_100a path against the CPU oracle and the golden
fixtures.  Every test calls libmdb200 through its C ABI (via ops.py)."""
import math

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, load_golden, ulp_diff_bf16
from oracle import nano_oracle as orc

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


def _status_clean(mdb):
    assert mdb._lib.device_status(clear=True) == 0


def _close_bf16(got, want, exact_frac=0.995, max_ulp=1):
    """bf16 results that may differ by fp32 summation order only."""
    d = ulp_diff_bf16(got.cpu(), want.cpu())
    assert int(d.max()) <= max_ulp, f"max ulp {int(d.max())}"
    assert float((d == 0).float().mean()) >= exact_frac


def _close_gemm(got, exact):
    """bf16 GEMM output vs the exact fp32 product: half a bf16 step of rounding
    plus fp32 accumulation-order noise (absolute, relative to the output scale)."""
    got, exact = got.cpu().float(), exact.float()
    tol = exact.abs() * 2.0 ** -8 + 2e-4 * float(exact.std())
    bad = (got - exact).abs() > tol
    assert not bool(bad.any()), f"{int(bad.sum())} of {bad.numel()} outside tolerance, worst {float((got - exact).abs().max())}"
    assert float((got == exact.to(BF).float()).float().mean()) >= 0.97


# --------------------------------------------------------------------- KV commit
def test_kv_commit_bit_exact(mdb):
    g = torch.Generator().manual_seed(1)
    pages, hkv = 5, 8
    k = torch.randn(70, hkv, 128, generator=g).to(BF)
    v = torch.randn(70, hkv, 128, generator=g).to(BF)
    slots = torch.tensor(list(range(240, 275)) + [-1] * 3 + list(range(1000, 1032)), dtype=torch.int32)
    kc = torch.randn(pages, 256, hkv, 128, generator=g).to(BF)
    vc = torch.randn(pages, 256, hkv, 128, generator=g).to(BF)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    orc.store_kvcache(k, v, kc_ref, vc_ref, slots)
    kc_d, vc_d = kc.to(DEV), vc.to(DEV)
    mdb.ops.store_kvcache(k.to(DEV), v.to(DEV), kc_d, vc_d, slots.to(DEV))
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)
    # 4-D form with strided (sliced) sources, as the qkv split produces them
    qkv = torch.randn(64, (16 + 2 * hkv) * 128, generator=g).to(BF).to(DEV)
    k4 = qkv[:, 16 * 128:(16 + hkv) * 128].view(2, 32, hkv, 128)
    v4 = qkv[:, (16 + hkv) * 128:].view(2, 32, hkv, 128)
    slots4 = torch.arange(300, 364, dtype=torch.int32).view(2, 32)
    mdb.ops.store_kvcache(k4, v4, kc_d, vc_d, slots4.to(DEV))
    orc.store_kvcache(k4.cpu().reshape(-1, hkv, 128), v4.cpu().reshape(-1, hkv, 128), kc_ref, vc_ref, slots4)
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)
    _status_clean(mdb)


def test_kv_commit_golden_and_bad_slot(mdb):
    g = load_golden("layers.npz")
    kc = torch.zeros(3, 256, 2, 128, dtype=BF, device=DEV)
    vc = torch.zeros_like(kc)
    mdb.ops.store_kvcache(bf16_from_bits(g["kv_k"]).to(DEV), bf16_from_bits(g["kv_v"]).to(DEV), kc, vc,
                          torch.from_numpy(g["kv_slots"]).to(DEV))
    touched = g["kv_touched"].tolist()
    assert torch.equal(kc.cpu().view(-1, 256)[touched], bf16_from_bits(g["kv_kc_rows"]))
    assert torch.equal(vc.cpu().view(-1, 256)[touched], bf16_from_bits(g["kv_vc_rows"]))
    assert abs(float(kc.float().abs().sum()) - float(g["kv_kc_sum"])) < 1e-3
    _status_clean(mdb)
    # a slot outside the pool is skipped and reported, never written
    before = kc.clone()
    bad = torch.tensor([3 * 256 + 5, -1, 7], dtype=torch.int32, device=DEV)
    src = torch.ones(3, 2, 128, dtype=BF, device=DEV)
    mdb.ops.store_kvcache(src, src, kc, vc, bad)
    assert mdb._lib.device_status(clear=True) & 1
    before.view(-1, 256)[7] = 1
    assert torch.equal(kc, before)
    # empty input is a no-op
    mdb.ops.store_kvcache(src[:0], src[:0], kc, vc, bad[:0])


# --------------------------------------------------------------------- norms, rope, silu
def test_rmsnorm_forms(mdb):
    g = load_golden("layers.npz")
    w, x, res = (bf16_from_bits(g[k]).to(DEV) for k in ("norm_w", "x", "res"))
    y, r = mdb.ops.add_rms_norm(x, None, w, 1e-6)
    _close_bf16(y, bf16_from_bits(g["y_plain"]))
    assert torch.equal(r, x)
    y, r = mdb.ops.add_rms_norm(x, res, w, 1e-6)
    _close_bf16(y, bf16_from_bits(g["y_add"]))
    assert torch.equal(r.cpu(), bf16_from_bits(g["res_out"]))
    # split-k form: rows arrive as fp32 slices, are summed, rounded to bf16, then normalised
    gen = torch.Generator().manual_seed(3)
    parts = torch.randn(3, 40, 2048, generator=gen)
    res2 = torch.randn(40, 2048, generator=gen).to(BF)
    w2 = (1 + 0.1 * torch.randn(2048, generator=gen)).to(BF)
    xin = parts.sum(0).to(BF)
    want_y, want_r = orc.add_rms_norm(xin, res2, w2, 1e-6)
    y, r = mdb.ops.add_rms_norm(None, res2.to(DEV), w2.to(DEV), 1e-6, partials=parts.to(DEV))
    _close_bf16(y, want_y, exact_frac=0.99)
    _close_bf16(r, want_r, exact_frac=0.99)
    _status_clean(mdb)


@pytest.mark.parametrize("h", [256, 512, 2048, 1536])
def test_rmsnorm_many_rows(mdb, h):
    """Steps of more than 64 rows take the warp-per-row kernel (row widths 256..2048 in powers of two; 1536 stays
    on the row-per-CTA kernel): same arithmetic per element, only the order of the fp32 sum of squares differs."""
    gen = torch.Generator().manual_seed(11)
    m = 333                                      # not a multiple of the rows per CTA
    x = (3 * torch.randn(m, h, generator=gen)).to(BF)
    res = torch.randn(m, h, generator=gen).to(BF)
    w = (1 + 0.1 * torch.randn(h, generator=gen)).to(BF)
    want_y, want_r = orc.add_rms_norm(x, res, w, 1e-6)
    y, r = mdb.ops.add_rms_norm(x.to(DEV), res.to(DEV), w.to(DEV), 1e-6)
    _close_bf16(y, want_y, exact_frac=0.99)
    assert torch.equal(r.cpu(), want_r)
    y, r = mdb.ops.add_rms_norm(x.to(DEV), None, w.to(DEV), 1e-6)
    _close_bf16(y, orc.rms_norm(x, w, 1e-6), exact_frac=0.99)
    assert torch.equal(r.cpu(), x)
    _status_clean(mdb)


@pytest.mark.parametrize("from_partials", [False, True])
def test_qknorm_rope_commit(mdb, from_partials):
    gen = torch.Generator().manual_seed(4)
    m, hq, hkv = 37, 16, 8
    ncols = (hq + 2 * hkv) * 128
    if from_partials:
        parts = torch.randn(2, m, ncols, generator=gen)
        qkv = parts.sum(0).to(BF)
    else:
        qkv = torch.randn(m, ncols, generator=gen).to(BF)
    pos = torch.randint(0, 4000, (m,), generator=gen)
    qn = (1 + 0.1 * torch.randn(128, generator=gen)).to(BF)
    kn = (1 + 0.1 * torch.randn(128, generator=gen)).to(BF)
    table = orc.rope_table(4096, 128, 1e6)
    q, k, v = qkv.split([hq * 128, hkv * 128, hkv * 128], dim=-1)
    q = orc.apply_rope(orc.rms_norm(q.reshape(m, hq, 128), qn, 1e-6), pos, table)
    k = orc.apply_rope(orc.rms_norm(k.reshape(m, hkv, 128), kn, 1e-6), pos, table)
    v = v.reshape(m, hkv, 128)
    slots = torch.tensor([-1 if i % 9 == 0 else 250 + i for i in range(m)], dtype=torch.int32)
    kc = torch.zeros(3, 256, hkv, 128, dtype=BF)
    vc = torch.zeros_like(kc)
    orc.store_kvcache(k, v, kc, vc, slots)
    kc_d, vc_d = torch.zeros_like(kc, device=DEV), torch.zeros_like(vc, device=DEV)
    kw = dict(partials=parts.to(DEV)) if from_partials else {}
    q_d, k_d, v_d = mdb.ops.qknorm_rope_commit(None if from_partials else qkv.to(DEV), pos.to(DEV), table.to(DEV),
                                               qn.to(DEV), kn.to(DEV), 1e-6, hq, hkv, slots.to(DEV), kc_d, vc_d,
                                               want_kv=True, **kw)
    _close_bf16(q_d, q, exact_frac=0.99)
    _close_bf16(k_d, k, exact_frac=0.99)
    assert torch.equal(v_d.cpu(), v)
    _close_bf16(kc_d, kc, exact_frac=0.99)
    assert torch.equal(vc_d.cpu(), vc)
    _status_clean(mdb)


@pytest.mark.parametrize("m,hq,hkv,k", [(200, 4, 2, 256), (129, 3, 1, 128), (2048, 16, 8, 2048)])
def test_qkv_proj_rope_commit_fused(mdb, m, hq, hkv, k):
    """qkv projection with the norm / rotary / KV-store epilogue (tcgen05 tile
    GEMM, many rows) against the projection followed by the stand-alone kernel,
    and, for the small shapes, against the oracle.  129 rows and 5 heads leave a
    partial row tile and a half-empty column tile."""
    gen = torch.Generator().manual_seed(m + hq)
    n = (hq + 2 * hkv) * 128
    x = torch.randn(m, k, generator=gen).to(BF)
    w = (torch.randn(n, k, generator=gen) / k ** 0.5).to(BF)
    pos = torch.randint(0, 4000, (m,), generator=gen)
    qn = (1 + 0.1 * torch.randn(128, generator=gen)).to(BF)
    kn = (1 + 0.1 * torch.randn(128, generator=gen)).to(BF)
    table = orc.rope_table(4096, 128, 1e6)
    pages = (m + 300 + 255) // 256
    slots = torch.tensor([-1 if i % 9 == 0 else 250 + i for i in range(m)], dtype=torch.int32)
    args = (pos.to(DEV), table.to(DEV), qn.to(DEV), kn.to(DEV), 1e-6, hq, hkv, slots.to(DEV))

    def run(fused):
        kc = torch.zeros(pages, 256, hkv, 128, dtype=BF, device=DEV)
        vc = torch.zeros_like(kc)
        kb = torch.zeros(m, hkv, 128, dtype=BF, device=DEV)
        vb = torch.zeros_like(kb)
        if fused:
            q, _, _ = mdb.ops.qkv_proj_rope_commit(x.to(DEV), w.to(DEV), *args, kc, vc, k_out=kb, v_out=vb)
        else:
            qkv = mdb.ops.linear(x.to(DEV), w.to(DEV))
            q, _, _ = mdb.ops.qknorm_rope_commit(qkv, *args, kc, vc, k_out=kb, v_out=vb)
        return q, kb, vb, kc, vc

    got, ref = run(True), run(False)
    for g_t, r_t, name in zip(got, ref, ("q", "k", "v", "k_cache", "v_cache")):
        diff = (g_t.float() - r_t.float()).abs()
        # same bf16 projection; only the order of the 128-term sum of squares differs
        assert float(diff.max()) <= 4e-2, name
        assert float((diff == 0).float().mean()) >= 0.995, name
    assert torch.equal(got[2], ref[2]) and torch.equal(got[4], ref[4])       # v passes through untouched
    if m <= 256:
        qkv = orc.linear(x, w)
        q, kk, v = qkv.split([hq * 128, hkv * 128, hkv * 128], dim=-1)
        q = orc.apply_rope(orc.rms_norm(q.reshape(m, hq, 128), qn, 1e-6), pos, table)
        kk = orc.apply_rope(orc.rms_norm(kk.reshape(m, hkv, 128), kn, 1e-6), pos, table)
        assert float((got[0].cpu().float() - q.float()).abs().max()) <= 6e-2
        assert float((got[1].cpu().float() - kk.float()).abs().max()) <= 6e-2
        assert float((got[0].cpu().float() - q.float()).abs().mean()) <= 2e-3
    _status_clean(mdb)


def test_rope_golden(mdb):
    g = load_golden("layers.npz")
    q, k = bf16_from_bits(g["rope_q"]), bf16_from_bits(g["rope_k"])
    m, hq, hkv = q.shape[0], q.shape[1], k.shape[1]
    ones = torch.ones(128, dtype=BF, device=DEV)
    # feed already-normalised rows: with unit weights the norm rescales, so compare through the oracle instead
    qkv = torch.cat([q.reshape(m, -1), k.reshape(m, -1), torch.zeros(m, hkv * 128, dtype=BF)], dim=1)
    pos = torch.from_numpy(g["rope_pos"])
    table = orc.rope_table(4096, 128, 1e6)
    q_d, k_d, _ = mdb.ops.qknorm_rope_commit(qkv.to(DEV), pos.to(DEV), table.to(DEV), ones, ones, 1e-6, hq, hkv,
                                             want_kv=True)
    w1 = torch.ones(128, dtype=BF)
    _close_bf16(q_d, orc.apply_rope(orc.rms_norm(q, w1, 1e-6), pos, table), exact_frac=0.99)
    _close_bf16(k_d, orc.apply_rope(orc.rms_norm(k, w1, 1e-6), pos, table), exact_frac=0.99)


def test_silu_mul_and_gather(mdb):
    gen = torch.Generator().manual_seed(5)
    x = (2 * torch.randn(50, 2 * 512, generator=gen)).to(BF)
    out = mdb.ops.silu_and_mul(x.to(DEV))
    _close_bf16(out, orc.silu_mul(x), exact_frac=0.99)
    table = torch.randn(1000, 256, generator=gen).to(BF)
    ids = torch.randint(0, 1000, (77,), generator=gen)
    assert torch.equal(mdb.ops.gather_rows(table.to(DEV), ids.to(DEV)).cpu(), table[ids])
    _status_clean(mdb)
    ids[3] = 1000
    out = mdb.ops.gather_rows(table.to(DEV), ids.to(DEV)).cpu()
    assert mdb._lib.device_status(clear=True) & 4 and bool((out[3] == 0).all())


# --------------------------------------------------------------------- GEMMs
@pytest.mark.parametrize("m", [1, 16, 32, 33, 64, 65, 100, 177, 256])
@pytest.mark.parametrize("n,k", [(512, 256), (2048, 2048), (4096, 6144)])
def test_gemm_streaming(mdb, m, n, k):
    """Weight-streaming kernel (bf16 output up to 64 rows, split-k slices up to 256 rows: the accumulator row of a
    thread is then drained 64 columns at a time); more rows of ``linear`` run on the tile GEMM."""
    gen = torch.Generator().manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=gen).to(BF)
    w = (0.02 * torch.randn(n, k, generator=gen)).to(BF)
    exact = x.float() @ w.float().t()
    y = mdb.ops.linear(x.to(DEV), w.to(DEV))
    _close_gemm(y, exact)
    for ks in (1, 2, 4, mdb.ops.pick_ksplit(m, n, k)):
        if k // ks < 256:
            continue
        parts = mdb.ops.gemm_splitk_partials(x.to(DEV), w.to(DEV), ks)
        assert parts.shape[0] == ks
        got = parts.sum(0).cpu()
        assert (got - exact).abs().max() <= 2e-5 * k ** 0.5 + 1e-6 * exact.abs().max()
    _status_clean(mdb)


@pytest.mark.parametrize("m", [8, 32, 48])
def test_gemm_gateup_swiglu(mdb, m):
    gen = torch.Generator().manual_seed(m)
    k, inter = 512, 768
    x = torch.randn(m, k, generator=gen).to(BF)
    w = (0.05 * torch.randn(2 * inter, k, generator=gen)).to(BF)
    want = orc.silu_mul(orc.linear(x, w))
    got = mdb.ops.gateup_swiglu(x.to(DEV), w.to(DEV)).cpu()
    # a one-step difference of the bf16 gate or up value moves the product by up to two steps
    tol = want.float().abs() * 2.0 ** -6 + 1e-3 * float(want.float().std())
    assert bool(((got.float() - want.float()).abs() <= tol).all())
    assert float((got == want).float().mean()) >= 0.95


@pytest.mark.parametrize("m", [65, 300])
def test_gemm_gateup_swiglu_many_rows(mdb, m):
    gen = torch.Generator().manual_seed(m)
    k, inter = 512, 768
    x = torch.randn(m, k, generator=gen).to(BF)
    w = (0.05 * torch.randn(2 * inter, k, generator=gen)).to(BF)
    want = orc.silu_mul(orc.linear(x, w))
    got = mdb.ops.gateup_swiglu(x.to(DEV), w.to(DEV)).cpu()
    tol = want.float().abs() * 2.0 ** -6 + 1e-3 * float(want.float().std())
    assert bool(((got.float() - want.float()).abs() <= tol).all())
    assert float((got == want).float().mean()) >= 0.95
    assert mdb._lib.device_status(clear=True) == 0


@pytest.mark.parametrize("m,n,k", [(65, 384, 256), (200, 4096, 2048), (1088, 2048, 6144), (129, 136, 64),
                                   (2048, 4096, 2048), (20, 136, 64),
                                   # few tiles: clusters of 8 / 4 / 2 CTAs split k and add their partial tiles
                                   (256, 2048, 2048), (512, 2048, 6144), (1024, 2048, 2048), (300, 520, 2048),
                                   (70, 136, 1024), (129, 2048, 2048), (257, 2048, 6144), (1100, 2048, 2048),
                                   (640, 4096, 1024)])
def test_gemm_tile_kernel(mdb, m, n, k):
    gen = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, k, generator=gen).to(BF)
    w = (0.02 * torch.randn(n, k, generator=gen)).to(BF)
    y = mdb.ops.linear(x.to(DEV), w.to(DEV))
    _close_gemm(y, x.float() @ w.float().t())
    # linearity: scaling x by 2 scales y by exactly 2
    y2 = mdb.ops.linear((x * 2).to(DEV), w.to(DEV))
    assert torch.equal(y2.float(), y.float() * 2)


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 520, 128), (512, 640, 128), (1088, 2048, 512), (2048, 4096, 2048)])
def test_gemm_cta_pair_matches_single_cta(mdb, m, n, k):
    """Steps of 256 rows and more run on pairs of CTAs (tcgen05.mma.cta_group::2, tiles of 256 x 256).
    Same products, same accumulation order: every epilogue must give the single-CTA kernel's bits
    (bf16 store, SiLU*mul, qkv + norm + rotary + KV store, LM head + sampler records), including
    partial row and column tiles."""
    gen = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, k, generator=gen).to(BF).to(DEV)
    w = (torch.randn(n, k, generator=gen) / k ** 0.5).to(BF).to(DEV)
    res = {}
    for pair in (0, 2):
        mdb.ops.set_option(mdb.ops.OPT_GEMM_PAIR, pair)
        out = [mdb.ops.linear(x, w)]
        if n % 256 == 0:
            out.append(mdb.ops.gateup_swiglu(x, w))
        if n % 128 == 0 and n >= 384:
            hq, hkv = n // 128 - 2, 1
            pos = torch.arange(m, device=DEV) % 1000
            table = orc.rope_table(1024, 128, 1e6).to(DEV)
            ones = torch.ones(128, dtype=BF, device=DEV)
            slots = torch.arange(m, dtype=torch.int32, device=DEV)
            kc = torch.zeros((m + 255) // 256, 256, hkv, 128, dtype=BF, device=DEV)
            vc = torch.zeros_like(kc)
            q, _, _ = mdb.ops.qkv_proj_rope_commit(x, w, pos, table, ones, ones, 1e-6, hq, hkv, slots, kc, vc)
            out += [q, kc, vc]
        temps = torch.ones(1, device=DEV)
        x0, conf = mdb.ops.lm_head_sample(x, w, temps, m, seed=7, step=1)
        out += [x0, conf]
        res[pair] = out
    mdb.ops.set_option(mdb.ops.OPT_GEMM_PAIR, 1)
    # the plain projection of the single-CTA form may split k over a cluster (few tiles), which changes the
    # order of the fp32 sum: compared with the exact product instead; every other epilogue bit for bit
    for a_t, b_t in zip(res[0][1:], res[2][1:]):
        assert torch.equal(a_t, b_t)
    _close_gemm(res[0][0], x.cpu().float() @ w.cpu().float().t())
    _close_gemm(res[2][0], x.cpu().float() @ w.cpu().float().t())
    _status_clean(mdb)


def test_gemm_activation_band_order(mdb):
    """A step whose activations outgrow L2 (16384 rows x 6144: 201 MB) walks its tiles one activation band
    after the other instead of one weight tile after the other; same products, checked against an fp32
    matmul on the device (the CPU oracle would need minutes)."""
    gen = torch.Generator(device=DEV).manual_seed(3)
    m, n, k = 16384, 2048, 6144
    x = torch.randn(m, k, generator=gen, device=DEV).to(BF)
    w = (torch.randn(n, k, generator=gen, device=DEV) / k ** 0.5).to(BF)
    got = mdb.ops.linear(x, w)
    for r0 in (0, 5120, m - 1024):           # three 1024-row bands: first, middle, last
        exact = x[r0:r0 + 1024].float() @ w.float().t()
        _close_gemm(got[r0:r0 + 1024], exact.cpu())
    _status_clean(mdb)


def test_gemm_rejects_bad_arguments(mdb):
    x = torch.zeros(4, 100, dtype=BF, device=DEV)
    w = torch.zeros(64, 100, dtype=BF, device=DEV)
    with pytest.raises(mdb._lib.MdbError):
        mdb.ops.linear(x, w)            # k not a multiple of 32
    with pytest.raises(TypeError):
        mdb.ops.linear(x.float(), w)
    with pytest.raises(RuntimeError):
        mdb.ops.linear(x.cpu(), w.cpu())


# --------------------------------------------------------------------- block attention over the paged cache
def _paged_case(seed, bs, block, hq, hkv, prefix_lens, pages_extra=3, poison=False):
    gen = torch.Generator().manual_seed(seed)
    ctx = [p + block if p >= 0 else 0 for p in prefix_lens]
    need = [(c + 255) // 256 for c in ctx]
    num_pages = sum(need) + pages_extra
    perm = torch.randperm(num_pages, generator=gen).tolist()
    width = max(max(need), 1)
    table = torch.full((bs, width), -1, dtype=torch.int32)
    kc = torch.zeros(num_pages, 256, hkv, 128, dtype=BF)
    vc = torch.zeros_like(kc)
    if poison:      # slots no context covers hold what uninitialised memory may hold
        kc.fill_(float("nan"))
        vc.fill_(float("inf"))
    at = 0
    for r in range(bs):
        for j in range(need[r]):
            table[r, j] = perm[at]
            at += 1
        if ctx[r] > 0:
            k = torch.randn(ctx[r], hkv, 128, generator=gen).to(BF)
            v = torch.randn(ctx[r], hkv, 128, generator=gen).to(BF)
            slots = torch.tensor(orc.get_slots(table[r, :need[r]].tolist(), 0, ctx[r]), dtype=torch.int32)
            orc.store_kvcache(k, v, kc, vc, slots)
    q = torch.randn(bs, block, hq, 128, generator=gen).to(BF)
    return q, kc, vc, torch.tensor(ctx, dtype=torch.int32), table


@pytest.mark.parametrize("hq,hkv", [(16, 2), (16, 8), (8, 4), (4, 4)])
@pytest.mark.parametrize("nsplit", [1, 3, 16])
def test_attn_paged_config1(mdb, hq, hkv, nsplit):
    """BASELINE config 1 (decode form): batch 4, prefix lengths uniform in
    [256, 2048] (seed 1), block 32, head_dim 128, 256-token pages in a
    permuted page table."""
    gen = torch.Generator().manual_seed(1)
    prefix = torch.randint(256, 2049, (4,), generator=gen).tolist()
    q, kc, vc, ctx, table = _paged_case(1, 4, 32, hq, hkv, prefix)
    want = orc.attn_paged(q, kc, vc, ctx, table, 128 ** -0.5, round_p=False)
    got = mdb.ops.block_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), ctx.to(DEV), table.to(DEV),
                                          nsplit=nsplit).cpu()
    err = (got.float() - want.float()).abs().max()
    assert err <= 2e-2, f"max-abs {float(err)}"      # north-star tolerance; typical value is ~2e-3
    assert (got.float() - want.float()).abs().mean() <= 5e-4
    _status_clean(mdb)


@pytest.mark.parametrize("block", [8, 16, 32, 64])
def test_attn_paged_edges(mdb, block):
    # prefix 0 (context = the block only), a request with context 0 (padding row), page-straddling lengths,
    # contexts that end inside a key tile with NaN / Inf in the cache slots behind them
    prefix = [0, -1, 250, 513, 1000, 128 - block, 256 - block]
    q, kc, vc, ctx, table = _paged_case(7, len(prefix), block, 16, 8, prefix, poison=True)
    want = orc.attn_paged(q, kc, vc, ctx, table, 128 ** -0.5)
    for nsplit in (1, 4):
        got = mdb.ops.block_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), ctx.to(DEV), table.to(DEV),
                                              nsplit=nsplit).cpu()
        assert (got.float() - want.float()).abs().max() <= 2e-2
        assert bool((got[1] == 0).all())
    _status_clean(mdb)


def test_attn_paged_properties_at_full_size(mdb):
    """BASELINE config 3 shape (64 requests, contexts up to ~6K, 8 KV heads):
    too big for the CPU oracle, checked through invariants instead."""
    gen = torch.Generator(device=DEV).manual_seed(3)
    bs, block, hq, hkv = 64, 32, 16, 8
    cg = torch.Generator().manual_seed(3)
    ctx = (torch.randint(512, 4097, (bs,), generator=cg) + torch.randint(0, 2049, (bs,), generator=cg) // 32 * 32 + 32)
    need = (ctx + 255) // 256
    num_pages = int(need.sum())
    width = int(need.max())
    perm = torch.randperm(num_pages, generator=cg)
    table = torch.full((bs, width), -1, dtype=torch.int32)
    at = 0
    for r in range(bs):
        table[r, :need[r]] = perm[at:at + need[r]].int()
        at += int(need[r])
    kc = torch.randn(num_pages, 256, hkv, 128, generator=gen, device=DEV, dtype=torch.float32).to(BF)
    vc = torch.randn(num_pages, 256, hkv, 128, generator=gen, device=DEV, dtype=torch.float32).to(BF)
    q = torch.randn(bs, block, hq, 128, generator=gen, device=DEV, dtype=torch.float32).to(BF)
    ctx_d, table_d = ctx.int().to(DEV), table.to(DEV)
    base = mdb.ops.block_attn_with_kvcache(q, kc, vc, ctx_d, table_d, nsplit=1)
    # (1) doubling V doubles the output exactly
    dbl = mdb.ops.block_attn_with_kvcache(q, kc, vc * 2, ctx_d, table_d, nsplit=1)
    assert torch.equal(dbl.float(), base.float() * 2)
    # (2) relocating pages (same logical keys, other physical pages) changes nothing
    perm2 = torch.randperm(num_pages, generator=cg).to(DEV)
    inv = torch.empty_like(perm2)
    inv[perm2] = torch.arange(num_pages, device=DEV)
    kc2, vc2 = kc[perm2], vc[perm2]                      # new page p holds old page perm2[p]
    table2 = torch.where(table_d >= 0, inv[table_d.clamp(min=0).long()].int(), table_d)
    moved = mdb.ops.block_attn_with_kvcache(q, kc2, vc2, ctx_d, table2, nsplit=1)
    assert torch.equal(moved, base)
    # (3) cutting the key range into parts only changes fp32 summation order
    split = mdb.ops.block_attn_with_kvcache(q, kc, vc, ctx_d, table_d, nsplit=5)
    assert (split.float() - base.float()).abs().max() <= 4e-3
    # (4) one request against the oracle
    r = int(ctx.argmin())
    want = orc.attn_paged(q[r:r + 1].cpu(), kc.cpu(), vc.cpu(), ctx[r:r + 1].int(), table[r:r + 1], 128 ** -0.5)
    assert (base[r].cpu().float() - want[0].float()).abs().max() <= 2e-2
    _status_clean(mdb)


# --------------------------------------------------------------------- staircase prefill attention
@pytest.mark.parametrize("stairs", [8, 32])
@pytest.mark.parametrize("hq,hkv", [(16, 2), (4, 2), (4, 4), (6, 2)])
def test_attn_staircase_vs_oracle(mdb, stairs, hq, hkv):
    gen = torch.Generator().manual_seed(stairs + hq)
    lens = [288 + 5, 32, 1, 700, 95]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    n = int(cu[-1])
    q = torch.randn(n, hq, 128, generator=gen).to(BF)
    k = torch.randn(n, hkv, 128, generator=gen).to(BF)
    v = torch.randn(n, hkv, 128, generator=gen).to(BF)
    want = orc.attn_staircase_varlen(q, k, v, cu, cu, stairs, mirror_rounding=True)
    got = mdb.ops.sparse_attn_varlen(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), cu.to(DEV), stairs).cpu()
    err = (got.float() - want.float()).abs()
    assert err.max() <= 2e-2 and err.mean() <= 5e-4, (float(err.max()), float(err.mean()))
    _status_clean(mdb)


def test_attn_staircase_config1_and_golden(mdb):
    """BASELINE config 1 prefill form (every row of prefix+block is a query)
    and the reference Triton kernel's own fp32 outputs."""
    gen = torch.Generator().manual_seed(1)
    lens = (torch.randint(256, 2049, (4,), generator=gen) + 32).tolist()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    n = int(cu[-1])
    q = torch.randn(n, 16, 128, generator=gen).to(BF)
    k = torch.randn(n, 2, 128, generator=gen).to(BF)
    v = torch.randn(n, 2, 128, generator=gen).to(BF)
    want = orc.attn_staircase_varlen(q, k, v, cu, cu, 32, mirror_rounding=True)
    got = mdb.ops.sparse_attn_varlen(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), cu.to(DEV), 32).cpu()
    assert (got.float() - want.float()).abs().max() <= 2e-2
    g = load_golden("staircase.npz")
    lens = g["lens"].tolist()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    q, k, v = (torch.from_numpy(g[x]).to(BF) for x in ("q", "k", "v"))
    for stairs in (32, 8):
        got = mdb.ops.sparse_attn_varlen(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), cu.to(DEV), stairs).cpu()
        ref = torch.from_numpy(g[f"out_fp32_s{stairs}"])       # fp32 kernel on fp16-rounded inputs
        assert (got.float() - ref).abs().max() <= 3e-2         # includes rounding the fp16 inputs to bf16
    # inputs that bf16 holds exactly: the kernel's own fp32 run on the same values, at the 2e-2 bar
    lens = g["lens_bf"].tolist()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).to(DEV)
    q, k, v = (bf16_from_bits(g[x]).to(DEV) for x in ("q_bf", "k_bf", "v_bf"))
    for stairs in (32, 8):
        got = mdb.ops.sparse_attn_varlen(q, k, v, cu, cu, stairs).cpu()
        err = float((got.float() - torch.from_numpy(g[f"out_fp32_bf_s{stairs}"])).abs().max())
        print(f"staircase kernel vs the Triton kernel in fp32, bf16-exact inputs, stairs {stairs}: max-abs {err:.5f}")
        assert err <= 2e-2


def test_attn_staircase_long_sequences(mdb):
    """Prefill shapes too long for the CPU oracle as a whole (the decoder's 16 query / 8 KV heads, sequences
    up to 3001 tokens, lengths around the 128-key tile edges): every sequence of up to 257 tokens against the
    oracle, and for the long ones two invariants -- a sequence's rows do not depend on what else is packed
    with it, and the rows of the first stairs do not depend on the tokens behind them (block causality)."""
    gen = torch.Generator(device=DEV).manual_seed(11)
    lens = [1, 31, 32, 33, 127, 128, 129, 1000, 3001, 257]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    n = int(cu[-1])
    q = torch.randn(n, 16, 128, generator=gen, device=DEV).to(BF)
    k = torch.randn(n, 8, 128, generator=gen, device=DEV).to(BF)
    v = torch.randn(n, 8, 128, generator=gen, device=DEV).to(BF)
    out = mdb.ops.sparse_attn_varlen(q, k, v, cu.to(DEV), cu.to(DEV), 32)
    for i, t in enumerate(lens):
        a, b = int(cu[i]), int(cu[i + 1])
        one = torch.tensor([0, t], dtype=torch.int32)
        if t <= 257:
            want = orc.attn_staircase_varlen(q[a:b].cpu(), k[a:b].cpu(), v[a:b].cpu(), one, one, 32, mirror_rounding=True)
            assert float((out[a:b].cpu().float() - want.float()).abs().max()) <= 2e-2, t
        else:
            alone = mdb.ops.sparse_attn_varlen(q[a:b].contiguous(), k[a:b].contiguous(), v[a:b].contiguous(),
                                               one.to(DEV), one.to(DEV), 32)
            assert torch.equal(alone, out[a:b])
            # right-aligned stairs: with T' = T - 32 * j the stair edges stay where they are, so the first
            # T' rows of the long sequence equal the rows of its T'-token prefix run on its own
            tp = t - 32 * 7
            cut = torch.tensor([0, tp], dtype=torch.int32).to(DEV)
            head = mdb.ops.sparse_attn_varlen(q[a:a + tp].contiguous(), k[a:a + tp].contiguous(),
                                              v[a:a + tp].contiguous(), cut, cut, 32)
            # (the lazy running maximum is shared by the rows of a warp, so only fp32 rounding may differ)
            assert float((head.float() - out[a:a + tp].float()).abs().max()) <= 4e-3
    # the tail of the 1000-token sequence against the oracle (its last 64 rows see every key)
    a, b = int(cu[7]), int(cu[8])
    one = torch.tensor([0, b - a], dtype=torch.int32)
    want = orc.attn_staircase_varlen(q[a:b].cpu(), k[a:b].cpu(), v[a:b].cpu(), one, one, 32, mirror_rounding=True)
    assert float((out[a:b].cpu().float() - want.float()).abs().max()) <= 2e-2
    _status_clean(mdb)


# --------------------------------------------------------------------- LM head + sampler
def test_logits_sample_golden(mdb):
    """Sampler statistics and the unmask rule on the reference's own cases."""
    g = load_golden("sampler.npz")
    mask_id, thr = int(g["mask_id"]), float(g["threshold"])
    for case in range(3):
        p = f"c{case}_"
        logits = bf16_from_bits(g[p + "logits"])
        bs, b, v = logits.shape
        temps = torch.full((bs,), float(g[p + "temp"]))
        noise = torch.from_numpy(g[p + "gumbel"]).reshape(bs * b, v).contiguous()
        x0, conf = mdb.ops.logits_sample(logits.reshape(bs * b, v).to(DEV), temps.to(DEV), b, noise=noise.to(DEV))
        assert torch.equal(x0.cpu().long().view(bs, b), torch.from_numpy(g[p + "x0"]))
        assert torch.allclose(conf.cpu().view(bs, b), torch.from_numpy(g[p + "x0_p"]), rtol=1e-4)
        blocks = torch.from_numpy(g[p + "before"]).to(DEV)
        transfer, counts = mdb.ops.unmask_decide(blocks, x0, conf, mask_id, thr)
        assert torch.equal(blocks.cpu(), torch.from_numpy(g[p + "after"]))
        assert torch.equal(transfer.cpu().bool(), torch.from_numpy(g[p + "transfer"]))
        assert int(counts.sum()) == int(g[p + "count"])


@pytest.mark.parametrize("m,block,v", [(32, 32, 4096), (64, 32, 4096), (16, 8, 4096), (128, 32, 4096),
                                       (320, 32, 4096), (160, 32, 1000)])
@pytest.mark.parametrize("mode", ["none", "explicit", "counter"])
def test_lmhead_sample(mdb, m, block, v, mode):
    """Short steps: weight-streaming kernel with the sampler in the epilogue.
    Many rows (m > 64): the tcgen05 tile GEMM with the sampler epilogue, also
    with a partial last row tile (320) and a partial last vocabulary tile
    (1000); explicit noise arrays go through materialised logits."""
    gen = torch.Generator().manual_seed(m)
    h = 256
    hidden = torch.randn(m, h, generator=gen).to(BF)
    w = (0.05 * torch.randn(v, h, generator=gen)).to(BF)
    temps = torch.tensor([1.0, 0.5, 0.2, 2.0] * (m // block))[:m // block].contiguous()
    kw, noise = {}, None
    if mode == "explicit":
        noise = -torch.empty(m, v).exponential_(generator=gen).log()
        kw["noise"] = noise.to(DEV)
    elif mode == "counter":
        kw.update(seed=1234, step=7)
        noise = mdb.ops.gumbel_noise(m, v, 1234, 7, DEV).cpu()
    x0, conf = mdb.ops.lm_head_sample(hidden.to(DEV), w.to(DEV), temps.to(DEV), block, **kw)
    logits = orc.linear(hidden, w).view(m // block, block, v)
    nz = None if noise is None else noise.view(m // block, block, v)
    want_x0, want_p = orc.sampler_prepare(logits, temps.view(-1, 1), nz)
    want_x0, want_p = want_x0.view(-1), want_p.view(-1)
    got = x0.cpu().long()
    agree = got == want_x0
    # a disagreement is only acceptable where the two candidates are within one bf16 step of a tie
    lf = logits.float().view(m, v) / temps.repeat_interleave(block).view(m, 1)
    noisy = lf if noise is None else lf + noise
    for i in (~agree).nonzero().flatten().tolist():
        assert abs(float(noisy[i, got[i]] - noisy[i, want_x0[i]])) <= 0.04 / float(temps[i // block])
    assert float(agree.float().mean()) >= 0.9
    assert torch.allclose(conf.cpu()[agree], want_p[agree], rtol=3e-2)
    _status_clean(mdb)


def test_gumbel_noise_distribution(mdb):
    z = mdb.ops.gumbel_noise(64, 8192, 99, 3, DEV).double()
    assert abs(float(z.mean()) - 0.5772) < 0.01
    assert abs(float(z.var()) - math.pi ** 2 / 6) < 0.03
    z2 = mdb.ops.gumbel_noise(64, 8192, 99, 4, DEV).double()
    assert abs(float(((z - z.mean()) * (z2 - z2.mean())).mean())) < 0.01      # steps are independent streams
    assert torch.equal(mdb.ops.gumbel_noise(64, 8192, 99, 3, DEV).double(), z)  # and reproducible


def test_unmask_decide_vs_oracle(mdb):
    gen = torch.Generator().manual_seed(8)
    for block in (8, 32, 64):
        bs, mask_id = 40, 151669
        blocks = torch.randint(0, 1000, (bs, block), generator=gen)
        blocks[torch.rand(bs, block, generator=gen) < 0.6] = mask_id
        blocks[0] = 5                      # nothing masked
        blocks[1] = mask_id                # everything masked
        conf = torch.rand(bs, block, generator=gen)
        conf[2] = 0.5                      # exact ties: lowest index wins
        conf[3, :] = 0.95                  # all above threshold
        x0 = torch.randint(0, 1000, (bs, block), generator=gen)
        want, want_t = orc.unmask_decision(blocks, x0, conf, mask_id, 0.9)
        d_blocks = blocks.to(DEV)
        t, counts = mdb.ops.unmask_decide(d_blocks, x0.int().to(DEV).view(-1), conf.to(DEV).view(-1), mask_id, 0.9)
        assert torch.equal(d_blocks.cpu(), want)
        assert torch.equal(t.cpu().bool(), want_t)
        assert torch.equal(counts.cpu().long(), want_t.sum(1))


def test_unmask_decide_hf_twin_quota(mdb):
    """Per-request quotas: the HF twin's ``_select_transfer_index`` on its own fixture
    (mineru_diffusion/modeling_mineru_diffusion.py:518-532) and the quota schedule helper."""
    g = load_golden("hf_twin.npz")
    for b, steps in g["sched_pairs"].tolist():
        assert mdb.ops.num_transfer_tokens(b, steps) == g[f"sched_{b}_{steps}"].tolist()
    thr, mask_id = float(g["threshold"]), 151669
    for i in range(int(g["num_cases"])):
        conf = torch.from_numpy(g[f"q{i}_conf"])
        masked = torch.from_numpy(g[f"q{i}_masked"])
        count = int(g[f"q{i}_count"])
        bs, block = conf.shape
        blocks = torch.where(masked, torch.full(masked.shape, mask_id, dtype=torch.int64),
                             torch.zeros(masked.shape, dtype=torch.int64))
        x0 = (torch.arange(conf.numel(), dtype=torch.int32) + 1).view(conf.shape)
        d_blocks = blocks.to(DEV)
        quotas = torch.full((bs,), count, dtype=torch.int32, device=DEV)
        t, counts = mdb.ops.unmask_decide(d_blocks, x0.to(DEV).view(-1), conf.to(DEV).view(-1), mask_id, thr,
                                          quotas=quotas)
        want = torch.from_numpy(g[f"q{i}_transfer"])
        assert torch.equal(t.cpu().bool(), want), i
        assert torch.equal(counts.cpu().long(), want.sum(1))
        assert torch.equal(d_blocks.cpu()[want], x0.long()[want])
        # the same quota as one scalar for the whole batch
        d2 = blocks.to(DEV)
        t2, _ = mdb.ops.unmask_decide(d2, x0.to(DEV).view(-1), conf.to(DEV).view(-1), mask_id, thr, quota=count)
        assert torch.equal(t2, t)
    # a quota of 0 (more steps than tokens) leaves only the threshold branch; fewer masked than the quota: all go
    conf = torch.tensor([[0.5, 0.95, 0.2, 0.1], [0.5, 0.6, 0.2, 0.1]])
    blocks = torch.full((2, 4), mask_id, dtype=torch.int64)
    blocks[1, 0] = 3
    x0 = torch.arange(8, dtype=torch.int32) + 100
    d = blocks.to(DEV)
    t, c = mdb.ops.unmask_decide(d, x0.to(DEV), conf.to(DEV).view(-1), mask_id, thr,
                                 quotas=torch.tensor([0, 7], dtype=torch.int32, device=DEV))
    assert t.cpu().tolist() == [[0, 1, 0, 0], [0, 1, 1, 1]] and c.cpu().tolist() == [1, 3]
    _status_clean(mdb)


def test_unmask_decide_hands_over_status_word(mdb):
    """The last kernel of a step copies the device status word next to its results and clears it."""
    kc = torch.zeros(1, 256, 2, 128, dtype=BF, device=DEV)
    src = torch.ones(1, 2, 128, dtype=BF, device=DEV)
    mdb.ops.store_kvcache(src, src, kc, kc.clone(), torch.tensor([999999], dtype=torch.int32, device=DEV))   # bad slot
    blocks = torch.full((1, 32), 7, dtype=torch.int64, device=DEV)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    mdb.ops.unmask_decide(blocks, torch.zeros(32, dtype=torch.int32, device=DEV), torch.zeros(32, device=DEV), 9, 0.9,
                          status_out=word)
    assert int(word.item()) == 1
    assert mdb._lib.device_status(clear=True) == 0


def test_attn_paged_context_beyond_page_table(mdb):
    """A context length the page-table row cannot address (device data the host never validates): the kernel
    cuts it to the row, raises MDB_STATUS_BAD_PAGE and never reads the table past the request's row; so does a
    page id outside the pool.  Outputs stay finite."""
    q, kc, vc, ctx, table = _paged_case(5, 3, 32, 16, 8, [200, 480, 300])
    assert table.shape[1] == 2
    bad_ctx = ctx.clone()
    bad_ctx[2] = 2 * 256 + 40                      # the last request: one tile past its (and the buffer's) last row
    got = mdb.ops.block_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), bad_ctx.to(DEV), table.to(DEV), nsplit=1)
    assert mdb._lib.device_status(clear=True) & 2
    assert bool(torch.isfinite(got.float()).all())
    want = orc.attn_paged(q, kc, vc, ctx, table, 128 ** -0.5)
    assert (got[:2].cpu().float() - want[:2].float()).abs().max() <= 2e-2      # the other requests are untouched
    bad_table = table.clone()
    bad_table[1, 1] = kc.shape[0] + 3
    got = mdb.ops.block_attn_with_kvcache(q.to(DEV), kc.to(DEV), vc.to(DEV), ctx.to(DEV), bad_table.to(DEV), nsplit=2)
    assert mdb._lib.device_status(clear=True) & 2
    assert bool(torch.isfinite(got.float()).all())


def test_bounded_wait_runs_out(mdb):
    """The error contract of the in-kernel waits: a consumer that waits for flag slots nobody raises gives up
    after the wait limit, the call returns, the kernel finishes, and MDB_STATUS_WAIT_TIMEOUT (bit 16) is set --
    and cleared by reading it.  One GPU, no peer: the slots are plain local memory that stays zero."""
    lib = mdb._lib.lib()
    old = mdb.ops.get_option(mdb.ops.OPT_WAIT_LIMIT_US)
    mdb.ops.set_option(mdb.ops.OPT_WAIT_LIMIT_US, 2000)          # 2 ms instead of 2 s
    try:
        m, h = 8, 256
        parts = torch.zeros(2, m, h, device=DEV)
        res = torch.zeros(m, h, dtype=BF, device=DEV)
        w = torch.ones(h, dtype=BF, device=DEV)
        y, r = torch.empty_like(res), torch.empty_like(res)
        flags = torch.zeros(4, dtype=torch.int32, device=DEV)    # never raised
        epoch = torch.ones(1, dtype=torch.int32, device=DEV)
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        mdb._lib.check(lib.mdb_add_rmsnorm_tp(None, parts.data_ptr(), 2, res.data_ptr(), w.data_ptr(), 1e-6,
                                              y.data_ptr(), r.data_ptr(), m, h, flags.data_ptr(), 4, 5,
                                              epoch.data_ptr(), torch.cuda.current_stream().cuda_stream),
                       "mdb_add_rmsnorm_tp")
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0                       # gave up after ~2 ms, not 2 s
        assert mdb._lib.device_status(clear=False) & 16
        assert mdb._lib.device_status(clear=True) & 16
        assert mdb._lib.device_status(clear=True) == 0
        assert bool((y == 0).all())                              # the kernel still wrote its rows
        # raised slots: no wait, no status
        flags.fill_(1 * 256 + 5)
        mdb._lib.check(lib.mdb_add_rmsnorm_tp(None, parts.data_ptr(), 2, res.data_ptr(), w.data_ptr(), 1e-6,
                                              y.data_ptr(), r.data_ptr(), m, h, flags.data_ptr(), 4, 5,
                                              epoch.data_ptr(), torch.cuda.current_stream().cuda_stream),
                       "mdb_add_rmsnorm_tp")
        assert mdb._lib.device_status(clear=True) == 0
    finally:
        mdb.ops.set_option(mdb.ops.OPT_WAIT_LIMIT_US, old)


@pytest.mark.parametrize("m", [32, 256])
def test_lmhead_sample_full_vocabulary(mdb, m):
    """The LM head at the decoder's own size (hidden 2048, vocabulary 151936) on identical inputs: a short
    step (weight-streaming kernel) and a many-row step (tile GEMM with the sampler epilogue).  Sampled tokens
    and confidences against the oracle's ``F.linear`` + ``Sampler.prepare``; a differing token must be a tie
    within one bf16 step of the logits."""
    gen = torch.Generator().manual_seed(m)
    h, v, block = 2048, 151936, 32
    hidden = torch.randn(m, h, generator=gen).to(BF)
    w = (0.02 * torch.randn(v, h, generator=gen)).to(BF)
    temps = torch.tensor([1.0, 0.3] * (m // block // 2) + [1.0] * (m // block % 2))
    noise = mdb.ops.gumbel_noise(m, v, 77, 3, DEV).cpu()
    x0, conf = mdb.ops.lm_head_sample(hidden.to(DEV), w.to(DEV), temps.to(DEV), block, seed=77, step=3)
    logits = orc.linear(hidden, w).view(m // block, block, v)
    want_x0, want_p = orc.sampler_prepare(logits, temps.view(-1, 1), noise.view(m // block, block, v))
    want_x0, want_p = want_x0.view(-1), want_p.view(-1)
    got = x0.cpu().long()
    agree = got == want_x0
    lf = logits.float().view(m, v) / temps.repeat_interleave(block).view(m, 1)
    noisy = lf + noise
    for i in (~agree).nonzero().flatten().tolist():
        assert abs(float(noisy[i, got[i]] - noisy[i, want_x0[i]])) <= 0.04 / float(temps[i // block])
    assert float(agree.float().mean()) >= 0.95
    # one bf16 step of the sampled token's logit (2^-5 at |logit| in [4, 8)) moves its probability by e^(step / T)
    row_t = temps.repeat_interleave(block)[agree]
    rel = (conf.cpu()[agree] - want_p[agree]).abs() / want_p[agree]
    assert bool((rel <= torch.expm1(0.03125 / row_t) + 2e-3).all()), float(rel.max())
    _status_clean(mdb)
