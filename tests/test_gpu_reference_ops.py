"""Second opinion on the GPU for the third-party calls of the reference that cannot run on a CPU in bf16.

The reference reaches flash-attn (``flash_attn_with_kvcache``, call site
``nanovllm/layers/sdar_attention.py:50-55``) and liger-kernel (``LigerSiLUMulFunction``, call site
``nanovllm/layers/activation.py:12-15``) through pip wheels that are not part of its sources; the CPU oracle
restates both.  Where the wheels installed next to this repository run on the device at hand, the CUDA
kernels of this repository are compared with the very calls the reference makes; where they do not import
or their first call raises, the test is skipped with the error text and the restatement stays the only pin.
The library calls are also timed (CUDA events) as the "library through torch" bar for the same inputs.
"""
import pytest
import torch

from conftest import record_parity
from oracle import nano_oracle as orc

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


_record = record_parity


def _time_us(fn, reps=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def _config1(hkv=2):
    """BASELINE config 1, decode form: batch 4, prefix lengths uniform in [256, 2048] (seed 1), block 32,
    16 query heads, head_dim 128, 256-token pages behind a permuted page table."""
    gen = torch.Generator().manual_seed(1)
    prefix = torch.randint(256, 2049, (4,), generator=gen).tolist()
    bs, block, hq = 4, 32, 16
    ctx = [p + block for p in prefix]
    need = [(c + 255) // 256 for c in ctx]
    pages = sum(need) + 3
    perm = torch.randperm(pages, generator=gen).tolist()
    table = torch.full((bs, max(need)), -1, dtype=torch.int32)
    kc = torch.zeros(pages, 256, hkv, 128, dtype=BF)
    vc = torch.zeros_like(kc)
    at = 0
    for r in range(bs):
        for j in range(need[r]):
            table[r, j] = perm[at]
            at += 1
        k = torch.randn(ctx[r], hkv, 128, generator=gen).to(BF)
        v = torch.randn(ctx[r], hkv, 128, generator=gen).to(BF)
        slots = torch.tensor(orc.get_slots(table[r, :need[r]].tolist(), 0, ctx[r]), dtype=torch.int32)
        orc.store_kvcache(k, v, kc, vc, slots)
    q = torch.randn(bs, block, hq, 128, generator=gen).to(BF)
    return q, kc, vc, torch.tensor(ctx, dtype=torch.int32), table


@pytest.mark.parametrize("hkv", [2, 8])
def test_block_attention_against_flash_attn_with_kvcache(mdb, hkv):
    try:
        from flash_attn import flash_attn_with_kvcache
    except Exception as exc:            # noqa: BLE001  (any import problem means: no second opinion here)
        pytest.skip(f"flash-attn does not import: {exc!r}")
    q, kc, vc, ctx, table = (t.to(DEV) for t in _config1(hkv))
    scale = 128 ** -0.5
    # flash-attn reads whole pages through the table: give the padding entries a valid page id
    table_fa = table.clamp(min=0)
    try:
        want = flash_attn_with_kvcache(q, kc, vc, cache_seqlens=ctx, block_table=table_fa, softmax_scale=scale,
                                       causal=False)
        torch.cuda.synchronize()
    except Exception as exc:            # noqa: BLE001
        pytest.skip(f"flash_attn_with_kvcache does not run on this device: {exc!r}")
    got = mdb.ops.block_attn_with_kvcache(q, kc, vc, ctx, table, scale)
    err = (got.float() - want.float()).abs()
    cpu = orc.attn_paged(q.cpu(), kc.cpu(), vc.cpu(), ctx.cpu(), table.cpu(), scale)
    fa_vs_cpu = float((want.cpu().float() - cpu.float()).abs().max())
    ws = torch.empty(max(16, mdb.ops.attn_workspace_bytes(4, 32, 16, 16)), dtype=torch.uint8, device=DEV)
    out = torch.empty_like(q)
    ns = mdb.ops.default_nsplit(4, 32, 16, hkv, int(ctx.max()))
    ours_us = _time_us(lambda: mdb.ops.block_attn_with_kvcache(q, kc, vc, ctx, table, scale, nsplit=ns, workspace=ws,
                                                               out=out))
    fa_us = _time_us(lambda: flash_attn_with_kvcache(q, kc, vc, cache_seqlens=ctx, block_table=table_fa,
                                                     softmax_scale=scale, causal=False))
    _record("block_attention_vs_flash_attn", hkv=hkv, max_abs=round(float(err.max()), 5),
            mean_abs=round(float(err.mean()), 6), flash_attn_vs_cpu_oracle_max_abs=round(fa_vs_cpu, 5),
            ours_us=round(ours_us, 1), flash_attn_us=round(fa_us, 1))
    assert float(err.max()) <= 2e-2 and float(err.mean()) <= 5e-4
    assert mdb._lib.device_status(clear=True) == 0


def test_swiglu_epilogue_against_liger(mdb):
    try:
        import torch.distributed.tensor  # noqa: F401  (liger 0.8 reads this submodule without importing it)
        from liger_kernel.ops.swiglu import LigerSiLUMulFunction
    except Exception as exc:            # noqa: BLE001
        pytest.skip(f"liger-kernel does not import: {exc!r}")
    gen = torch.Generator().manual_seed(5)
    m, k, inter = 32, 512, 768
    x = torch.randn(m, k, generator=gen).to(BF).to(DEV)
    w = (0.05 * torch.randn(2 * inter, k, generator=gen)).to(BF).to(DEV)
    gate_up = mdb.ops.linear(x, w)                                   # bf16 projection, as F.linear leaves it
    gate, up = gate_up.chunk(2, -1)
    try:
        want = LigerSiLUMulFunction.apply(gate.contiguous(), up.contiguous())      # activation.py:14-15
        torch.cuda.synchronize()
    except Exception as exc:            # noqa: BLE001
        pytest.skip(f"liger SiLU*mul does not run on this device: {exc!r}")
    alone = mdb.ops.silu_and_mul(gate_up)
    fused = mdb.ops.gateup_swiglu(x, w)
    cpu = orc.silu_mul(gate_up.cpu())
    exact_alone = float((alone == want).float().mean())
    exact_fused = float((fused == want).float().mean())
    exact_cpu = float((cpu == want.cpu()).float().mean())
    # a one-step difference of bf16(silu(gate)) moves the product by up to two bf16 steps
    tol = want.float().abs() * 2.0 ** -6 + 1e-3 * float(want.float().std())
    _record("swiglu_vs_liger", exact_standalone=round(exact_alone, 5), exact_fused=round(exact_fused, 5),
            cpu_oracle_exact=round(exact_cpu, 5))
    assert bool(((alone.float() - want.float()).abs() <= tol).all())
    assert bool(((fused.float() - want.float()).abs() <= tol).all())
    assert exact_alone >= 0.99 and exact_fused >= 0.95
    assert mdb._lib.device_status(clear=True) == 0
