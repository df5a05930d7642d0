"""Per-kernel timings of the decode-step operators on the current GPU.

    python mineru-diffusion_b200/microbench.py attn --bs 64 --ctx 1536 5120
    python mineru-diffusion_b200/microbench.py stair --lens 4096 4096 4096 4096
    python mineru-diffusion_b200/microbench.py gemm --m 2048
    python mineru-diffusion_b200/microbench.py lmhead --m 2048
    python mineru-diffusion_b200/microbench.py elementwise --m 2048

Each operator is captured ``--reps`` times into one CUDA graph and the graph
is timed with CUDA events, so host launch cost stays out of the figure; the
inputs of one call are larger than L2 for the bandwidth-bound cases.  With
``--plain`` the operator is launched ``--reps`` times without a graph (the
form to put under a profiler).  Shapes default to the 2.5B-class decoder
(hidden 2048, 16 query / 8 KV heads of 128, MLP 6144, vocabulary 151936).
"""
from __future__ import annotations

import argparse
import importlib
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
pkg = importlib.import_module("mineru-diffusion_b200")
ops = pkg.ops
DEV, BF = "cuda", torch.bfloat16


def timed(fn, reps: int, plain: bool) -> float:
    """Milliseconds per call."""
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if plain:
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fn()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(reps):
                fn()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def line(name: str, ms: float, flops: float | None = None, nbytes: float | None = None) -> None:
    extra = ""
    if flops:
        extra += f"  {flops / ms / 1e9:8.1f} TFLOP/s"
    if nbytes:
        extra += f"  {nbytes / ms / 1e6:8.1f} GB/s"
    print(f"{name:34s} {ms * 1e3:9.1f} us{extra}", flush=True)


def _mat(gen, r, c, scale=0.02):
    return (torch.randn(r, c, generator=gen, device=DEV) * scale).to(BF)


def attn_case(bs: int, ctx_range, block: int = 32, hq: int = 16, hkv: int = 8, nsplit: int = 0, kernel: int = 0,
              reps: int = 10, plain: bool = False, seed: int = 3) -> dict:
    """Block attention over the paged cache for ``bs`` requests with prefix lengths uniform in ``ctx_range``.
    Returns milliseconds per launch, the algorithmic bytes (K and V rows of every context once + q and out)
    and flops."""
    cg = torch.Generator().manual_seed(seed)
    lo, hi = ctx_range
    ctx = torch.randint(lo, hi + 1, (bs,), generator=cg) + block
    need = (ctx + 255) // 256
    pages = int(need.sum())
    perm = torch.randperm(pages, generator=cg)
    table = torch.full((bs, int(need.max())), -1, dtype=torch.int32)
    at = 0
    for r in range(bs):
        table[r, :need[r]] = perm[at:at + need[r]].int()
        at += int(need[r])
    g = torch.Generator(device=DEV).manual_seed(seed)
    kc = torch.randn(pages, 256, hkv, 128, generator=g, device=DEV).to(BF)
    vc = torch.randn(pages, 256, hkv, 128, generator=g, device=DEV).to(BF)
    q = torch.randn(bs, block, hq, 128, generator=g, device=DEV).to(BF)
    out = torch.empty_like(q)
    ctx_d, table_d = ctx.int().to(DEV), table.to(DEV)
    nbytes = int((2 * ctx * hkv * 128 * 2).sum()) + 2 * q.numel() * 2
    flops = int((4 * block * hq * 128 * ctx).sum())
    ops.set_option(ops.OPT_ATTN_KERNEL, kernel)
    ns = nsplit or ops.default_nsplit(bs, block, hq, hkv, int(ctx.max()))
    ws = torch.empty(max(16, ops.attn_workspace_bytes(bs, block, hq, ns)), dtype=torch.uint8, device=DEV)
    try:
        ms = timed(lambda: ops.block_attn_with_kvcache(q, kc, vc, ctx_d, table_d, nsplit=ns, workspace=ws, out=out),
                   reps, plain)
    finally:
        ops.set_option(ops.OPT_ATTN_KERNEL, 0)
    return {"ms": ms, "bytes": nbytes, "flops": flops, "nsplit": ns}


def bench_attn(a) -> None:
    for kern in a.kernel:
        r = attn_case(a.bs, a.ctx, a.block, a.hq, a.hkv, a.nsplit, kern, a.reps, a.plain, a.seed)
        name = {0: "auto", 1: "mma.sync", 2: "tcgen05"}[kern]
        line(f"attn[{name}] bs={a.bs} ctx[{a.ctx[0]},{a.ctx[1]}] hkv={a.hkv} ns={r['nsplit']}", r["ms"], r["flops"],
             r["bytes"])


def bench_stair(a) -> None:
    """Staircase (prefill) attention over packed sequences of the given lengths; flops are counted over the
    visible part of the mask only (T^2 / 2 + T * block / 2 query-key pairs per head)."""
    import numpy as np
    lens = a.lens
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
    n = int(cu[-1])
    g = torch.Generator(device=DEV).manual_seed(a.seed)
    q = torch.randn(n, a.hq, 128, generator=g, device=DEV).to(BF)
    k = torch.randn(n, a.hkv, 128, generator=g, device=DEV).to(BF)
    v = torch.randn(n, a.hkv, 128, generator=g, device=DEV).to(BF)
    out = torch.empty_like(q)
    flops = sum(4.0 * a.hq * 128 * (t * t / 2 + t * a.block / 2) for t in lens)
    for kern in a.kernel:
        ops.set_option(ops.OPT_ATTN_KERNEL, kern)
        ms = timed(lambda: ops.sparse_attn_varlen(q, k, v, cu, cu, a.block, max_seqlen=max(lens), out=out), a.reps, a.plain)
        name = {0: "auto", 1: "mma.sync", 2: "tcgen05"}[kern]
        line(f"staircase[{name}] {len(lens)} seqs, {n} tokens", ms, flops)
    ops.set_option(ops.OPT_ATTN_KERNEL, 0)


def bench_gemm(a) -> None:
    g = torch.Generator(device=DEV).manual_seed(a.seed)
    m, h, inter = a.m, a.hidden, a.inter
    qkv_n = (a.hq + 2 * a.hkv) * 128
    for name, (n, k) in {"qkv": (qkv_n, h), "o_proj": (a.hq * 128, h), "down_proj": (h, inter)}.items():
        if a.only and name not in a.only:
            continue
        x, w = _mat(g, m, k, 1.0), _mat(g, n, k)
        y = torch.empty(m, n, dtype=BF, device=DEV)
        line(f"{name} m={m} n={n} k={k}", timed(lambda: ops.linear(x, w, out=y), a.reps, a.plain), 2.0 * m * n * k,
             2.0 * n * k)
    if not a.only or "gate_up" in a.only:
        x, w = _mat(g, m, h, 1.0), _mat(g, 2 * inter, h)
        act = torch.empty(m, inter, dtype=BF, device=DEV)
        line(f"gate_up+SiLU*mul m={m} n={2 * inter} k={h}", timed(lambda: ops.gateup_swiglu(x, w, out=act), a.reps, a.plain),
             4.0 * m * inter * h, 4.0 * inter * h)


def bench_lmhead(a) -> None:
    g = torch.Generator(device=DEV).manual_seed(a.seed)
    m, h, v = a.m, a.hidden, a.vocab
    x, w = _mat(g, m, h, 1.0), _mat(g, v, h)
    temps = torch.ones(max(1, m // a.block), device=DEV)
    ws = torch.empty(ops.lmhead_workspace_bytes(m, v), dtype=torch.uint8, device=DEV)
    x0 = torch.empty(m, dtype=torch.int32, device=DEV)
    conf = torch.empty(m, device=DEV)
    ms = timed(lambda: ops.lm_head_sample(x, w, temps, a.block, seed=1, step=3, workspace=ws, x0=x0, conf=conf),
               a.reps, a.plain)
    line(f"lm_head+sampler (Gumbel) m={m} v={v}", ms, 2.0 * m * v * h, 2.0 * v * h)
    ms = timed(lambda: ops.lm_head_sample(x, w, temps, a.block, workspace=ws, x0=x0, conf=conf), a.reps, a.plain)
    line(f"lm_head+sampler (argmax) m={m} v={v}", ms, 2.0 * m * v * h, 2.0 * v * h)


def bench_elementwise(a) -> None:
    g = torch.Generator(device=DEV).manual_seed(a.seed)
    m, h = a.m, a.hidden
    x, res = _mat(g, m, h, 1.0), _mat(g, m, h, 1.0)
    wn = torch.ones(h, dtype=BF, device=DEV)
    o1, o2 = torch.empty_like(x), torch.empty_like(x)
    line(f"add_rms_norm m={m} h={h}", timed(lambda: ops.add_rms_norm(x, res, wn, 1e-6, out=o1, residual_out=o2),
                                           a.reps, a.plain), None, 4.0 * m * h * 2)
    gate_up = _mat(g, m, 2 * a.inter, 1.0)
    line(f"silu_and_mul m={m} inter={a.inter}", timed(lambda: ops.silu_and_mul(gate_up), a.reps, a.plain), None,
         3.0 * m * a.inter * 2)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("op", choices=["attn", "stair", "gemm", "lmhead", "elementwise"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--plain", action="store_true", help="launch without a CUDA graph")
    ap.add_argument("--seed", type=int, default=3)
    ap.add_argument("--m", type=int, default=2048, help="step rows (requests x block)")
    ap.add_argument("--bs", type=int, default=64)
    ap.add_argument("--ctx", type=int, nargs=2, default=[1536, 5120], help="prefix length range (uniform)")
    ap.add_argument("--block", type=int, default=32)
    ap.add_argument("--hq", type=int, default=16)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=6144)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--nsplit", type=int, default=0, help="key-range parts per request (0: the library's choice)")
    ap.add_argument("--kernel", type=int, nargs="+", default=[1, 2], help="attention kernels: 1 mma.sync, 2 tcgen05")
    ap.add_argument("--lens", type=int, nargs="+", default=[4096] * 4, help="stair: sequence lengths of the packed batch")
    ap.add_argument("--only", nargs="*", default=None, help="gemm: subset of qkv o_proj down_proj gate_up")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a GPU")
    {"attn": bench_attn, "stair": bench_stair, "gemm": bench_gemm, "lmhead": bench_lmhead, "elementwise": bench_elementwise}[a.op](a)
    status = pkg._lib.device_status()
    print("device status", status)
    if status:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
