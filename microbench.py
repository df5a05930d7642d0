"""Per-kernel timings of the decode-step operators on the current GPU.

    python microbench.py attn --bs 64 --ctx 1536 5120
    python microbench.py stair --lens 4096 4096 4096 4096
    python microbench.py gemm --m 2048
    python microbench.py lmhead --m 2048
    python microbench.py elementwise --m 2048
    python microbench.py kvcommit --m 32768

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

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
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


def attn_case(bs: int, ctx_range, block: int = 32, hq: int = 16, hkv: int = 8, nsplit: int = 0,
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
    ns = nsplit or ops.default_nsplit(bs, block, hq, hkv, int(ctx.max()))
    ws = torch.empty(max(16, ops.attn_workspace_bytes(bs, block, hq, ns)), dtype=torch.uint8, device=DEV)
    ms = timed(lambda: ops.block_attn_with_kvcache(q, kc, vc, ctx_d, table_d, nsplit=ns, workspace=ws, out=out),
               reps, plain)
    return {"ms": ms, "bytes": nbytes, "flops": flops, "nsplit": ns}


def bench_attn(a) -> None:
    r = attn_case(a.bs, a.ctx, a.block, a.hq, a.hkv, a.nsplit, a.reps, a.plain, a.seed)
    line(f"attn bs={a.bs} ctx[{a.ctx[0]},{a.ctx[1]}] hkv={a.hkv} ns={r['nsplit']}", r["ms"], r["flops"], r["bytes"])


def stair_case(lens, block: int = 32, hq: int = 16, hkv: int = 8, reps: int = 10, plain: bool = False,
               seed: int = 3) -> dict:
    """Staircase (prefill) attention over packed sequences of the given lengths: milliseconds per launch,
    flops over the visible part of the mask (T^2 / 2 + T * block / 2 query-key pairs per head) and the
    algorithmic bytes (q, k, v in and out once)."""
    import numpy as np
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
    n = int(cu[-1])
    g = torch.Generator(device=DEV).manual_seed(seed)
    q = torch.randn(n, hq, 128, generator=g, device=DEV).to(BF)
    k = torch.randn(n, hkv, 128, generator=g, device=DEV).to(BF)
    v = torch.randn(n, hkv, 128, generator=g, device=DEV).to(BF)
    out = torch.empty_like(q)
    flops = sum(4.0 * hq * 128 * (t * t / 2 + t * block / 2) for t in lens)
    nbytes = (2 * n * hq * 128 + 2 * n * hkv * 128) * 2
    ms = timed(lambda: ops.sparse_attn_varlen(q, k, v, cu, cu, block, max_seqlen=max(lens), out=out), reps, plain)
    return {"ms": ms, "flops": flops, "bytes": nbytes, "tokens": n}


def bench_stair(a) -> None:
    r = stair_case(a.lens, a.block, a.hq, a.hkv, a.reps, a.plain, a.seed)
    line(f"staircase {len(a.lens)} seqs, {r['tokens']} tokens", r["ms"], r["flops"], r["bytes"])


def gemm_cases(m: int, hidden: int = 2048, inter: int = 6144, hq: int = 16, hkv: int = 8, reps: int = 10,
               plain: bool = False, seed: int = 3, only=None) -> list[dict]:
    """The four projections of a layer at ``m`` step rows: name, shape, milliseconds per launch, flops and
    weight bytes.  qkv is the plain projection (its fused norm / rotary / KV-store form is `qkv+rope+store`)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    h = hidden
    qkv_n = (hq + 2 * hkv) * 128
    out = []
    for name, (n, k) in {"qkv": (qkv_n, h), "o_proj": (h, hq * 128), "down_proj": (h, inter)}.items():
        if only and name not in only:
            continue
        x, w = _mat(g, m, k, 1.0), _mat(g, n, k)
        y = torch.empty(m, n, dtype=BF, device=DEV)
        out.append(dict(op=name, m=m, n=n, k=k, ms=timed(lambda: ops.linear(x, w, out=y), reps, plain),
                        flops=2.0 * m * n * k, bytes=2.0 * n * k))
    if (not only or "qkv+rope+store" in only) and ops.qkv_rope_commit_supported(m, h):
        x, w = _mat(g, m, h, 1.0), _mat(g, qkv_n, h)
        pos = torch.arange(m, device=DEV) % 4096
        table = pkg.decoder.rope_table(4096, 128, 1e6, DEV)
        ones = torch.ones(128, dtype=BF, device=DEV)
        pages = (m + 255) // 256
        kc = torch.zeros(pages, 256, hkv, 128, dtype=BF, device=DEV)
        vc = torch.zeros_like(kc)
        slots = torch.arange(m, dtype=torch.int32, device=DEV)
        q = torch.empty(m, hq, 128, dtype=BF, device=DEV)
        out.append(dict(op="qkv+rope+store", m=m, n=qkv_n, k=h,
                        ms=timed(lambda: ops.qkv_proj_rope_commit(x, w, pos, table, ones, ones, 1e-6, hq, hkv, slots, kc,
                                                                  vc, q_out=q), reps, plain),
                        flops=2.0 * m * qkv_n * h, bytes=2.0 * qkv_n * h))
    if not only or "gate_up" in only:
        x, w = _mat(g, m, h, 1.0), _mat(g, 2 * inter, h)
        act = torch.empty(m, inter, dtype=BF, device=DEV)
        out.append(dict(op="gate_up+SiLU*mul", m=m, n=2 * inter, k=h,
                        ms=timed(lambda: ops.gateup_swiglu(x, w, out=act), reps, plain),
                        flops=4.0 * m * inter * h, bytes=4.0 * inter * h))
    return out


def bench_gemm(a) -> None:
    for c in gemm_cases(a.m, a.hidden, a.inter, a.hq, a.hkv, a.reps, a.plain, a.seed, a.only):
        line(f"{c['op']} m={c['m']} n={c['n']} k={c['k']}", c["ms"], c["flops"], c["bytes"])


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


def kvcommit_cases(m: int, hq: int = 16, hkv: int = 8, reps: int = 10, plain: bool = False, seed: int = 3) -> list[dict]:
    """The paged KV write/commit at ``m`` token rows: the plain row scatter (``store_kvcache``) and the step's
    form fused with the q/k norm and the rotary embedding.  Bytes = what each must move once: the scatter reads
    and writes the K and V rows (2 * 2 * m * hkv * 128 * 2 B); the fused form reads the bf16 qkv row and writes
    q plus the K and V cache rows."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    d = 128
    pages = (m + 255) // 256 + 1
    k = torch.randn(m, hkv, d, generator=g, device=DEV).to(BF)
    v = torch.randn(m, hkv, d, generator=g, device=DEV).to(BF)
    kc = torch.zeros(pages, 256, hkv, d, dtype=BF, device=DEV)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(pages * 256, generator=g, device=DEV)[:m].int()
    out = [dict(op="kv_commit", m=m, ms=timed(lambda: ops.store_kvcache(k, v, kc, vc, slots), reps, plain),
                bytes=2.0 * 2 * m * hkv * d * 2)]
    qkv = torch.randn(m, (hq + 2 * hkv) * d, generator=g, device=DEV).to(BF)
    pos = torch.arange(m, device=DEV) % 4096
    table = pkg.decoder.rope_table(4096, d, 1e6, DEV)
    ones = torch.ones(d, dtype=BF, device=DEV)
    q = torch.empty(m, hq, d, dtype=BF, device=DEV)
    out.append(dict(op="qknorm_rope_commit", m=m,
                    ms=timed(lambda: ops.qknorm_rope_commit(qkv, pos, table, ones, ones, 1e-6, hq, hkv, slots, kc, vc,
                                                            q_out=q), reps, plain),
                    bytes=2.0 * m * (hq + 2 * hkv) * d * 2))
    return out


def bench_kvcommit(a) -> None:
    for c in kvcommit_cases(a.m, a.hq, a.hkv, a.reps, a.plain, a.seed):
        line(f"{c['op']} m={c['m']}", c["ms"], None, c["bytes"])


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
    ap.add_argument("op", choices=["attn", "stair", "gemm", "lmhead", "elementwise", "kvcommit"])
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
    ap.add_argument("--lens", type=int, nargs="+", default=[4096] * 4, help="stair: sequence lengths of the packed batch")
    ap.add_argument("--only", nargs="*", default=None, help="gemm: subset of qkv qkv+rope+store o_proj down_proj gate_up")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a GPU")
    {"attn": bench_attn, "stair": bench_stair, "gemm": bench_gemm, "lmhead": bench_lmhead, "elementwise": bench_elementwise,
     "kvcommit": bench_kvcommit}[a.op](a)
    status = pkg._lib.device_status()
    print("device status", status)
    if status:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
