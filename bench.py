"""Benchmark of the block-diffusion decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at N=1 ("config2"): the full decoder at the reference's configuration
defaults (28 layers, hidden 2048, 16 query / 8 KV heads, vocabulary 151936,
bf16), seeded N(0, 0.02) weights with RMSNorm weights 1, one request whose
prompt is 1024 synthetic visual embedding rows N(0, 1) plus 32 random text
ids; 1024 tokens are generated in blocks of 32, threshold 0.9, temperature 1,
Gumbel noise on.  A step is one pass of the hot path (``ModelRunner.run`` in
decode form: a denoising pass or the KV-commit pass of a finished block).
With N > 1 every rank runs its own request of the same shape (request-level
data parallelism, no data-path collective).

Printed JSON line: ``value`` = tokens committed in the K timed steps divided by
the device time of those steps (inputs resident, CUDA events around the GPU
work of each step), summed over the GPUs; ``e2e`` = the same tokens divided by
the bracketed wall time of the K calls through the public API, host->device
and device->host copies included.  ``roofline`` is measured live for the
dominant kernel symbol (the weight-streaming GEMM writing split-k slices: qkv,
o_proj and down_proj of every layer) by launching it over the 28 layers'
distinct weights (far beyond L2) inside a CUDA graph between two events;
``roofline.per_op`` lists every GEMM of a step, the gate/up projection and the
LM head included.  Further keys of the one-GPU line: ``block_attn`` and
``staircase_prefill_attn`` (the attention kernels at prefixes >= 4K),
``config1`` (the stand-alone attention op of BASELINE config 1 on the GPU and
as torch masked SDPA on the host cores), ``batched`` (BASELINE config 3: 64
concurrent requests), ``cpu_baseline`` (the CPU oracle timed on a bounded
sample) and ``parity`` (the CUDA runner teacher-forced against that oracle on
the full-size decoder).  With ``--gpus N`` the line carries ``dp_completion``
(a fixed request set partitioned over the ranks and run to completion) and, at
N = 2, ``tp2`` (the tensor-parallel pair against one GPU).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from dataclasses import dataclass, replace

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

TEXT_IDS = 32
WEIGHT_SEED = 20260320
MASK_ID = 151669
METRIC = "decoded tokens/sec (block diffusion, bf16), summed over the GPUs of the job"


@dataclass
class Workload:
    """One BASELINE configuration as the benchmark runs it."""
    name: str
    requests: int = 1               # concurrent requests per GPU
    visual_rows: int = 1024         # one request: its visual rows; several: lower end of the uniform range
    visual_max: int = 1024          # several requests: upper end of the uniform range
    new_tokens: int = 1024
    block: int = 32
    threshold: float = 0.9
    temperature: float = 1.0
    fuse_commit: bool = False

    def describe(self) -> str:
        if self.requests == 1:
            what = f"1 request per GPU, {self.visual_rows} synthetic visual rows + {TEXT_IDS} text ids"
        else:
            what = (f"{self.requests} concurrent requests per GPU, visual rows uniform in "
                    f"[{self.visual_rows}, {self.visual_max}] + {TEXT_IDS} text ids")
        return (f"{self.name}: full decoder (28 layers, hidden 2048, 16q/8kv heads, vocab 151936), {what}, "
                f"{self.new_tokens} new tokens, block {self.block}, threshold {self.threshold}, "
                f"temperature {self.temperature}")


WORKLOADS = {
    "config2": Workload("config2"),
    "config3": Workload("config3", requests=64, visual_rows=512, visual_max=4096, new_tokens=2048),
    "config4": Workload("config4", visual_rows=4096, visual_max=4096, new_tokens=4096),
    "config5": Workload("config5 sweep point", requests=64, visual_rows=512, visual_max=8192, new_tokens=2048),
}


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- workload
def make_request(pkg, dcfg, wl: Workload, seed: int, visual_rows: int, new_tokens: int | None = None):
    g = torch.Generator().manual_seed(seed)
    visual = torch.randn(visual_rows, dcfg.hidden_size, generator=g).to(torch.bfloat16)
    text = torch.randint(0, 151000, (TEXT_IDS,), generator=g).tolist()
    ids = [0] * visual_rows + text                 # the visual positions' ids are never embedded
    sp = pkg.SamplingParams(temperature=wl.temperature, max_new_tokens=new_tokens or wl.new_tokens, ignore_eos=True,
                            dynamic_threshold=wl.threshold)
    return pkg.Sequence(ids, sp, denoising_block_size=wl.block, mask_token_id=MASK_ID, inputs_embeds=visual.pin_memory())


def build_engine(pkg, wl: Workload, device: str, tp: int, rank: int, seed: int, visual_rows: list[int],
                 new_tokens: list[int] | None = None, weights=None):
    """Engine replica (or this rank's half of a tensor-parallel pair) with pages for every request's full length."""
    dcfg = pkg.DecoderConfig()
    news = new_tokens or [wl.new_tokens] * len(visual_rows)
    lens = [v + TEXT_IDS + n + wl.block for v, n in zip(visual_rows, news)]
    in_flight = min(wl.requests, len(visual_rows))
    # pages: every request in flight at its full length (requests beyond that wait for pages to come back)
    pages = sum(sorted(((t + 255) // 256 for t in lens), reverse=True)[:in_flight]) + 2
    max_len = max(4096, (max(lens) + 255) // 256 * 256)
    cfg = pkg.Config(max_num_batched_tokens=max(max_len, 16384 if in_flight > 1 else 0), max_num_seqs=in_flight,
                     max_model_len=max_len, enforce_eager=False, num_kvcache_blocks=pages, decoder_config=dcfg,
                     tensor_parallel_size=tp, block_size=wl.block, fuse_commit_pass=wl.fuse_commit)
    runner = pkg.ModelRunner(cfg, rank=rank if tp == 2 else 0, weights=weights, weight_seed=WEIGHT_SEED, noise="gumbel",
                             noise_seed=seed, device=device)
    engine = pkg.LLMEngine(cfg, runner)
    for i, (v, n) in enumerate(zip(visual_rows, news)):
        engine.add_sequence(make_request(pkg, dcfg, wl, seed=seed + 1000 * i, visual_rows=v, new_tokens=n))
    return cfg, runner, engine


def timed_steps(engine, runner, steps: int, warmup: int, local_rank: int, world: int, sample_clocks: bool = True):
    """Prefill (untimed), ``warmup`` decode steps (untimed), then ``steps`` timed decode steps bracketed by a
    barrier + synchronize on both sides.  Device time: CUDA events around the GPU work of each step."""
    stream = torch.cuda.current_stream()
    engine.step()
    while engine.scheduler.waiting:
        engine.step()
    for _ in range(warmup):
        engine.step()
    # the timed region holds exactly the timed steps: a step launched ahead by the last warm-up call is dropped, and
    # the last timed call launches none
    ahead_setting = runner.launch_ahead
    runner.cancel_ahead()
    torch.cuda.synchronize()
    # one event pair per step launched; with launch-ahead a step is launched during the call before the one that
    # collects it, so the runner takes pairs from an iterator and names the pair of the step each call collected
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps + 2)]
    used = []
    sampler = ClockSampler(local_rank) if sample_clocks else None
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    if sampler:
        sampler.start()
    tokens = steps_done = 0
    wall0 = time.perf_counter()
    e_all0, e_all1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_all0.record(stream)
    runner.step_events = iter(ev)
    hits0 = runner.ahead_hits
    for i in range(steps):
        if engine.is_finished():
            break
        if i == steps - 1:
            runner.launch_ahead = False
        _, n = engine.step()
        tokens += -n if n < 0 else 0
        steps_done += 1
        used.append(runner.last_step_events)
    e_all1.record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    if world > 1:
        torch.distributed.barrier()
    clocks = sampler.stop() if sampler else None
    runner.step_events = None
    runner.launch_ahead = ahead_setting
    dev_ms = sum(p[0].elapsed_time(p[1]) for p in used if p is not None)   # a prefill step carries no pair
    e2e_ms = max(e_all0.elapsed_time(e_all1), wall * 1e3)
    return dict(tokens=tokens, steps=steps_done, dev_ms=dev_ms, e2e_ms=e2e_ms, clocks=clocks,
                ahead_hits=runner.ahead_hits - hits0)


def run_workload(pkg, wl: Workload, args, rank: int, world: int, local_rank: int, tp: int = 1):
    device = f"cuda:{local_rank}"
    torch.cuda.set_device(device)
    nreq = wl.requests
    if nreq > 1:
        vg = torch.Generator().manual_seed(3 + (0 if tp == 2 else rank))   # a TP pair serves the same requests
        visual_rows = torch.randint(wl.visual_rows, wl.visual_max + 1, (nreq,), generator=vg).tolist()
    else:
        visual_rows = [wl.visual_rows]
    # tensor-parallel pair: both ranks serve the same request with the same noise; replicas: one request set each
    seed = 2 if tp == 2 else 2 + rank
    cfg, runner, engine = build_engine(pkg, wl, device, tp, rank, seed, visual_rows)
    res = timed_steps(engine, runner, args.steps, args.warmup, local_rank, world)
    # the packed step inputs: a step collected from a launch made ahead took its block ids and step counters from
    # the device and copied only the rest
    ahead = res.get("ahead_hits", 0) / max(res["steps"], 1)
    res.update(h2d=int(round(runner.inputs.nbytes - ahead * runner.inputs.o_pos)),
               d2h=nreq * (wl.block * 8 + wl.block + 4) + 4,
               launches=runner.launches_per_decode_step(nreq) * res["steps"],
               status=pkg._lib.device_status(clear=True))
    return res, runner, engine


# ----------------------------------------------------------------------------- kernel measurements
def _graph_time_us(fn, launches: int, reps: int = 5) -> float:
    """Average device time of one launch: the launches are captured in a CUDA
    graph (no host launch cost in the timed region) and the graph is replayed
    ``reps`` times between two events on the launching stream."""
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * launches)


def measure_dominant_kernel(pkg, runner, block: int):
    """Live roofline of the step's GEMM kernels at m = block rows: each is launched once per layer over the 28
    layers' distinct weights (0.2 - 1.4 GB per sweep, far beyond the 126 MB L2).  Algorithmic bytes per launch
    = (m k + k n + m n) * 2: activations in, weight once, a bf16 result out (the fp32 split-k slices the
    kernel really writes are an implementation detail and are not counted)."""
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    eng, dcfg, ops = runner.engine, runner.dcfg, pkg.ops
    m = block
    h, inter, d = dcfg.hidden_size, dcfg.intermediate_size, dcfg.head_dim
    hq, hkv, vocab = dcfg.num_attention_heads, dcfg.num_key_value_heads, dcfg.vocab_size
    nqkv = (hq + 2 * hkv) * d
    layers = runner.weights.layers
    x, act, attn = eng.x[:m], eng.act[:m], eng.attn[:m].view(m, hq * d)

    def parts(ks, n):
        return eng.partials[:ks * m * n].view(ks, m, n)

    def algo(n, k):
        return (m * k + k * n + m * n) * 2

    temps = torch.ones(1, device=x.device)
    cases = [
        ("gate_up + SiLU*mul", "gemm_ws_kernel<swiglu>", 2 * inter * h * 2 + m * h * 2 + m * inter * 2, len(layers),
         lambda: [ops.gateup_swiglu(x, lw.gate_up, out=act) for lw in layers]),
        ("qkv", "gemm_ws_kernel<partial>", algo(nqkv, h), len(layers),
         lambda: [ops.gemm_splitk_partials(x, lw.qkv, eng.ks_qkv, parts(eng.ks_qkv, nqkv)) for lw in layers]),
        ("o_proj", "gemm_ws_kernel<partial>", algo(h, hq * d), len(layers),
         lambda: [ops.gemm_splitk_partials(attn, lw.o, eng.ks_o, parts(eng.ks_o, h)) for lw in layers]),
        ("down_proj", "gemm_ws_kernel<partial>", algo(h, inter), len(layers),
         lambda: [ops.gemm_splitk_partials(act, lw.down, eng.ks_down, parts(eng.ks_down, h)) for lw in layers]),
        ("lm_head + sampler scan", "gemm_ws_kernel<lm_head> + sampler_finalize_kernel", vocab * h * 2 + m * h * 2 + m * 16, 2,
         lambda: [eng.sample(eng.final[:m], temps, seed=1) for _ in range(2)]),
    ]
    out = []
    for label, kernel, nbytes, launches, fn in cases:
        us = _graph_time_us(fn, launches)
        out.append({"op": label, "kernel": kernel, "us_per_launch": round(us, 2), "bytes_per_launch": nbytes,
                    "achieved_gbs": round(nbytes / us / 1e3, 1), "frac": round(nbytes / us / 1e3 / peak, 4)})
    # The kernel symbol with the largest share of a step is the split-k slice instantiation: it runs three
    # times per layer (qkv, o_proj, down_proj).  Its roofline entry averages those launches.
    part = [o for o in out if o["kernel"].endswith("<partial>")]
    nbytes = sum(o["bytes_per_launch"] for o in part) / len(part)
    us = sum(o["us_per_launch"] for o in part) / len(part)
    achieved = nbytes / us / 1e3
    return {"bound": "hbm", "kernel": f"gemm_ws_kernel<partial> (qkv, o_proj, down_proj launches of a step averaged, m={m})",
            "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
            # dram__bytes_read.sum + dram__bytes_write.sum per launch, averaged over the same three launches: a
            # figure from the ncu capture summarised in the file named below, not measured in this run
            "traffic": 17051819, "traffic_source": "profiles/gemm_ws_kernel_partial_config2_m32.md",
            "peak_source": "measured" if peaks else "fallback", "bytes_per_launch": round(nbytes),
            "us_per_launch": round(us, 2), "per_op": out}


def measure_attention(block: int = 32):
    """The second half of the metric.  ``block_attn``: HBM GB/s of the block attention over the paged cache at
    prefixes >= 4K (64 requests, prefix lengths U[4096, 8192], 16 query / 8 KV heads, 1.7 GB of K/V per launch,
    far beyond L2), ten launches in a CUDA graph between two events.  ``staircase_prefill_attn``: the prefill
    form on four packed sequences of 4096 tokens (compute-bound: TFLOP/s of the visible part of the mask)."""
    import microbench as mb
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    tpeak = float(peaks.get("bf16_tflops", 1590.0))
    src = "measured" if peaks else "fallback"
    out = {}
    try:
        r = mb.attn_case(64, (4096, 8192), block=block, hq=16, hkv=8, reps=10)
        achieved = r["bytes"] / (r["ms"] * 1e-3) / 1e9
        out["block_attn"] = {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4), "peak_source": src, "us_per_launch": round(r["ms"] * 1e3, 1),
            "workload": "block attention over the paged KV cache, 64 requests, prefix U[4096,8192], 16q/8kv heads "
                        f"x 128, block {block}, 256-token pages"}
        r = mb.stair_case([4096] * 4, block=block, hq=16, hkv=8, reps=5)
        tf = r["flops"] / (r["ms"] * 1e-3) / 1e12
        out["staircase_prefill_attn"] = {
            "bound": "tensor", "achieved": round(tf, 1), "peak": tpeak, "unit": "TFLOP/s", "frac": round(tf / tpeak, 4),
            "peak_source": src, "us_per_launch": round(r["ms"] * 1e3, 1),
            "gbs_algorithmic": round(r["bytes"] / (r["ms"] * 1e-3) / 1e9, 1),
            "workload": f"staircase prefill attention, 4 packed sequences of 4096 tokens, 16q/8kv heads x 128, stairs {block}"}
    except torch.OutOfMemoryError:
        pass
    return out


def measure_config1():
    """BASELINE config 1, the attention op alone: batch 4, prefix lengths uniform in [256, 2048] (seed 1), block
    32, 16 query / 2 KV heads, head_dim 128, bf16 N(0, 1), 256-token pages.  Decode form (the block's rows
    against the paged cache) and prefill form (every row of prefix + block under the right-aligned staircase)
    on the GPU, and the reference's CPU route for the same tensors: torch SDPA with a boolean mask
    (mineru_diffusion/modeling_mineru_diffusion.py:189-206) on the host cores."""
    import microbench as mb
    import torch.nn.functional as F
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    block, hq, hkv = 32, 16, 2
    dec = mb.attn_case(4, (256, 2048), block=block, hq=hq, hkv=hkv, reps=20, seed=1)
    g = torch.Generator().manual_seed(1)
    prefix = torch.randint(256, 2049, (4,), generator=g).tolist()
    lens = [p + block for p in prefix]
    pre = mb.stair_case(lens, block=block, hq=hq, hkv=hkv, reps=20, seed=1)
    dec_gbs = dec["bytes"] / (dec["ms"] * 1e-3) / 1e9
    pre_gbs = pre["bytes"] / (pre["ms"] * 1e-3) / 1e9
    # the CPU route on the same shapes: one SDPA call per sequence (the HF twin runs batch 1), GQA by repetition
    threads = len(os.sched_getaffinity(0))
    torch.set_num_threads(threads)
    gcpu = torch.Generator().manual_seed(1)

    def cpu_case(prefill: bool):
        cases = []
        for t in lens:
            rows = t if prefill else block
            q = torch.randn(1, hq, rows, 128, generator=gcpu).to(torch.bfloat16)
            k = torch.randn(1, hkv, t, 128, generator=gcpu).to(torch.bfloat16).repeat_interleave(hq // hkv, dim=1)
            v = torch.randn(1, hkv, t, 128, generator=gcpu).to(torch.bfloat16).repeat_interleave(hq // hkv, dim=1)
            if prefill:
                i = torch.arange(t)
                pad = (t + block - 1) // block * block - t
                limit = ((i + pad) // block + 1) * block - 1 - pad
                mask = (torch.arange(t)[None, :] <= limit[:, None])[None, None]
            else:
                mask = torch.ones(1, 1, rows, t, dtype=torch.bool)
            cases.append((q, k, v, mask))
        with torch.inference_mode():
            for q, k, v, mask in cases:            # warm-up
                F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
            reps = 3 if prefill else 20
            t0 = time.perf_counter()
            for _ in range(reps):
                for q, k, v, mask in cases:
                    F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
            return (time.perf_counter() - t0) / reps * 1e3
    cpu_dec_ms, cpu_pre_ms = cpu_case(False), cpu_case(True)
    return {
        "workload": "attention op alone: batch 4, prefix U[256,2048] (seed 1), block 32, 16q/2kv heads x 128, bf16 N(0,1), "
                    "256-token pages",
        "prefix_lengths": prefix, "peak_gbs": peak,
        "decode_form": {"us": round(dec["ms"] * 1e3, 2), "algorithmic_bytes": dec["bytes"], "gbs": round(dec_gbs, 1),
                        "frac_of_hbm_peak": round(dec_gbs / peak, 4), "key_range_parts": dec["nsplit"]},
        "prefill_form": {"us": round(pre["ms"] * 1e3, 2), "algorithmic_bytes": pre["bytes"], "gbs": round(pre_gbs, 1),
                         "frac_of_hbm_peak": round(pre_gbs / peak, 4),
                         "tflops": round(pre["flops"] / (pre["ms"] * 1e-3) / 1e12, 1)},
        "cpu_masked_sdpa": {"cores": threads, "decode_form_ms": round(cpu_dec_ms, 3), "prefill_form_ms": round(cpu_pre_ms, 2),
                            "decode_form_gbs": round(dec["bytes"] / (cpu_dec_ms * 1e-3) / 1e9, 2),
                            "prefill_form_gbs": round(pre["bytes"] / (cpu_pre_ms * 1e-3) / 1e9, 2),
                            "kind": "torch.nn.functional.scaled_dot_product_attention with a boolean mask, bf16, one call "
                                    "per sequence (the reference's CPU route)"},
        "note": "6.6 MB of K/V in total: both forms are bound by launch and pipeline latency at this size, not by HBM"}


def measure_batched(pkg, args, local_rank: int):
    """BASELINE config 3 on one GPU: 64 concurrent requests, 2048 rows per step; plus the four projections and
    the LM head at 2048 rows against the sustained cuBLAS figure, and the clocks of that region."""
    import microbench as mb
    peaks = load_peaks()
    sustained = float(peaks.get("bf16_tflops_sustained", 1400.0))
    wl = WORKLOADS["config3"]
    a = argparse.Namespace(steps=min(args.steps, 40), warmup=3)
    res, runner, engine = run_workload(pkg, wl, a, 0, 1, local_rank)
    ms = res["dev_ms"] / max(res["steps"], 1)
    out = {"workload": wl.describe(), "steps": res["steps"], "ms_per_step": round(ms, 3),
           "tokens_per_s": round(res["tokens"] / (res["dev_ms"] * 1e-3), 1),
           "e2e_tokens_per_s": round(res["tokens"] / (res["e2e_ms"] * 1e-3), 1),
           "e2e_ms_per_step": round(res["e2e_ms"] / max(res["steps"], 1), 3), "clocks": res["clocks"],
           "device_status": res["status"], "gpu_launches": res["launches"]}
    runner.exit()
    del runner, engine
    torch.cuda.empty_cache()
    ops_out = []
    for c in mb.gemm_cases(2048, reps=10, only=["qkv+rope+store", "o_proj", "down_proj", "gate_up"]):
        tf = c["flops"] / (c["ms"] * 1e-3) / 1e12
        ops_out.append({"op": c["op"], "us": round(c["ms"] * 1e3, 1), "tflops": round(tf, 1),
                        "frac_of_sustained": round(tf / sustained, 4)})
    out["per_op_m2048"] = ops_out
    out["tensor_peak_sustained_tflops"] = sustained
    r = mb.attn_case(64, (512, 4096), block=32, hq=16, hkv=8, reps=10)
    out["block_attn_gbs"] = round(r["bytes"] / (r["ms"] * 1e-3) / 1e9, 1)
    return out


# ----------------------------------------------------------------------------- CPU arm
def cpu_weights():
    """Full-size decoder weights for the CPU oracle, seeded N(0, 0.02): one layer is drawn and the others are
    row-rotated copies of it (distinct memory and distinct matrices, a twenty-eighth of the random draws)."""
    from oracle import nano_oracle as orc
    cfg = orc.DecoderConfig()
    g = torch.Generator().manual_seed(WEIGHT_SEED)
    bf = torch.bfloat16

    def mat(r, c):
        return (torch.randn(r, c, generator=g) * 0.02).to(bf)

    h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    base = orc.LayerWeights(torch.ones(h, dtype=bf), mat((hq + 2 * hkv) * d, h), torch.ones(d, dtype=bf),
                            torch.ones(d, dtype=bf), mat(h, hq * d), torch.ones(h, dtype=bf), mat(2 * i, h), mat(h, i))
    layers = [base]
    for j in range(1, cfg.num_hidden_layers):
        layers.append(orc.LayerWeights(base.input_ln, base.qkv.roll(j, 0).contiguous(), base.q_norm, base.k_norm,
                                       base.o.roll(j, 0).contiguous(), base.post_ln,
                                       base.gate_up.roll(j, 0).contiguous(), base.down.roll(j, 0).contiguous()))
    embed = mat(cfg.vocab_size, h)
    return cfg, orc.DecoderWeights(embed, layers, torch.ones(h, dtype=bf), embed.roll(1, 0).contiguous())


def run_cpu_sample(steps: int, warmup: int, wl: Workload, threads: int | None = None, prepared=None):
    """The reference's torch CPU path (restated in oracle/) on a bounded sample
    of the workload: decode-form denoising passes of the full-size decoder at
    the context length reached half way through generation, KV cache filled
    with seeded noise instead of a CPU prefill."""
    from oracle import nano_oracle as orc
    # every core this process may run on (a torchrun launch sets OMP_NUM_THREADS=1, which would leave 1 thread)
    torch.set_num_threads(threads or len(os.sched_getaffinity(0)))
    cfg, weights = prepared or cpu_weights()
    orc.use_native_linear(True)
    g = torch.Generator().manual_seed(WEIGHT_SEED + 1)
    block = wl.block
    prefix = wl.visual_rows + TEXT_IDS + wl.new_tokens // 2
    pages = (prefix + block + 255) // 256
    runner = orc.OracleModelRunner(cfg, weights, num_pages=pages, block_size=block, mask_token_id=MASK_ID,
                                   noise_fn=lambda step, shape: -torch.empty(shape).exponential_(generator=g).log())
    runner.decoder.kv_cache.normal_(generator=g)

    class Req:
        def __init__(self):
            from types import SimpleNamespace
            self.seq_id = 0
            self.token_ids = [1] * prefix
            self.block_table = list(range(pages))
            self.num_cached_tokens = 0
            self.temperature = wl.temperature
            self.mask_token_id = MASK_ID
            self.sampling_params = SimpleNamespace(dynamic_threshold=wl.threshold)
            self.current_denoising_block = torch.full((block,), MASK_ID, dtype=torch.int64)
            self.current_step_map = torch.zeros(block, dtype=torch.int32)
            self.current_denoise_step = 0

        def __len__(self):
            return len(self.token_ids)

        def __getitem__(self, k):
            return self.token_ids[k]

    req = Req()
    try:
        with torch.inference_mode():
            for _ in range(warmup):
                runner.run([req], False)
            t0 = time.perf_counter()
            tokens = 0
            for _ in range(steps):
                tokens += runner.run([req], False)
            dt = time.perf_counter() - t0
    finally:
        orc.use_native_linear(False)
    return tokens, dt, torch.get_num_threads(), prefix


def run_parity(pkg, prepared, device: str):
    """The CUDA runner teacher-forced against the CPU oracle on the full-size decoder (the weights of the CPU
    sample), context ~1.1K: a few passes at temperature 1 and at a temperature low enough for the threshold
    branch.  The oracle is the checker here; nothing of it is timed or shipped."""
    from oracle import parity
    cfg, weights = prepared
    gw = pkg.DecoderWeights.from_reference_layout(weights, device)
    out = {}
    for name, temp, passes in (("temperature_1", 1.0, 6), ("temperature_0.005", 0.005, 5)):
        r = parity.decode_parity(pkg, cfg, weights, context=1056, passes=passes, temperature=temp, seed=11,
                                 device=device, eager=False, gpu_weights=gw)
        r["disagreements"] = r["disagreements"][:8]
        out[name] = r
    out["note"] = ("decision_agreement: positions changed by either path that hold the same token in both; robust_*: "
                   "passes whose decision a 2e-2 move of every logit cannot flip (floor_robust_*: a move of the oracle's own "
                   "floor); oracle_floor_logits_fp32_max_abs: the "
                   "CPU oracle against itself with the rounding inside its attention placed differently (first pass), "
                   "i.e. what two equally valid implementations differ by after 28 bf16 layers at this width; every "
                   "recorded disagreement is a tie within the logits error of its pass over T")
    return out


# ----------------------------------------------------------------------------- multi-GPU extras
def run_dp_completion(pkg, args, rank: int, world: int, local_rank: int):
    """Strong scaling of request-level data parallelism where it can fail: a fixed seeded request set with
    BASELINE config 5's distributions (visual rows and output lengths uniform, scaled down so that every N
    finishes within the time limit: 32 requests, visual rows U[512, 8192], outputs U[64, 512] rounded up to
    whole blocks), partitioned over the ranks by ``engine/dp.py:partition_requests`` (greedy longest-first on a
    time model of a replica) and run to completion at a low temperature, so that the threshold decides how many
    passes a block takes.  Same set for every N.  Returns tokens/s over the slowest rank's time, per-rank finish
    times and the max/mean imbalance."""
    dp = importlib.import_module("mineru-diffusion_b200.engine.dp")
    device = f"cuda:{local_rank}"
    wl = replace(WORKLOADS["config5"], name="config5 (scaled) run to completion", requests=16, temperature=0.005,
                 new_tokens=512)
    total_requests = 32
    g = torch.Generator().manual_seed(5)
    visual = torch.randint(512, 8193, (total_requests,), generator=g).tolist()
    news = ((torch.randint(64, 513, (total_requests,), generator=g) + wl.block - 1) // wl.block * wl.block).tolist()
    # time model of a replica, microseconds: prefill 4 us per prompt token (4 GFLOP per token at ~1 PFLOP/s), a
    # decode step 1600 us of weight streaming whatever the batch + 130 us per request in flight (config-3 step:
    # (10.0 - 1.7) ms / 63), three passes per block at this temperature
    steps_est = [3 * n // wl.block for n in news]
    costs = [4.0 * (v + TEXT_IDS) + 130.0 * s for v, s in zip(visual, steps_est)]
    mine = dp.partition_requests(costs, world, steps=steps_est, step_cost=1600.0)[rank]
    cfg, runner, engine = build_engine(pkg, wl, device, 1, 0, seed=5, visual_rows=[visual[i] for i in mine],
                                       new_tokens=[news[i] for i in mine])
    # distinct request seeds whatever the rank: rebuild the requests with their global index
    engine.scheduler.waiting.clear()
    for i in mine:
        engine.add_sequence(make_request(pkg, pkg.DecoderConfig(), wl, seed=5000 + i, visual_rows=visual[i],
                                         new_tokens=news[i]))
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps = 0
    while not engine.is_finished():
        engine.step()
        steps += 1
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    generated = sum(news[i] for i in mine)
    status = pkg._lib.device_status(clear=True)
    runner.exit()
    del runner, engine
    torch.cuda.empty_cache()
    if world > 1:
        t = torch.tensor([ms, float(generated), float(steps), float(sum(costs[i] for i in mine)), float(status)],
                         dtype=torch.float64, device=device)
        allt = [torch.empty_like(t) for _ in range(world)]
        torch.distributed.all_gather(allt, t)
        rows = [x.tolist() for x in allt]
    else:
        rows = [[ms, float(generated), float(steps), float(sum(costs)), float(status)]]
    times = [r[0] for r in rows]
    return {"workload": f"{total_requests} requests, visual rows U[512,8192], outputs U[64,512] (whole blocks), block "
                        f"{wl.block}, threshold {wl.threshold}, temperature {wl.temperature}, at most {wl.requests} in "
                        "flight per GPU, prefill included, run to completion; same set for every N",
            "scaling": "strong", "partitioner": "engine/dp.py:partition_requests (greedy longest-first on a time model: 4 us per prompt token "
                                           "+ 130 us per request-step + 1600 us x the rank's longest stay in steps)",
            "tokens": int(sum(r[1] for r in rows)), "tokens_per_s": round(sum(r[1] for r in rows) / (max(times) * 1e-3), 1),
            "rank_finish_ms": [round(x, 1) for x in times], "rank_tokens": [int(r[1]) for r in rows],
            "rank_steps": [int(r[2]) for r in rows], "rank_cost": [int(r[3]) for r in rows],
            "imbalance_max_over_mean": round(max(times) / (sum(times) / len(times)), 4),
            "device_status": int(max(r[4] for r in rows))}


def measure_tp2_against_one_gpu(pkg, args, rank: int, local_rank: int):
    """At N = 2 the two ranks also form one tensor-parallel pair (o_proj / down_proj all-reduce fused into the
    GEMM epilogues as NVLink peer stores) and time BASELINE config 3 (64 requests) and config 4 (one long
    request); then each rank times the same two workloads alone on its GPU, and rank 0 reports pair against
    single GPU.  The pair serves the same requests as the single GPU."""
    device = f"cuda:{local_rank}"
    pair, one = {}, {}
    for key, steps in (("config3", min(args.steps, 30)), ("config4", min(args.steps, 60))):
        a = argparse.Namespace(steps=steps, warmup=3)
        res, runner, engine = run_workload(pkg, WORKLOADS[key], a, rank, 2, local_rank, tp=2)
        t = torch.tensor([res["dev_ms"], res["e2e_ms"], float(res["status"])], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        dev_ms, e2e_ms, status = t.tolist()
        pair[key] = {"ms_per_step": round(dev_ms / max(res["steps"], 1), 3),
                     "tokens_per_s": round(res["tokens"] / (dev_ms * 1e-3), 1),
                     "e2e_tokens_per_s": round(res["tokens"] / (e2e_ms * 1e-3), 1), "steps": res["steps"],
                     "clocks": res["clocks"], "device_status": int(status)}
        runner.exit()
        del runner, engine
        torch.cuda.empty_cache()
    for key, steps in (("config3", min(args.steps, 30)), ("config4", min(args.steps, 60))):
        a = argparse.Namespace(steps=steps, warmup=3)
        res, runner, engine = run_workload(pkg, WORKLOADS[key], a, 0, 1, local_rank)     # seeds of rank 0 on both
        one[key] = {"ms_per_step": round(res["dev_ms"] / max(res["steps"], 1), 3),
                    "tokens_per_s": round(res["tokens"] / (res["dev_ms"] * 1e-3), 1), "clocks": res["clocks"]}
        runner.exit()
        del runner, engine
        torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"pair": pair, "one_gpu": one,
            "speedup": {k: round(one[k]["ms_per_step"] / pair[k]["ms_per_step"], 3) for k in pair}}


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=330)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="only the headline workload (no config1/batched/parity/"
                    "dp_completion/tp2 keys)")
    ap.add_argument("--workload", default="config2", choices=sorted(WORKLOADS),
                    help="config3: 64 concurrent requests, visual rows uniform in [512, 4096], 2048 new tokens each; "
                         "config4: one request, 4096 visual rows, 4096 new tokens (the TP=2 vs TP=1 comparison); "
                         "config5: one point of the request-parallel sweep (64 requests in flight per GPU out of the "
                         "512 / N share, visual rows uniform in [512, 8192], --block and --threshold set the point)")
    ap.add_argument("--block", type=int, default=32, choices=[8, 16, 32, 64], help="denoising block size")
    ap.add_argument("--threshold", type=float, default=0.9, help="confidence threshold of the unmask rule")
    ap.add_argument("--temperature", type=float, default=1.0,
                    help="sampling temperature; with random weights only a low one (0.02) lets confidences pass the "
                         "threshold, so that steps commit several tokens as they do on a trained model")
    ap.add_argument("--fuse-commit", action="store_true",
                    help="Config.fuse_commit_pass: a block's commit pass also runs the next block's first denoising "
                         "pass (not the reference's schedule; off for the headline number)")
    ap.add_argument("--tp", type=int, default=1, choices=[1, 2], help="2: the two ranks form one tensor-parallel pair")
    ap.add_argument("--requests", type=int, default=0,
                    help="requests in flight per GPU instead of the workload's own count (config3 / config5: the "
                         "batch sizes between one request and 64)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = replace(WORKLOADS[args.workload], block=args.block, threshold=args.threshold, temperature=args.temperature,
                 fuse_commit=args.fuse_commit)
    if args.requests > 0 and wl.requests > 1:
        wl = replace(wl, name=f"{wl.name} with {args.requests} requests in flight", requests=args.requests)
    config = {"workload": wl.describe(), "block_size": wl.block, "requests_per_gpu": wl.requests,
              "parallelism": f"tp{args.tp}" if args.tp == 2 else f"dp{args.gpus}",
              "l2_policy": "per-step weight traffic (3.4 GB) exceeds L2 (126 MB); no explicit flush"}
    if wl.fuse_commit:
        config["fuse_commit_pass"] = True

    if args.impl == "reference":
        if rank != 0:
            return
        steps = min(args.steps, 6)
        tokens, dt, threads, prefix = run_cpu_sample(steps, min(args.warmup, 1), WORKLOADS["config2"])
        value = tokens / dt
        config["ranks"] = "rank 0 alone runs the CPU arm whatever --gpus says; the other ranks exit without work"
        line = {"impl": "reference", "metric": METRIC,
                "value": round(value, 4), "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
                "warmup": min(args.warmup, 1), "ms_per_step": round(dt / steps * 1e3, 2), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": round(value, 4), "unit": "tokens/s", "cores": threads, "kind": "port",
                                 "sample": f"{steps} denoising passes at context {prefix + wl.block} (mid-generation), "
                                           "full-size decoder, reference torch CPU ops restated in oracle/ (a port: "
                                           "the reference is Python and is not installed on this box)"},
                "e2e": {"value": round(value, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    pkg = importlib.import_module("mineru-diffusion_b200")
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    res, runner, engine = run_workload(pkg, wl, args, rank, world, local_rank, tp=args.tp)
    extras = not args.no_extras and args.workload == "config2" and args.tp == 1
    roof = attn = None
    if rank == 0 and args.tp == 1 and wl.requests == 1:
        roof = measure_dominant_kernel(pkg, runner, wl.block)
    runner.exit()
    del runner, engine
    torch.cuda.empty_cache()
    if rank == 0 and args.tp == 1:
        attn = measure_attention(wl.block)
    if args.tp == 2:
        res["tokens"] = res["tokens"] if rank == 0 else 0      # one request served by the pair: count it once
    tokens, dev_ms, e2e_ms = res["tokens"], res["dev_ms"], res["e2e_ms"]
    dp = importlib.import_module("mineru-diffusion_b200.engine.dp")
    tokens, (dev_ms, e2e_ms), (launches, status) = dp.reduce_throughput(tokens, [dev_ms, e2e_ms],
                                                                        [res["launches"], res["status"]],
                                                                        f"cuda:{local_rank}")
    dp_completion = tp2 = None
    if extras and world > 1:
        dp_completion = run_dp_completion(pkg, args, rank, world, local_rank)
        if world == 2:
            tp2 = measure_tp2_against_one_gpu(pkg, args, rank, local_rank)
    if rank == 0:
        line = {"metric": METRIC,
                "value": round(tokens / (dev_ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": res["steps"], "warmup": args.warmup, "ms_per_step": round(dev_ms / max(res["steps"], 1), 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": config,
                "per_gpu": round(tokens / (dev_ms * 1e-3) / max(args.gpus if args.tp == 1 else 1, 1), 2),
                "e2e": {"value": round(tokens / (e2e_ms * 1e-3), 2), "unit": "tokens/s",
                        "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                        "ms_per_step": round(e2e_ms / max(res["steps"], 1), 4)},
                "gpu_launches": launches, "device_status": status, "clocks": res["clocks"], "roofline": roof,
                "tokens": tokens}
        if attn:
            line.update(attn)
        if extras and world == 1:
            line["dp_completion"] = run_dp_completion(pkg, args, 0, 1, local_rank)
            line["config1"] = measure_config1()
            line["batched"] = measure_batched(pkg, args, local_rank)
        if dp_completion is not None:
            line["dp_completion"] = dp_completion
        if tp2 is not None:
            line["tp2"] = tp2
        if args.gpus == 1 and not args.no_cpu_baseline and args.tp == 1:
            prepared = cpu_weights()
            ctok, cdt, threads, prefix = run_cpu_sample(3, 1, WORKLOADS["config2"], prepared=prepared)
            line["cpu_baseline"] = {"value": round(ctok / cdt, 4), "unit": "tokens/s", "cores": threads, "kind": "port",
                                    "sample": f"3 denoising passes at context {prefix + wl.block} (mid-generation), full-size "
                                              "decoder, reference torch CPU ops restated in oracle/"}
            if extras:
                line["parity"] = run_parity(pkg, prepared, f"cuda:{local_rank}")
        else:
            line["cpu_baseline"] = None
        if status:
            raise SystemExit(f"device status word {status:#x} after the timed steps: the numbers are void")
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
