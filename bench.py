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
work of each step); ``e2e`` = the same tokens divided by the bracketed wall
time of the K calls through the public API, host->device and device->host
copies included.  ``roofline`` is measured live for the dominant kernel symbol
(the weight-streaming GEMM writing split-k slices: qkv, o_proj and down_proj
of every layer) by launching it over the 28 layers' distinct weights (far
beyond L2) inside a CUDA graph between two events; ``roofline.per_op`` lists
every GEMM of a step, the gate/up projection and the LM head included.
``cpu_baseline`` times the CPU oracle (the reference's torch ops on the host
cores) on a bounded sample of the same workload.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

BLOCK = 32
VISUAL_ROWS = 1024
TEXT_IDS = 32
NEW_TOKENS = 1024
THRESHOLD = 0.9
REQUESTS = 1
TEMPERATURE = 1.0
VISUAL_MAX = 4096      # upper end of the per-request visual row count when several requests run
WEIGHT_SEED = 20260320


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
def make_request(pkg, dcfg, seed: int, device, visual_rows: int | None = None):
    g = torch.Generator().manual_seed(seed)
    rows = VISUAL_ROWS if visual_rows is None else visual_rows
    visual = torch.randn(rows, dcfg.hidden_size, generator=g).to(torch.bfloat16)
    text = torch.randint(0, 151000, (TEXT_IDS,), generator=g).tolist()
    ids = [0] * rows + text                 # the visual positions' ids are never embedded
    sp = pkg.SamplingParams(temperature=TEMPERATURE, max_new_tokens=NEW_TOKENS, ignore_eos=True, dynamic_threshold=THRESHOLD)
    return pkg.Sequence(ids, sp, denoising_block_size=BLOCK, mask_token_id=151669,
                        inputs_embeds=visual.pin_memory() if device != "cpu" else visual)


def run_ours(args, rank: int, world: int, local_rank: int):
    pkg = importlib.import_module("mineru-diffusion_b200")
    device = f"cuda:{local_rank}"
    torch.cuda.set_device(device)
    dcfg = pkg.DecoderConfig()
    total_len = VISUAL_ROWS + TEXT_IDS + NEW_TOKENS + BLOCK
    max_len = max(4096, (total_len + 255) // 256 * 256)
    nreq = REQUESTS
    if nreq > 1:
        # config 3: per-request visual rows uniform in [512, 4096]; pages for every request's full length
        vg = torch.Generator().manual_seed(3 + (0 if args.tp == 2 else rank))   # a TP pair serves the same requests
        visual_rows = torch.randint(512, VISUAL_MAX + 1, (nreq,), generator=vg).tolist()
        pages = sum((v + TEXT_IDS + NEW_TOKENS + BLOCK + 255) // 256 for v in visual_rows) + 2
        max_len = (VISUAL_MAX + TEXT_IDS + NEW_TOKENS + BLOCK + 255) // 256 * 256
    else:
        visual_rows = [VISUAL_ROWS]
        pages = (total_len + 255) // 256 + 1
    cfg = pkg.Config(max_num_batched_tokens=max(max_len, 16384 if nreq > 1 else 0), max_num_seqs=nreq,
                     max_model_len=max_len, enforce_eager=False, num_kvcache_blocks=pages, decoder_config=dcfg,
                     tensor_parallel_size=args.tp, block_size=BLOCK, fuse_commit_pass=getattr(args, "fuse_commit", False))
    # tensor-parallel pair: both ranks serve the same request with the same noise; replicas: one request each
    seed = 2 if args.tp == 2 else 2 + rank
    runner = pkg.ModelRunner(cfg, rank=rank if args.tp == 2 else 0, weight_seed=WEIGHT_SEED, noise="gumbel",
                             noise_seed=seed, device=device)
    engine = pkg.LLMEngine(cfg, runner)
    for i, v in enumerate(visual_rows):
        engine.add_sequence(make_request(pkg, dcfg, seed=seed + 1000 * i, device=device, visual_rows=v))
    stream = torch.cuda.current_stream()

    # prefill (first denoising pass of the first block; several batches when there are many requests)
    # + warm-up decode steps, untimed
    engine.step()
    while engine.scheduler.waiting:
        engine.step()
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()

    # per-step device time: events around the GPU work of each step
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    sampler = ClockSampler(local_rank)
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    sampler.start()
    tokens = 0
    steps_done = 0
    launches_per_step = runner.launches_per_decode_step(nreq)
    wall0 = time.perf_counter()
    e_all0 = torch.cuda.Event(enable_timing=True)
    e_all1 = torch.cuda.Event(enable_timing=True)
    e_all0.record(stream)
    for i in range(args.steps):
        if engine.is_finished():
            break
        runner.step_events = ev[i]
        _, n = engine.step()
        tokens += -n if n < 0 else 0
        steps_done += 1
    e_all1.record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - wall0
    if world > 1:
        torch.distributed.barrier()
    clocks = sampler.stop()
    runner.step_events = None
    dev_ms = sum(a.elapsed_time(b) for a, b in ev[:steps_done])
    e2e_ms = e_all0.elapsed_time(e_all1)
    h2d = runner.inputs.nbytes        # the packed step inputs (first node of the step graph)
    d2h = nreq * (BLOCK * 8 + BLOCK + 4)

    roof = measure_dominant_kernel(pkg, runner) if rank == 0 and args.tp == 1 and nreq == 1 else None
    attn = measure_block_attention() if rank == 0 and args.tp == 1 else None
    return dict(attention=attn, tokens=tokens, steps=steps_done, dev_ms=dev_ms, e2e_ms=max(e2e_ms, wall * 1e3), clocks=clocks,
                h2d=h2d, d2h=d2h, launches=launches_per_step * steps_done, roofline=roof,
                ctx_end=len(engine.scheduler.running[0]) if engine.scheduler.running else total_len)


def measure_block_attention():
    """The second half of the metric: HBM GB/s of the block attention over the
    paged cache at prefixes >= 4K (64 requests, prefix lengths U[4096, 8192], the
    decoder's 16 query / 8 KV heads, block 32; 1.7 GB of K/V per launch, far
    beyond L2), ten launches in a CUDA graph between two events."""
    mb = importlib.import_module("mineru-diffusion_b200.microbench")
    peaks = {}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
    peak = float(peaks.get("hbm_gbs", 6650.0))
    try:
        r = mb.attn_case(64, (4096, 8192), block=BLOCK, hq=16, hkv=8, reps=10)
    except torch.OutOfMemoryError:
        return None
    achieved = r["bytes"] / (r["ms"] * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
            "peak_source": "measured" if peaks else "fallback", "us_per_launch": round(r["ms"] * 1e3, 1),
            "workload": "block attention over the paged KV cache, 64 requests, prefix U[4096,8192], 16q/8kv heads x 128, "
                        "block 32, 256-token pages"}


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


def measure_dominant_kernel(pkg, runner):
    """Live roofline of the step's GEMM kernels at m = 32: each is launched once
    per layer over the 28 layers' distinct weights (0.2 - 1.4 GB per sweep, far
    beyond the 126 MB L2)."""
    peaks = {}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
    peak = float(peaks.get("hbm_gbs", 6650.0))
    eng, dcfg, ops = runner.engine, runner.dcfg, pkg.ops
    m = BLOCK
    h, inter, d = dcfg.hidden_size, dcfg.intermediate_size, dcfg.head_dim
    hq, hkv, vocab = dcfg.num_attention_heads, dcfg.num_key_value_heads, dcfg.vocab_size
    nqkv = (hq + 2 * hkv) * d
    layers = runner.weights.layers
    x, act, attn = eng.x[:m], eng.act[:m], eng.attn[:m].view(m, hq * d)
    tc = ops.get_option(ops.OPT_STREAM_KERNEL) == 0
    kname = "gemm_ws_kernel" if tc else "gemm_skinny_kernel"

    def parts(ks, n):
        return eng.partials[:ks * m * n].view(ks, m, n)

    temps = torch.ones(1, device=x.device)
    cases = [
        ("gate_up + SiLU*mul", f"{kname}<swiglu>", 2 * inter * h * 2 + m * h * 2 + m * inter * 2, len(layers),
         lambda: [ops.gateup_swiglu(x, lw.gate_up, out=act) for lw in layers]),
        ("qkv", f"{kname}<partial>", nqkv * h * 2 + m * h * 2 + eng.ks_qkv * m * nqkv * 4, len(layers),
         lambda: [ops.gemm_splitk_partials(x, lw.qkv, eng.ks_qkv, parts(eng.ks_qkv, nqkv)) for lw in layers]),
        ("o_proj", f"{kname}<partial>", h * hq * d * 2 + m * hq * d * 2 + eng.ks_o * m * h * 4, len(layers),
         lambda: [ops.gemm_splitk_partials(attn, lw.o, eng.ks_o, parts(eng.ks_o, h)) for lw in layers]),
        ("down_proj", f"{kname}<partial>", h * inter * 2 + m * inter * 2 + eng.ks_down * m * h * 4, len(layers),
         lambda: [ops.gemm_splitk_partials(act, lw.down, eng.ks_down, parts(eng.ks_down, h)) for lw in layers]),
        ("lm_head + sampler scan", f"{kname}<lm_head> + sampler_finalize_kernel", vocab * h * 2 + m * h * 2 + m * 16, 2,
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
    return {"bound": "hbm", "kernel": f"{kname}<partial> (qkv, o_proj, down_proj launches of a step averaged, m=32)",
            "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
            # dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in
            # profiles/gemm_ws_kernel_partial_config2_m32.md (same three launches, averaged)
            "traffic": 17051819 if tc else None,
            "peak_source": "measured" if peaks else "fallback", "bytes_per_launch": round(nbytes),
            "us_per_launch": round(us, 2), "per_op": out}


# ----------------------------------------------------------------------------- CPU arm
def run_cpu_sample(steps: int, warmup: int, threads: int | None = None):
    """The reference's torch CPU path (restated in oracle/) on a bounded sample
    of the workload: decode-form denoising passes of the full-size decoder at
    the context length reached half way through generation, KV cache filled
    with seeded noise instead of a CPU prefill."""
    from oracle import nano_oracle as orc
    # every core this process may run on (a torchrun launch sets OMP_NUM_THREADS=1, which would leave 1 thread)
    torch.set_num_threads(threads or len(os.sched_getaffinity(0)))
    orc.use_native_linear(True)
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
    for _ in range(cfg.num_hidden_layers - 1):     # distinct memory per layer, same distribution
        layers.append(orc.LayerWeights(base.input_ln, base.qkv.roll(1, 0).contiguous(), base.q_norm, base.k_norm,
                                       base.o.roll(1, 0).contiguous(), base.post_ln,
                                       base.gate_up.roll(1, 0).contiguous(), base.down.roll(1, 0).contiguous()))
    embed = mat(cfg.vocab_size, h)
    weights = orc.DecoderWeights(embed, layers, torch.ones(h, dtype=bf), embed.roll(1, 0).contiguous())
    prefix = VISUAL_ROWS + TEXT_IDS + NEW_TOKENS // 2
    pages = (prefix + BLOCK + 255) // 256
    runner = orc.OracleModelRunner(cfg, weights, num_pages=pages, block_size=BLOCK, mask_token_id=151669,
                                   noise_fn=lambda step, shape: -torch.empty(shape).exponential_(generator=g).log())
    runner.decoder.kv_cache.normal_(generator=g)

    class Req:
        def __init__(self):
            from types import SimpleNamespace
            self.seq_id = 0
            self.token_ids = [1] * prefix
            self.block_table = list(range(pages))
            self.num_cached_tokens = 0
            self.temperature = 1.0
            self.mask_token_id = 151669
            self.sampling_params = SimpleNamespace(dynamic_threshold=THRESHOLD)
            self.current_denoising_block = torch.full((BLOCK,), 151669, dtype=torch.int64)
            self.current_step_map = torch.zeros(BLOCK, dtype=torch.int32)
            self.current_denoise_step = 0

        def __len__(self):
            return len(self.token_ids)

        def __getitem__(self, k):
            return self.token_ids[k]

    req = Req()
    with torch.inference_mode():
        for _ in range(warmup):
            runner.run([req], False)
        t0 = time.perf_counter()
        tokens = 0
        for _ in range(steps):
            tokens += runner.run([req], False)
        dt = time.perf_counter() - t0
    orc.use_native_linear(False)
    return tokens, dt, torch.get_num_threads(), prefix


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=330)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="config2", choices=["config2", "config3", "config4", "config5"],
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
    args = ap.parse_args()
    global VISUAL_ROWS, NEW_TOKENS, REQUESTS, BLOCK, THRESHOLD, VISUAL_MAX, TEMPERATURE
    BLOCK, THRESHOLD, TEMPERATURE = args.block, args.threshold, args.temperature
    if args.workload == "config5":
        NEW_TOKENS, REQUESTS, VISUAL_MAX = 2048, 64, 8192
    if args.workload == "config4":
        VISUAL_ROWS, NEW_TOKENS = 4096, 4096
    if args.workload == "config3":
        NEW_TOKENS, REQUESTS = 2048, 64
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": "config2: full decoder (28 layers, hidden 2048, 16q/8kv heads, vocab 151936), 1 request per "
                          "GPU, 1024 synthetic visual rows + 32 text ids, 1024 new tokens, block 32, threshold 0.9, "
                          "temperature 1.0",
              "block_size": BLOCK, "requests_per_gpu": 1,
              "parallelism": f"tp{args.tp}" if args.tp == 2 else f"dp{args.gpus}",
              "l2_policy": "per-step weight traffic (3.4 GB) exceeds L2 (126 MB); no explicit flush"}

    if args.impl == "reference":
        if rank != 0:
            return
        steps = min(args.steps, 6)
        tokens, dt, threads, prefix = run_cpu_sample(steps, min(args.warmup, 1))
        value = tokens / dt
        line = {"impl": "reference", "metric": "decoded tokens/sec per B200 (block diffusion, bf16)",
                "value": round(value, 4), "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
                "warmup": min(args.warmup, 1), "ms_per_step": round(dt / steps * 1e3, 2), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": round(value, 4), "unit": "tokens/s", "cores": threads, "kind": "port",
                                 "sample": f"{steps} denoising passes at context {prefix + BLOCK} (mid-generation), "
                                           "full-size decoder, reference torch CPU ops restated in oracle/"},
                "e2e": {"value": round(value, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if args.workload == "config3":
        config["workload"] = ("config3: full decoder, 64 concurrent requests on one GPU, visual rows uniform in "
                              "[512, 4096] + 32 text ids, 2048 new tokens each, block 32, threshold 0.9, temperature 1.0")
        config["requests_per_gpu"] = 64
    if args.workload == "config5":
        config["workload"] = (f"config5 sweep point: full decoder, 64 requests in flight per GPU (of 512 / N), visual "
                              f"rows uniform in [512, 8192] + 32 text ids, block {BLOCK}, threshold {THRESHOLD}, "
                              "temperature 1.0")
        config["requests_per_gpu"] = 64
    config["block_size"] = BLOCK
    if args.workload == "config4":
        config["workload"] = ("config4: full decoder, 1 request, 4096 synthetic visual rows + 32 text ids, 4096 new "
                              "tokens, block 32, threshold 0.9, temperature 1.0")
    if args.fuse_commit:
        config["fuse_commit_pass"] = True
    if TEMPERATURE != 1.0:
        config["workload"] = config["workload"].replace("temperature 1.0", f"temperature {TEMPERATURE}")
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device(f"cuda:{local_rank}"))
    res = run_ours(args, rank, world, local_rank)
    if args.tp == 2:
        res["tokens"] = res["tokens"] if rank == 0 else 0      # one request served by the pair: count it once
    tokens, dev_ms, e2e_ms = res["tokens"], res["dev_ms"], res["e2e_ms"]
    dp = importlib.import_module("mineru-diffusion_b200.engine.dp")
    tokens, (dev_ms, e2e_ms), (launches,) = dp.reduce_throughput(tokens, [dev_ms, e2e_ms], [res["launches"]],
                                                                 f"cuda:{local_rank}")
    if rank == 0:
        cpu = None
        if args.gpus == 1 and not args.no_cpu_baseline:
            ctok, cdt, threads, prefix = run_cpu_sample(3, 1)
            cpu = {"value": round(ctok / cdt, 4), "unit": "tokens/s", "cores": threads, "kind": "port",
                   "sample": f"3 denoising passes at context {prefix + BLOCK} (mid-generation), full-size decoder, "
                             "reference torch CPU ops restated in oracle/"}
        line = {"metric": "decoded tokens/sec per B200 (block diffusion, bf16)",
                "value": round(tokens / (dev_ms * 1e-3), 2), "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": res["steps"], "warmup": args.warmup, "ms_per_step": round(dev_ms / max(res["steps"], 1), 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": config,
                "e2e": {"value": round(tokens / (e2e_ms * 1e-3), 2), "unit": "tokens/s",
                        "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                        "ms_per_step": round(e2e_ms / max(res["steps"], 1), 4)},
                "gpu_launches": launches, "clocks": res["clocks"], "roofline": res["roofline"], "cpu_baseline": cpu,
                "staircase_attn": res.get("attention"), "tokens": tokens}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
