"""Drop-in for the reference's ``ModelRunner`` on one B200.

Same constructor shape, ``call("run", seqs, is_prefill) -> int`` contract and
side effects on the ``Sequence`` objects as
``engines/nano_dvlm/nanovllm/engine/model_runner.py:15-219`` of the reference;
the decoder underneath is ``DecoderEngine`` (hand-written sm_100a kernels via
libmdb200).  The sampler's statistics and the unmask rule run on the device;
one packed host->device copy feeds a step and one device->host copy returns
the new block ids, transfer mask and counts.

The vision tower is outside this path: a request carries the rows that stand
for its output in ``Sequence.inputs_embeds`` and they overwrite the token
embeddings of the first prompt positions, which is what
``DMLLM._prepare_inputs_embeds`` does with the projector's rows
(``nanovllm/models/dmllm.py:136-157``).
"""
from __future__ import annotations

import torch

from .. import ops
from ..decoder import DecoderEngine, DecoderWeights
from .config import Config, DecoderConfig
from .context import Context
from .sequence import Sequence
from .step_inputs import build_decode_inputs, build_prefill_inputs, fill_decode_inputs_small


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


class _StepInputs:
    """One pinned host buffer and its device twin holding every per-step input
    of the decode form, so a step costs a single host->device copy.

    Layout (all offsets 16-byte aligned): ids int64 [bs*B] | step uint32 [4] |
    positions int64 [bs*B] | slots int32 [bs*B] | ctx_lens int32 [bs] |
    block_tables int32 [bs*max_pages] | temperatures fp32 [bs].  The first two
    fields are what a step changes on the device itself (block ids handed on by
    the unmask rule, step counters incremented): a step launched ahead of the
    host copies only the rest (``o_pos`` onwards)."""

    def __init__(self, max_bs: int, block: int, max_pages: int, device):
        self.max_bs, self.block, self.max_pages = max_bs, block, max_pages
        n = max_bs * block
        off = 0
        self.o_ids = off; off += _round_up(n * 8, 16)
        self.o_step = off; off += 16
        self.o_pos = off; off += _round_up(n * 8, 16)
        self.o_slots = off; off += _round_up(n * 4, 16)
        self.o_ctx = off; off += _round_up(max_bs * 4, 16)
        self.o_tab = off; off += _round_up(max_bs * max_pages * 4, 16)
        self.o_temp = off; off += _round_up(max_bs * 4, 16)
        self.nbytes = off
        self.host = torch.zeros(off, dtype=torch.uint8, pin_memory=True)
        self.dev = torch.zeros(off, dtype=torch.uint8, device=device)

    def _view(self, base, off, count, dtype):
        return base[off:off + count * torch.empty(0, dtype=dtype).element_size()].view(dtype)

    def views(self, base):
        n = self.max_bs * self.block
        return dict(
            ids=self._view(base, self.o_ids, n, torch.int64).view(self.max_bs, self.block),
            pos=self._view(base, self.o_pos, n, torch.int64).view(self.max_bs, self.block),
            slots=self._view(base, self.o_slots, n, torch.int32).view(self.max_bs, self.block),
            ctx=self._view(base, self.o_ctx, self.max_bs, torch.int32),
            tab=self._view(base, self.o_tab, self.max_bs * self.max_pages, torch.int32).view(self.max_bs, self.max_pages),
            temp=self._view(base, self.o_temp, self.max_bs, torch.float32),
            step=self._view(base, self.o_step, 4, torch.int32),
        )


class _NextBlock:
    """Stand-in for the block a request opens after the one it is committing: a fresh masked block at the
    positions behind the committed one, on the same pages (``Config.fuse_commit_pass``).  Quacks like a
    Sequence for the builders of the step inputs."""
    __slots__ = ("seq", "current_denoising_block", "block_table", "temperature")

    def __init__(self, seq: Sequence):
        self.seq = seq
        self.current_denoising_block = seq._fresh_block()
        self.block_table = seq.block_table
        self.temperature = seq.temperature

    def __len__(self):
        return len(self.seq) + self.seq.denoising_block_size


class ModelRunner:

    def __init__(self, config: Config, rank: int = 0, event=None, weights: DecoderWeights | None = None,
                 weight_seed: int = 20260320, noise: str = "gumbel", noise_seed: int = 0, device: str | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("ModelRunner needs a CUDA device: the decode path has no CPU implementation")
        if config.tensor_parallel_size not in (1, 2):
            raise NotImplementedError("tensor_parallel_size must be 1 or 2 (more GPUs serve as request-parallel replicas)")
        if noise not in ("gumbel", "none", "explicit"):
            raise ValueError("noise must be 'gumbel', 'none' or 'explicit'")
        self.config = config
        self.rank = rank
        self.event = event
        self.world_size = config.tensor_parallel_size
        self.block_size = config.block_size
        self.kvcache_block_size = config.kvcache_block_size
        if self.kvcache_block_size != Sequence.kvcache_block_size:
            raise AssertionError("only 256-token pages are consistent end to end")
        self.enforce_eager = config.enforce_eager
        self.device = torch.device(device or f"cuda:{rank}")
        torch.cuda.set_device(self.device)
        self.full_dcfg = self._decoder_config(config)
        self.dcfg = self.full_dcfg
        from .. import loader
        model_dir = getattr(config, "model", None)
        from_checkpoint = weights is None and loader.has_checkpoint(model_dir)
        if self.world_size == 2:
            # One process per GPU, every rank calling run() with the same requests (the sampler's decisions
            # are bit-identical on both ranks, so the two schedulers stay in step without a control channel).
            from .. import tp as tp_mod
            if not torch.distributed.is_initialized():
                torch.distributed.init_process_group("nccl", init_method="tcp://127.0.0.1:2333", world_size=2,
                                                     rank=rank, device_id=self.device)
            self.dcfg = tp_mod.shard_config(self.full_dcfg, 2)
        if from_checkpoint:
            # the model directory holds safetensors files: read this rank's share, as the reference's load_model does
            self.weights = loader.load_decoder_weights(model_dir, self.full_dcfg, self.device, rank if self.world_size == 2
                                                       else 0, self.world_size)
        else:
            full = weights if weights is not None else DecoderWeights.random_init(self.full_dcfg, weight_seed, self.device)
            if self.world_size == 2:
                self.weights = tp_mod.shard_weights(full, self.full_dcfg, rank, 2)
                del full
            else:
                self.weights = full
        self.noise = noise
        self.noise_seed = noise_seed
        self.noise_fn = None          # explicit mode: fn(step_index, m, vocab) -> fp32 [m, vocab] CUDA tensor
        self.step_index = 0
        self.allocate_kv_cache()
        b = self.block_size
        self.fuse_commit_pass = bool(getattr(config, "fuse_commit_pass", False))
        # with fused commit passes a request can stand in a step twice (the block it commits + the one it opens)
        self.max_bs = min(config.max_num_seqs * (2 if self.fuse_commit_pass else 1), 512)
        max_tokens = max(config.max_num_batched_tokens + config.max_num_seqs * b, self.max_bs * b)
        max_tokens = min(max_tokens, config.max_model_len * config.max_num_seqs + config.max_num_seqs * b)
        self.engine = DecoderEngine(self.dcfg, self.weights, self.kv_cache, max_tokens, self.max_bs, b,
                                    tp_rank=rank if self.world_size == 2 else 0, tp_size=self.world_size)
        self.max_pages = (config.max_model_len + b + self.kvcache_block_size - 1) // self.kvcache_block_size
        self.inputs = _StepInputs(self.max_bs, b, self.max_pages, self.device)
        self.hv = self.inputs.views(self.inputs.host)
        self.hn = {k: v.numpy() for k, v in self.hv.items()}   # numpy views of the pinned buffer
        self.dv = self.inputs.views(self.inputs.dev)
        self.tp_pair = None
        if self.world_size == 2:
            from .. import tp as tp_mod
            self.tp_pair = tp_mod.TensorParallelPair(rank, self.device, self.dcfg.hidden_size, self.engine.ks_o,
                                                     self.engine.ks_down,
                                                     max(ops.lmhead_workspace_bytes(64, self.dcfg.vocab_size),
                                                         int(ops._lib.lib().mdb_lmhead_tp_workspace_bytes(
                                                             self.max_bs * b, self.dcfg.vocab_size))),
                                                     many_rows=max_tokens)
            # word 1 of the step slot is the flag epoch: step index + 1, so that real steps never reuse the
            # sequence numbers of the warm-up launches made while graphs are captured (epoch 0)
            self.engine.attach_tp(self.tp_pair, self.dv["step"][1:2])
        # sampler state: one flat device buffer and its pinned mirror, laid out per batch size as
        # ids int64 [bs, B] | counts int32 [bs] | transfer u8 [bs, B], so the results of a step come back in one copy
        # ... followed by the device status word of the step (4 bytes)
        # ... twice: a step launched ahead writes the other set while the host still reads this one
        self.res_dev = [torch.zeros(self.max_bs * (9 * b + 4) + 4, dtype=torch.uint8, device=self.device)
                        for _ in range(2)]
        self.res_host = [torch.zeros(self.max_bs * (9 * b + 4) + 4, dtype=torch.uint8, pin_memory=True)
                         for _ in range(2)]
        self._done = [torch.cuda.Event(), torch.cuda.Event()]   # results of set p have reached pinned memory
        self._parity = 0
        self._tails: dict[tuple, torch.cuda.CUDAGraph] = {}     # (bs, set, mask id, threshold) -> graph
        self.quota_host = torch.ones(self.max_bs, dtype=torch.int32, pin_memory=True)
        self.quota_dev = torch.ones(self.max_bs, dtype=torch.int32, device=self.device)
        self._res_views: dict[tuple, tuple] = {}
        self._decode_key = None       # lengths and page counts the pinned step inputs were last built for
        self._decode_seqs: list = []  # ... and the requests themselves
        self._last_rows, self._last_blocks = None, None   # blocks handed to the requests after the last step
        self._decode_max_ctx = 0
        self.graphs: dict[int, tuple[torch.cuda.CUDAGraph, int]] = {}
        self.graph_bs: list[int] = []
        self.last: dict = {}
        self.keep_last = False        # tests: keep x0 / confidence / hidden of the last step
        # benchmark: CUDA events around the GPU work of a step -- one (start, end) pair used for every step, or an
        # iterator of pairs, one taken per step launched; last_step_events = the pair of the step last collected
        self.step_events = None
        self.last_step_events = None
        # launch-ahead (Config.launch_ahead): the step launched before the scheduler asked for it
        self.launch_ahead = bool(getattr(config, "launch_ahead", False))
        self._ahead = None            # record of the step launched ahead (see _launch_ahead)
        self._pair = None             # event pair of the step being launched / collected
        self.ahead_hits = self.ahead_misses = 0
        if not self.enforce_eager:
            self.capture_cudagraph()

    @staticmethod
    def _decoder_config(config) -> DecoderConfig:
        """Decoder dimensions of a ``Config``: this package's ``decoder_config`` field, or what the reference's
        ``Config`` carries instead (``hf_config.language_model_config`` / ``text_config`` read from config.json,
        ``nanovllm/config.py:16-31,56-59``)."""
        dcfg = getattr(config, "decoder_config", None)
        if dcfg is not None:
            return dcfg
        hf = getattr(config, "hf_config", None)
        text = None
        for name in ("language_model_config", "text_config"):
            text = getattr(hf, name, None) if hf is not None else None
            if text is not None:
                break
        if text is None:
            text = hf
        if text is None:
            raise AssertionError("the config names no decoder dimensions (decoder_config or hf_config)")
        if isinstance(text, dict):
            from types import SimpleNamespace
            text = SimpleNamespace(**text)
        return DecoderConfig.from_namespace(text)

    # ------------------------------------------------------------------ control plane
    def call(self, method_name, *args):
        return getattr(self, method_name)(*args)

    def exit(self):
        torch.cuda.synchronize(self.device)      # a step launched ahead may still be running
        self._ahead = None
        self.graphs.clear()
        self._tails.clear()
        if self.tp_pair is not None:
            self.tp_pair.close()
            self.tp_pair = None

    # ------------------------------------------------------------------ memory
    def allocate_kv_cache(self):
        """kv_cache[2, L, pages, 256, Hkv, D] bf16, pages from the free-memory
        budget unless ``config.num_kvcache_blocks`` is preset (> 0)."""
        config, d = self.config, self.dcfg
        block_bytes = 2 * d.num_hidden_layers * self.kvcache_block_size * d.num_key_value_heads * d.head_dim * 2
        if config.num_kvcache_blocks <= 0:
            free, total = torch.cuda.mem_get_info(self.device)
            used = total - free
            budget = int(total * config.gpu_memory_utilization) - used
            # leave room for the activation buffers allocated after the cache
            reserve = 6 << 30
            config.num_kvcache_blocks = (budget - reserve) // block_bytes
        if config.num_kvcache_blocks <= 0:
            raise AssertionError("no memory left for the KV cache")
        self.kv_cache = torch.zeros(2, d.num_hidden_layers, config.num_kvcache_blocks, self.kvcache_block_size,
                                    d.num_key_value_heads, d.head_dim, dtype=torch.bfloat16, device=self.device)

    # ------------------------------------------------------------------ host -> step tensors
    def prepare_prefill(self, seqs: list[Sequence]):
        inp = build_prefill_inputs(seqs, self.block_size)
        dev = self.device

        def up(a):
            return torch.from_numpy(a).pin_memory().to(dev, non_blocking=True)

        cu_q = up(inp["cu_seqlens"])
        ctx = Context(True, cu_q, cu_q, inp["max_seqlen"], inp["max_seqlen"], up(inp["slot_mapping"]), None, None,
                      self.block_size)
        return up(inp["input_ids"]), up(inp["positions"]), ctx, inp["cu_seqlens"].tolist()

    def _result_views(self, bs: int, p: int = 0):
        """Views of result set ``p`` of the sampler-state buffers for a step of ``bs`` requests:
        (device bytes, pinned bytes, device ids/counts/transfer, pinned ids and numpy views of the pinned
        counts/transfer, device status word, numpy view of its pinned copy)."""
        v = self._res_views.get((bs, p))
        if v is None:
            b = self.block_size
            o1, o2, o3 = bs * b * 8, bs * b * 8 + bs * 4, bs * (9 * b + 4)
            dev, pinned = self.res_dev[p], self.res_host[p]
            def split(buf):
                return (buf[:o1].view(torch.int64).view(bs, b), buf[o1:o2].view(torch.int32), buf[o2:o3].view(bs, b))
            host = split(pinned)
            v = ((dev[:o3 + 4], pinned[:o3 + 4]) + split(dev)
                 + (host[0], host[1].numpy(), host[2].numpy())
                 + (dev[o3:o3 + 4].view(torch.int32), pinned[o3:o3 + 4].view(torch.int32).numpy()))
            self._res_views[(bs, p)] = v
        return v

    def prepare_decode(self, seqs: list[Sequence], copy: bool = True):
        """Fills the packed pinned buffer and (``copy``) starts its copy; returns the longest context.
        While the same requests stay on the same blocks (one denoising step after another) only the
        token ids and the step counter change, so everything else is left as the last step wrote it."""
        b, bs = self.block_size, len(seqs)
        hn = self.hn
        # The cached inputs belong to these very objects (kept referenced, so that their identity cannot pass to
        # another request), at these lengths, holding this many pages.
        key = (tuple(map(len, seqs)), tuple(len(seq.block_table) for seq in seqs))
        held = self._decode_seqs
        if key == self._decode_key and len(held) == bs and all(a is b for a, b in zip(seqs, held)):
            ids, rows = hn["ids"], self._last_rows
            if rows is not None and len(rows) == bs:
                # the blocks handed out after the last step, in one copy; a request that has started a new
                # block since holds another tensor
                ids[:bs] = self._last_blocks
                for i, seq in enumerate(seqs):
                    if seq.current_denoising_block is not rows[i]:
                        ids[i] = seq.current_denoising_block.numpy()
            else:
                for i, seq in enumerate(seqs):
                    ids[i] = seq.current_denoising_block.numpy()
        elif bs <= 4:
            hn["slots"].fill(-1)
            hn["ctx"].fill(0)
            self._decode_max_ctx = fill_decode_inputs_small(seqs, b, hn["ids"], hn["pos"], hn["slots"], hn["ctx"],
                                                            hn["tab"])
            for i, seq in enumerate(seqs):
                hn["temp"][i] = seq.temperature
            self._decode_key, self._decode_seqs = key, list(seqs)
        else:
            inp = build_decode_inputs(seqs, b)
            width = inp["block_tables"].shape[1]
            if width > self.max_pages:
                raise AssertionError("page table wider than max_model_len allows")
            hn["slots"].fill(-1)
            hn["ctx"].fill(0)
            hn["ids"][:bs] = inp["input_ids"]
            hn["pos"][:bs] = inp["positions"]
            hn["slots"][:bs] = inp["slot_mapping"]
            hn["ctx"][:bs] = inp["context_lens"]
            hn["tab"][:bs, :width] = inp["block_tables"]
            for i, seq in enumerate(seqs):
                hn["temp"][i] = seq.temperature
            self._decode_key, self._decode_seqs = key, list(seqs)
            self._decode_max_ctx = int(inp["context_lens"].max())
        hn["step"][0] = self.step_index
        hn["step"][1] = self.step_index + 1
        if copy:
            self.inputs.dev.copy_(self.inputs.host, non_blocking=True)
        return self._decode_max_ctx

    def prepare_sample(self, seqs: list[Sequence]) -> torch.Tensor:
        t = torch.tensor([seq.temperature for seq in seqs], dtype=torch.float32, pin_memory=True)
        return t.to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ forward passes
    def _noise_args(self, m: int):
        if self.noise == "gumbel":
            return dict(seed=self.noise_seed)
        if self.noise == "explicit":
            if self.noise_fn is None:
                raise RuntimeError("noise='explicit' needs runner.noise_fn")
            return dict(noise=self.noise_fn(self.step_index, m, self.dcfg.vocab_size))
        return {}

    def _decode_body(self, bs: int, nsplit: int):
        """Everything of a decode step that depends only on device buffers:
        embedding gather, layer stack, LM head + sampler statistics."""
        b = self.block_size
        m = bs * b
        dv, eng = self.dv, self.engine
        ops.gather_rows(self.weights.embed, dv["ids"][:bs].reshape(-1), out=eng.embeds[:m])
        ctx = Context(False, slot_mapping=dv["slots"][:bs], context_lens=dv["ctx"][:bs],
                      block_tables=dv["tab"][:bs], block_size=b)
        hidden = eng.forward(m, dv["pos"][:bs], ctx, nsplit=nsplit)
        kw = self._noise_args(m)
        if "seed" in kw:
            kw["step_dev"] = dv["step"]
        eng.sample(hidden, dv["temp"][:bs], **kw)
        return hidden

    @torch.inference_mode()
    def run_model_decode(self, seqs: list[Sequence]):
        bs = len(seqs)
        use_graph = (not self.enforce_eager) and self.noise != "explicit" and bs <= self.max_bs and self.graph_bs
        max_ctx = self.prepare_decode(seqs, copy=not use_graph)   # a graph starts with the copy of the packed inputs
        self._pair = self._next_event_pair()
        if self._pair is not None:
            self._pair[0].record()
        if use_graph:
            o = self.inputs.o_pos
            self.inputs.dev[:o].copy_(self.inputs.host[:o], non_blocking=True)   # block ids, step counters
            gbs = next(x for x in self.graph_bs if x >= bs)
            graph, _ = self.graphs[gbs]
            graph.replay()
            return None
        return self._decode_body(bs, self.engine.attn_nsplit(bs, max_ctx))

    @torch.inference_mode()
    def run_model_prefill(self, seqs: list[Sequence]):
        b = self.block_size
        input_ids, positions, ctx, cu = self.prepare_prefill(seqs)
        self._decode_key = None            # pages may have been handed out anew
        m = input_ids.numel()
        eng = self.engine
        if m > eng.max_tokens:
            raise AssertionError("prefill batch exceeds the activation buffers")
        if self.tp_pair is not None:       # the flag sequence numbers of this step
            self.hn["step"][0] = self.step_index
            self.hn["step"][1] = self.step_index + 1
            self.dv["step"].copy_(self.hv["step"], non_blocking=True)
        ops.gather_rows(self.weights.embed, input_ids, out=eng.embeds[:m])
        for i, seq in enumerate(seqs):
            rows = getattr(seq, "inputs_embeds", None)      # the reference's Sequence has no such attribute
            if rows is not None and seq.num_cached_tokens == 0:
                eng.embeds[cu[i]:cu[i] + rows.shape[0]].copy_(rows.to(self.device, non_blocking=True))
        hidden = eng.forward(m, positions, ctx, max_seqlen=ctx.max_seqlen_q)
        # the LM head sees the last B rows of every sequence (embed_head.py:63-66 of the reference)
        last = torch.tensor([cu[i + 1] - b + j for i in range(len(seqs)) for j in range(b)], dtype=torch.int64,
                            pin_memory=True).to(self.device, non_blocking=True)
        rows = ops.gather_rows(hidden, last, out=eng.lm_rows[:len(seqs) * b])
        temps = self.prepare_sample(seqs)
        eng.sample(rows, temps, step=self.step_index, **self._noise_args(rows.shape[0]))
        return rows

    # ------------------------------------------------------------------ entry point
    def _next_event_pair(self):
        ev = self.step_events
        if ev is None:
            return None
        if isinstance(ev, (tuple, list)):
            return ev
        return next(ev, None)

    def _use_graph(self, bs: int) -> bool:
        return bool((not self.enforce_eager) and self.noise != "explicit" and bs <= self.max_bs and self.graph_bs)

    def _tail(self, bs: int, p: int, mask_id: int, threshold: float) -> torch.cuda.CUDAGraph:
        """What follows the forward pass of a graph-launched decode step, as a graph of its own per batch-size
        bucket ``bs`` (the mask id and the threshold are kernel arguments: the configuration's mask id with the
        default threshold is captured with the forward graphs, anything else on first use): the unmask rule on
        result set ``p``, the new block ids handed on to the next step's input, the step counters advanced, the
        results copied to pinned memory.  Rows of the bucket beyond the step's requests carry whatever the padded
        forward rows produced; nobody reads them."""
        key = (bs, p, int(mask_id), float(threshold))
        graph = self._tails.get(key)
        if graph is None:
            (d_all, h_all, d_ids, d_counts, d_transfer, _, _, _, d_status, _) = self._result_views(bs, p)
            m = bs * self.block_size
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                d_ids.copy_(self.dv["ids"][:bs], non_blocking=True)
                ops.unmask_decide(d_ids, self.engine.x0[:m], self.engine.conf[:m], mask_id, threshold, 1,
                                  transfer=d_transfer, counts=d_counts, status_out=d_status)
                self.dv["ids"][:bs].copy_(d_ids, non_blocking=True)
                self.dv["step"].add_(1)
                h_all.copy_(d_all, non_blocking=True)
            self._tails[key] = graph
        return graph

    def _launch(self, seqs: list[Sequence], is_prefill: bool):
        """Everything of a step up to, not including, the wait for its results: forward pass, unmask rule, the
        copy of the results to pinned memory.  Returns the (possibly extended) request list and the record of
        the launch (batch size, result set, event pair, whether it was a graph launch)."""
        bs, b = len(seqs), self.block_size
        self._pair = None
        p = self._parity
        self._parity ^= 1
        if is_prefill:
            hidden = self.run_model_prefill(seqs)
        else:
            if self.fuse_commit_pass:
                extra = [_NextBlock(seq) for seq in seqs if seq.is_caching and self._next_block_ready(seq)]
                extra = extra[:self.max_bs - bs]
                if extra:
                    seqs = list(seqs) + extra
                    bs = len(seqs)
            self.run_model_decode(seqs)
            hidden = self.engine.final[:bs * b]     # final-norm rows of the step (graph replays write here too)
        sp = seqs[0].sampling_params
        if sp.denoising_strategy != "low_confidence_dynamic":
            raise NotImplementedError(f"Denoising strategy {sp.denoising_strategy} not implemented")
        with torch.inference_mode():
            quotas = self._step_quotas(seqs, is_prefill)
            graph_tail = (not is_prefill) and quotas is None and not self.keep_last and self._use_graph(bs)
            vbs = bs          # rows of the result views
            if graph_tail:
                vbs = next(x for x in self.graph_bs if x >= bs)
                self._tail(vbs, p, seqs[0].mask_token_id, sp.dynamic_threshold).replay()
                if self._pair is not None:
                    self._pair[1].record()
            else:
                # sampler state: the host copy of each block is the source of truth, as in the reference
                # (a decode step has just sent those ids down as its input)
                (d_all, h_all, d_ids, d_counts, d_transfer, h_ids, h_counts, h_transfer, d_status,
                 h_status) = self._result_views(bs, p)
                if is_prefill:
                    torch.stack([seq.current_denoising_block for seq in seqs], out=h_ids)
                    d_ids.copy_(h_ids, non_blocking=True)
                else:
                    d_ids.copy_(self.dv["ids"][:bs], non_blocking=True)
                m = bs * b
                ops.unmask_decide(d_ids, self.engine.x0[:m], self.engine.conf[:m], seqs[0].mask_token_id,
                                  sp.dynamic_threshold, 1, transfer=d_transfer, counts=d_counts, quotas=quotas,
                                  status_out=d_status)
                if self._pair is not None and not is_prefill:
                    self._pair[1].record()
                h_all.copy_(d_all, non_blocking=True)
                if self.keep_last:
                    self.last = dict(x0=self.engine.x0[:m].clone(), conf=self.engine.conf[:m].clone(),
                                     hidden=None if hidden is None else hidden.clone())
            self._done[p].record()
        return seqs, dict(bs=bs, vbs=vbs, set=p, pair=self._pair, graph=graph_tail)

    def _launch_ahead(self, seqs: list[Sequence], cur: dict) -> dict:
        """The decode step after the graph-launched step ``cur`` of the same requests, put on the GPU before the
        results of ``cur`` are known: its block ids are the ones the unmask rule of ``cur`` leaves on the device,
        its step counters the incremented ones, everything else is unchanged in the pinned inputs."""
        bs = cur["bs"]
        p = self._parity
        self._parity ^= 1
        pair = self._next_event_pair()
        sp = seqs[0].sampling_params
        with torch.inference_mode():
            if pair is not None:
                pair[0].record()
            gbs = cur["vbs"]
            self.graphs[gbs][0].replay()
            self._tail(gbs, p, seqs[0].mask_token_id, sp.dynamic_threshold).replay()
            if pair is not None:
                pair[1].record()
            self._done[p].record()
        key = (tuple(map(len, seqs)), tuple(len(seq.block_table) for seq in seqs))
        return dict(bs=bs, vbs=cur["vbs"], set=p, pair=pair, graph=True, seqs=list(seqs), key=key)

    def _ahead_possible(self, seqs: list[Sequence]) -> bool:
        """May the step after this decode step be launched before the scheduler asks for it, and before this
        step's results are known?  Only the plain case: graph launches, the nano engine's unmask rule, one GPU,
        and no request on its commit pass (the scheduler gives those a new block or retires them, so the next step
        has other inputs).  Whatever this step unmasks, the next step of these requests has the same positions,
        slots and pages: another denoising pass, or the commit pass of a block that has just lost its last mask."""
        if not self.launch_ahead or self.keep_last or self.fuse_commit_pass or self.tp_pair is not None:
            return False
        if any(seq.is_caching for seq in seqs):
            return False
        return all(getattr(seq.sampling_params, "denoising_steps", None) is None for seq in seqs)

    def _ahead_matches(self, ahead: dict, seqs: list[Sequence]) -> bool:
        held, rows = ahead["seqs"], self._last_rows
        if len(seqs) != len(held) or rows is None or len(rows) != len(held):
            return False
        if not all(a is b for a, b in zip(seqs, held)):
            return False
        if ahead["key"] != (tuple(map(len, seqs)), tuple(len(seq.block_table) for seq in seqs)):
            return False
        return all(seq.current_denoising_block is rows[i] for i, seq in enumerate(seqs))

    def _wait_results(self, rec: dict):
        self._done[rec["set"]].synchronize()
        views = self._result_views(rec["vbs"], rec["set"])
        status = int(views[-1][0])
        if status:
            # a kernel of this step skipped an access or gave up a wait (bad slot / page / token id / position,
            # or a bounded wait that ran out): the step's tokens cannot be trusted.  The word is already cleared.
            raise RuntimeError(f"decode step {self.step_index}: device status word {status:#x} "
                               "(1 bad slot, 2 bad page, 4 bad token id, 8 bad position, 16 wait timed out)")
        return views

    def cancel_ahead(self) -> None:
        """Waits for a step launched ahead, if one is in flight, and drops its results (the next ``run`` then
        launches the step it is asked for from the host's state)."""
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            self.ahead_misses += 1
            self._wait_results(ahead)

    def run(self, seqs: list[Sequence], is_prefill: bool) -> int:
        if len(seqs) > self.max_bs:
            raise AssertionError("batch larger than max_num_seqs")
        ahead, self._ahead = self._ahead, None
        if ahead is not None and not is_prefill and self._ahead_matches(ahead, seqs):
            # the step asked for is the one already on the GPU
            self.ahead_hits += 1
            cur = ahead
        else:
            if ahead is not None:
                # another step was asked for: let the one in flight finish (its K/V rows are tentative ones of the
                # same blocks; the step that now runs gets its block ids and step counters from the host again, so
                # it also reuses the noise step number) and drop its results
                self.ahead_misses += 1
                self._wait_results(ahead)
            seqs, cur = self._launch(seqs, is_prefill)
        if cur["graph"] and self._ahead_possible(seqs):
            self._ahead = self._launch_ahead(seqs, cur)
        (_, _, _, _, _, h_ids, h_counts, h_transfer, _, _) = self._wait_results(cur)
        self.last_step_events = cur["pair"]
        bs = cur["bs"]            # the views may hold the rows of a whole batch-size bucket
        # one copy of the results for the whole batch; every request keeps a row of it
        blocks = h_ids[:bs].clone()
        rows = blocks.unbind(0)
        moved = h_transfer[:bs] != 0
        moved_any = moved.any(axis=1)
        for i, seq in enumerate(seqs):
            if type(seq) is _NextBlock:     # applied by Scheduler.postprocess once the block before it is appended
                seq.seq.pending_first_step = (rows[i], moved[i].copy() if moved_any[i] else None)
                continue
            seq.current_denoising_block = rows[i]
            if moved_any[i]:
                seq.current_step_map.numpy()[moved[i]] = seq.current_denoise_step
            seq.current_denoise_step += 1
        self._last_rows, self._last_blocks = rows, blocks.numpy()   # shares memory with the rows
        self.step_index += 1
        return int(h_counts[:bs].sum())

    def _step_quotas(self, seqs, is_prefill: bool):
        """Per-request quota of this pass, or None for the nano engine's rule (one token unless more pass the
        threshold, ``nanovllm/layers/sampler.py:44-50``).  With ``SamplingParams.denoising_steps`` set (a field
        of this package, absent from the reference's class) a block follows the HF twin's schedule: pass ``s``
        of a block takes ``num_transfer_tokens[min(s, steps - 1)]``
        (``mineru_diffusion/modeling_mineru_diffusion.py:617-623,712``)."""
        steps = getattr(seqs[0].sampling_params, "denoising_steps", None)
        if not steps:
            return None
        b = self.block_size
        table = ops.num_transfer_tokens(b, int(steps))
        q = self.quota_host.numpy()
        for i, seq in enumerate(seqs):
            owner = seq.seq if type(seq) is _NextBlock else seq
            start = len(seq)
            # passes made on the block that starts at this length, kept on the request object itself
            at, done = getattr(owner, "_block_passes", (-1, 0))
            if at != start:
                done = 0
            q[i] = table[min(done, len(table) - 1)]
            owner._block_passes = (start, done + 1)
        self.quota_dev[:len(seqs)].copy_(self.quota_host[:len(seqs)], non_blocking=True)
        return self.quota_dev

    def _next_block_ready(self, seq: Sequence) -> bool:
        """True when the request being committed goes on to another block (the finishing rule of
        ``Scheduler.postprocess``) and already holds the pages that block needs."""
        b = self.block_size
        if seq.num_completion_tokens + b >= seq.max_new_tokens:
            return False
        if not seq.ignore_eos:
            block = seq.current_denoising_block.numpy()
            if any(bool((block == t).any()) for t in seq.sampling_params.stop_token_ids):
                return False
        return seq.num_tokens + 2 * b <= Sequence.kvcache_block_size * len(seq.block_table)

    def launches_per_decode_step(self, bs: int = 1) -> int:
        """Kernels of libmdb200 launched by one decode-form step: row gather,
        per layer 2 norms + 4 GEMMs + q/k norm-rope-store + attention (+ merge
        of the key-range splits), final norm, LM-head scan + merge, unmask rule."""
        if self.graph_bs:
            nsplit = self.graphs[next(x for x in self.graph_bs if x >= bs)][1]
        else:
            nsplit = self.engine.attn_nsplit(bs, self.config.max_model_len)
        per_layer = 8 + (1 if nsplit > 1 else 0)
        m = bs * self.block_size
        if m > 64:
            if ops.qkv_rope_commit_supported(m, self.dcfg.hidden_size):
                per_layer -= 1  # q/k norm, rotary embedding and KV store run in the qkv GEMM's epilogue
        return 1 + self.dcfg.num_hidden_layers * per_layer + 1 + 2 + 1

    # ------------------------------------------------------------------ CUDA graphs
    @torch.inference_mode()
    def capture_cudagraph(self):
        """One graph per batch-size bucket covering the copy of the packed
        step inputs (all but the block ids and the step counters) from pinned
        memory, embedding gather, all layers, the LM head and the sampler
        statistics.  Padded rows carry
        slot -1 and context length 0, which every kernel treats as a no-op."""
        if self.noise == "explicit":
            return
        self._decode_key = None            # the pinned input buffer is rewritten below
        max_bs = self.max_bs
        self.graph_bs = [x for x in (1, 2, 4, 8) if x <= max_bs] + list(range(16, max_bs + 1, 16))
        if self.graph_bs[-1] != max_bs:      # a batch limit between two buckets gets a bucket of its own
            self.graph_bs.append(max_bs)
        hv = self.hv
        hv["ids"].zero_(); hv["pos"].zero_(); hv["slots"].fill_(-1); hv["ctx"].zero_(); hv["tab"].fill_(-1)
        hv["temp"].fill_(1.0)
        self.inputs.dev.copy_(self.inputs.host)
        pool = None
        for bs in reversed(self.graph_bs):
            nsplit = self.engine.attn_nsplit(bs, self.config.max_model_len)
            self._decode_body(bs, nsplit)   # warm-up: sets kernel attributes outside capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool):
                # pinned buffer, read at replay time; block ids and step counters are not part of this copy: the
                # launcher sends them, or the step before has left them on the device
                o = self.inputs.o_pos
                self.inputs.dev[o:].copy_(self.inputs.host[o:], non_blocking=True)
                self._decode_body(bs, nsplit)
            if pool is None:
                pool = graph.pool()
            self.graphs[bs] = (graph, nsplit)
        for bs in self.graph_bs:
            for p in (0, 1):
                self._tail(bs, p, self.config.mask_token_id, 0.9)     # SamplingParams' default threshold
        torch.cuda.synchronize()
