"""The SDAR decoder stack as a launch sequence over libmdb200.

``DecoderEngine.forward`` is what ``SDARModel.forward`` is in the reference
(nanovllm/models/sdar.py:167-181): token rows in, final-norm hidden rows out,
K/V of the step written into the paged cache on the way.  Per layer it issues

    add+RMSNorm -> qkv GEMM -> q/k norm + RoPE + KV store -> attention
    -> o GEMM -> add+RMSNorm -> gate_up GEMM (+SiLU*mul) -> down GEMM

For steps of at most 64 rows the GEMMs are the weight-streaming kernels: they
leave fp32 split-k slices that the *next* kernel sums, rounds to bf16 and
consumes, so no stand-alone reduction or activation pass exists.  Longer
steps (prefill, big decode batches) use the tile GEMM with fused epilogues.
All buffers are allocated once here; a step allocates nothing, which is what
lets the decode step be captured in a CUDA graph.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops
from .engine.config import DecoderConfig
from .engine.context import Context

PAGE = 256
SKINNY_MAX_ROWS = 64
# o_proj / down_proj keep the split-k slice form of the weight-streaming kernel up to 128 rows: it still beats the
# tile GEMM there although that one splits k over clusters when it has few tiles.  Measured on B200 (projection +
# the norm that follows, slice form against tile GEMM): o_proj 11.0 / 11.8 / 15.4 us against 12.9 / 12.9 / 13.4 at
# 96 / 128 / 192 rows; down_proj 13.5 / 14.1 / 19.0 against 15.7 / 15.6 / 18.5.
SLICE_MAX_ROWS = (128, 128)     # (o_proj, down_proj), one GPU; a tensor-parallel pair switches at SKINNY_MAX_ROWS


@dataclass
class LayerWeights:
    input_ln: torch.Tensor
    qkv: torch.Tensor       # [(Hq+2Hkv)*D, H] rows q|k|v, as QKVParallelLinear stores them
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    o: torch.Tensor         # [H, Hq*D]
    post_ln: torch.Tensor
    gate_up: torch.Tensor   # [2I, H] rows gate|up, as MergedColumnParallelLinear stores them
    down: torch.Tensor      # [H, I]


@dataclass
class DecoderWeights:
    embed: torch.Tensor
    layers: list[LayerWeights]
    final_ln: torch.Tensor
    lm_head: torch.Tensor

    @classmethod
    def random_init(cls, cfg: DecoderConfig, seed: int, device, std: float = 0.02) -> "DecoderWeights":
        """Seeded N(0, std) matrices generated on ``device`` (RMSNorm weights 1)."""
        g = torch.Generator(device=device).manual_seed(seed)
        bf = torch.bfloat16

        def mat(r, c):
            return (torch.randn(r, c, generator=g, device=device, dtype=torch.float32) * std).to(bf)

        def ones(n):
            return torch.ones(n, dtype=bf, device=device)

        h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        embed = mat(cfg.vocab_size, h)
        layers = [LayerWeights(ones(h), mat((hq + 2 * hkv) * d, h), ones(d), ones(d), mat(h, hq * d), ones(h),
                               mat(2 * i, h), mat(h, i)) for _ in range(cfg.num_hidden_layers)]
        lm_head = embed if cfg.tie_word_embeddings else mat(cfg.vocab_size, h)
        return cls(embed, layers, ones(h), lm_head)

    @classmethod
    def from_reference_layout(cls, src, device) -> "DecoderWeights":
        """Copy a weight set held in the reference's tensor layout (any object
        with the same attribute names, tensors on any device) to ``device``."""
        def mv(t):
            return t.detach().to(device=device, dtype=torch.bfloat16).contiguous()
        layers = [LayerWeights(mv(l.input_ln), mv(l.qkv), mv(l.q_norm), mv(l.k_norm), mv(l.o), mv(l.post_ln),
                               mv(l.gate_up), mv(l.down)) for l in src.layers]
        return cls(mv(src.embed), layers, mv(src.final_ln), mv(src.lm_head))

    def nbytes(self) -> int:
        n = self.embed.numel() + self.final_ln.numel()
        if self.lm_head.data_ptr() != self.embed.data_ptr():
            n += self.lm_head.numel()
        for l in self.layers:
            n += sum(t.numel() for t in (l.input_ln, l.qkv, l.q_norm, l.k_norm, l.o, l.post_ln, l.gate_up, l.down))
        return 2 * n


def rope_table(max_pos: int, head_dim: int, base: float, device) -> torch.Tensor:
    """fp32 [max_pos, head_dim] cos|sin table built the way the reference builds
    its ``cos_sin_cache`` (nanovllm/layers/rotary_embedding.py:19-35)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(device)


class DecoderEngine:

    def __init__(self, cfg: DecoderConfig, weights: DecoderWeights, kv_cache: torch.Tensor, max_tokens: int,
                 max_seqs: int, block_size: int, tp_rank: int = 0, tp_size: int = 1):
        """``cfg`` and ``weights`` are this rank's shard when ``tp_size`` is 2
        (see tp.shard_config / tp.shard_weights); ``attach_tp`` then supplies
        the peer buffers before the first step."""
        self.tp = None              # TensorParallelPair once attached
        self.tp_epoch = None        # device word the runner advances every step
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.cfg = cfg
        self.w = weights
        self.kv_cache = kv_cache    # [2, L, pages, 256, Hkv, D]
        self.block_size = block_size
        self.max_tokens = max_tokens
        self.max_seqs = max_seqs
        dev = kv_cache.device
        self.device = dev
        bf = torch.bfloat16
        h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
        hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        if d != 128:
            raise ValueError("the attention kernels are built for head_dim 128")
        self.nqkv = (hq + 2 * hkv) * d
        self.num_pages = kv_cache.shape[2]
        self.rope = rope_table(cfg.max_position_embeddings, d, cfg.rope_theta, dev)
        self.scale = d ** -0.5
        t = max_tokens

        def buf(*shape, dtype=bf):
            return torch.empty(shape, dtype=dtype, device=dev)

        self.embeds = buf(t, h)
        self.x = buf(t, h)
        self.res = buf(t, h)
        self.q = buf(t, hq, d)
        self.kbuf = buf(t, hkv, d)
        self.vbuf = buf(t, hkv, d)
        self.attn = buf(t, hq, d)
        self.act = buf(t, i)
        self.final = buf(t, h)
        self.lm_rows = buf(max_seqs * block_size, h)
        # weight-streaming path: fp32 split-k slices shared by all four GEMMs
        rows = min(t, max(SKINNY_MAX_ROWS, *SLICE_MAX_ROWS))
        self.ks_qkv = ops.pick_ksplit(rows, self.nqkv, h)
        self.ks_o = ops.pick_ksplit(rows, h, hq * d)
        self.ks_down = ops.pick_ksplit(rows, h, i)
        part_elems = rows * max(self.ks_qkv * self.nqkv, self.ks_o * h, self.ks_down * h)
        self.partials = buf(part_elems, dtype=torch.float32)
        # tiled path: materialised bf16 GEMM outputs
        if t > SKINNY_MAX_ROWS:
            self.qkv_out = buf(t, self.nqkv)
            self.h_out = buf(t, h)
        self.max_nsplit = 64
        ws = ops._lib.lib().mdb_attn_paged_workspace_bytes(max_seqs, block_size, hq, self.max_nsplit)
        # attention partials are only needed while CTAs are scarce: cap at what 64 requests use
        ws = min(ws, ops._lib.lib().mdb_attn_paged_workspace_bytes(min(max_seqs, 64), block_size, hq, self.max_nsplit))
        self.attn_ws = buf(max(int(ws), 16), dtype=torch.uint8)
        self.lm_ws = buf(max(ops.lmhead_workspace_bytes(max_seqs * block_size, cfg.vocab_size), 16), dtype=torch.uint8)
        self.x0 = buf(max_seqs * block_size, dtype=torch.int32)
        self.conf = buf(max_seqs * block_size, dtype=torch.float32)

    # ------------------------------------------------------------------
    def attn_nsplit(self, bs: int, max_ctx: int) -> int:
        cfg = self.cfg
        n = ops.default_nsplit(bs, self.block_size, cfg.num_attention_heads, cfg.num_key_value_heads, max_ctx)
        while n > 1 and ops._lib.lib().mdb_attn_paged_workspace_bytes(
                bs, self.block_size, cfg.num_attention_heads, n) > self.attn_ws.numel():
            n -= 1
        return n

    def forward(self, m: int, positions: torch.Tensor, ctx: Context, nsplit: int = 1,
                max_seqlen: int = 0) -> torch.Tensor:
        """Runs the layer stack over rows [0, m) of ``self.embeds``; returns
        the final-norm hidden rows (a view of an internal buffer)."""
        cfg = self.cfg
        h, inter = cfg.hidden_size, cfg.intermediate_size
        hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        eps = cfg.rms_norm_eps
        skinny = m <= SKINNY_MAX_ROWS
        if self.tp_size > 1 and self.tp is None:
            raise RuntimeError("tensor-parallel engine used before attach_tp()")
        x, res = self.x[:m], self.res[:m]
        q, attn, act = self.q[:m], self.attn[:m], self.act[:m]
        pos = positions.reshape(-1)
        slots = ctx.slot_mapping.reshape(-1) if ctx.slot_mapping is not None and ctx.slot_mapping.numel() else None
        prev = None  # output of the previous row-parallel projection, see _row_gemm
        for li, lw in enumerate(self.w.layers):
            k_cache, v_cache = self.kv_cache[0, li], self.kv_cache[1, li]
            if prev is None:
                ops.add_rms_norm(self.embeds[:m], None, lw.input_ln, eps, out=x, residual_out=res)
            else:
                self._add_norm(prev, res, lw.input_ln, eps, x)

            kb = self.kbuf[:m] if ctx.is_prefill else None
            vb = self.vbuf[:m] if ctx.is_prefill else None
            if skinny:
                parts = self.partials[:self.ks_qkv * m * self.nqkv].view(self.ks_qkv, m, self.nqkv)
                ops.gemm_splitk_partials(x, lw.qkv, self.ks_qkv, parts)
                ops.qknorm_rope_commit(None, pos, self.rope, lw.q_norm, lw.k_norm, eps, hq, hkv, slots, k_cache,
                                       v_cache, partials=parts, q_out=q, k_out=kb, v_out=vb)
            elif ops.qkv_rope_commit_supported(m, h):
                ops.qkv_proj_rope_commit(x, lw.qkv, pos, self.rope, lw.q_norm, lw.k_norm, eps, hq, hkv, slots, k_cache,
                                         v_cache, q_out=q, k_out=kb, v_out=vb)
            else:
                qkv = self.qkv_out[:m]
                ops.linear(x, lw.qkv, out=qkv)
                ops.qknorm_rope_commit(qkv, pos, self.rope, lw.q_norm, lw.k_norm, eps, hq, hkv, slots, k_cache,
                                       v_cache, q_out=q, k_out=kb, v_out=vb)

            if ctx.is_prefill:
                ops.sparse_attn_varlen(q, kb, vb, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.block_size,
                                       max_seqlen=max_seqlen, out=attn)
            else:
                bs = m // self.block_size
                ops.block_attn_with_kvcache(q.view(bs, self.block_size, hq, d), k_cache, v_cache, ctx.context_lens,
                                            ctx.block_tables, self.scale, nsplit=nsplit, workspace=self.attn_ws,
                                            out=attn.view(bs, self.block_size, hq, d))
            prev = self._row_gemm(0, attn.view(m, hq * d), lw.o, m, li)
            self._add_norm(prev, res, lw.post_ln, eps, x)
            ops.gateup_swiglu(x, lw.gate_up, out=act)
            prev = self._row_gemm(1, act, lw.down, m, li)
        out = self.final[:m]
        self._add_norm(prev, res, self.w.final_ln, eps, out)
        return out

    # ------------------------------------------------------------------ row-parallel projections
    def attach_tp(self, pair, epoch_word: torch.Tensor):
        """Second half of TP = 2 set-up: the peer buffers and the step word."""
        self.tp, self.tp_epoch = pair, epoch_word

    def _row_gemm(self, which: int, x_in: torch.Tensor, w: torch.Tensor, m: int, li: int):
        """o_proj (which = 0) or down_proj (1), the reference's RowParallelLinear
        (nanovllm/layers/linear.py:131-157).  Returns how the following
        norm finds the result: ("bf16", y) | ("parts", slices) | ("tp", slices,
        flag slots to wait on, their number, launch tag)."""
        h = self.cfg.hidden_size
        ks = self.ks_o if which == 0 else self.ks_down
        if m <= SKINNY_MAX_ROWS or (self.tp is None and m <= SLICE_MAX_ROWS[which] and ks > 1):
            if self.tp is None:
                parts = self.partials[:ks * m * h].view(ks, m, h)
                ops.gemm_splitk_partials(x_in, w, ks, parts)
                return ("parts", parts)
            view, mine, theirs = self.tp.o_slices(m) if which == 0 else self.tp.down_slices(m)
            wait_ptr, signal_ptr = self.tp.flags(which)
            tag = 2 * li + 1 + which
            ops.gemm_splitk_partials_tp(x_in, w, ks, mine, theirs, signal_ptr, tag, self.tp_epoch)
            return ("tp", view, wait_ptr, ops.tp_grid_size(m, h, x_in.shape[1], ks), tag)
        ho = self.h_out[:m]
        k = x_in.shape[1]
        if self.tp is not None:
            if m > self.tp.many_rows:
                raise RuntimeError(f"step of {m} rows exceeds the tensor-parallel landing buffers ({self.tp.many_rows} rows)")
            # the all-reduce rides in the GEMM epilogue: every tile goes to the local output and, over NVLink,
            # to the peer's landing buffer; the following norm adds the two
            land, peer_ptr = self.tp.landing(which, m)
            wait_ptr, signal_ptr = self.tp.flags(which)
            tag = 2 * li + 1 + which
            slots = ops.linear_tp_rows(x_in, w, ho, peer_ptr, signal_ptr, tag, self.tp_epoch)
            return ("tp_rows", ho, land, wait_ptr, slots, tag)
        ops.linear(x_in, w, out=ho)
        return ("bf16", ho)

    def _add_norm(self, prev, res: torch.Tensor, ln: torch.Tensor, eps: float, out: torch.Tensor):
        if prev[0] == "parts":
            ops.add_rms_norm(None, res, ln, eps, partials=prev[1], out=out, residual_out=res)
        elif prev[0] == "tp":
            _, view, wait_ptr, count, tag = prev
            ops.add_rms_norm_tp(view, res, ln, eps, out, res, wait_ptr, count, tag, self.tp_epoch)
        elif prev[0] == "tp_rows":
            _, own, land, wait_ptr, count, tag = prev
            ops.add_rms_norm_tp_rows(own, land, res, ln, eps, out, res, wait_ptr, count, tag, self.tp_epoch)
        else:
            ops.add_rms_norm(prev[1], res, ln, eps, out=out, residual_out=res)

    def sample(self, rows: torch.Tensor, temperatures: torch.Tensor, noise=None, seed=None, step: int = 0,
               step_dev=None):
        """LM head + sampler statistics over ``rows`` [m, H]; returns views of
        the internal x0 / confidence buffers."""
        m = rows.shape[0]
        if self.tp is None:
            return ops.lm_head_sample(rows, self.w.lm_head, temperatures, self.block_size, noise=noise, seed=seed,
                                      step=step, step_dev=step_dev, workspace=self.lm_ws, x0=self.x0[:m],
                                      conf=self.conf[:m])
        lib = ops._lib.lib()
        ws, peer_ws = self.tp.lm_workspace()
        wait_ptr, signal_ptr = self.tp.flags(2)
        tag = 2 * len(self.w.layers) + 1
        if m > SKINNY_MAX_ROWS:
            # Many-row steps: the tile GEMM over half of the 256-column vocabulary tiles per rank, one sampler
            # record per tile mirrored into the peer's workspace; logits are never gathered.
            vocab = self.cfg.vocab_size
            can_split = (noise is None and vocab % 128 == 0
                         and ws.numel() >= lib.mdb_lmhead_tp_workspace_bytes(m, vocab))
            if not can_split:
                # both ranks hold the whole LM head and bit-identical hidden rows: each scans all of it
                return ops.lm_head_sample(rows, self.w.lm_head, temperatures, self.block_size, noise=noise, seed=seed,
                                          step=step, step_dev=step_dev, workspace=self.lm_ws, x0=self.x0[:m],
                                          conf=self.conf[:m])
            from .tp import lm_head_split
            begin, count, peer_cols = lm_head_split(vocab, self.tp_rank, many_rows=True)
            if count == 0 or peer_cols == 0:
                return ops.lm_head_sample(rows, self.w.lm_head, temperatures, self.block_size, noise=noise, seed=seed,
                                          step=step, step_dev=step_dev, workspace=self.lm_ws, x0=self.x0[:m],
                                          conf=self.conf[:m])
            return ops.lm_head_sample_tp(rows, self.w.lm_head, temperatures, self.block_size, ws, peer_ws, begin, count,
                                         signal_ptr, wait_ptr, lib.mdb_lmhead_tp_slots(m, peer_cols), tag,
                                         self.tp_epoch, self.x0[:m], self.conf[:m], noise=None, seed=seed, step=step,
                                         step_dev=step_dev)
        # vocabulary tiles (128 rows) split between the two ranks; records are exchanged, never logits
        tiles = self.cfg.vocab_size // 128
        first = (tiles + 1) // 2
        begin, count = (0, first) if self.tp_rank == 0 else (first, tiles - first)
        ws, peer_ws = self.tp.lm_workspace()
        wait_ptr, signal_ptr = self.tp.flags(2)
        peer_count = tiles - count
        return ops.lm_head_sample_tp(rows, self.w.lm_head, temperatures, self.block_size, ws, peer_ws, begin, count,
                                     signal_ptr, wait_ptr, min(peer_count, 148), 2 * len(self.w.layers) + 1,
                                     self.tp_epoch, self.x0[:m], self.conf[:m], noise=noise, seed=seed, step=step,
                                     step_dev=step_dev)
