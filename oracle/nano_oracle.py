"""CPU restatement of the nano_dvlm block-diffusion decode step (TEST INFRASTRUCTURE).

This module is the checker, never the product: only the test-suite, the smoke
entry and the benchmark's CPU-baseline leg may import it.  It restates, with
plain torch ops on CPU tensors, what the reference engine computes on the path
``ModelRunner.run`` -> decoder -> LM head -> sampler.  Paths below are relative
to the reference project root; ``NV/`` abbreviates
``engines/nano_dvlm/nanovllm/``.

Parity status: the reference ships no tests, golden vectors or fixtures for
this path.  The restatement is pinned instead against outputs of the reference's
own modules executed on seeded inputs (fixtures under ``tests/golden``, written
by ``tests/golden/make_golden.py``).  Three third-party calls of the reference
cannot execute on a CPU in bf16 and are restated from their published
semantics: ``flash_attn_with_kvcache`` (flash-attn 2.8.3, call site
``NV/layers/sdar_attention.py:50-55``), the Triton staircase kernel in bf16
(``NV/kernels/triton/attention/block_prefill_attention_v2.py``; pinned in fp32
through the Triton interpreter) and liger's SiLU*mul (liger-kernel 0.6.4,
call site ``NV/layers/activation.py:15``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

PAGE = 256  # NV/engine/sequence.py:17 (class attribute, the only consistent value)
LOG2E = 1.44269504  # literal used at block_prefill_attention_v2.py:194


# --------------------------------------------------------------------------
# index contracts (integer, bit-exact)
# --------------------------------------------------------------------------
def get_slots(block_table: list[int], lo: int, hi: int, page: int = PAGE) -> list[int]:
    """Cache slot of every position in [lo, hi).  NV/engine/sequence.py:117-141.

    The reference walks first/middle/last pages; position p always lands at
    ``block_table[p // page] * page + p % page``.  An empty table (warm-up
    sequences) yields -1 for every position.
    """
    if not block_table:
        return [-1] * (hi - lo)
    return [block_table[p // page] * page + (p % page) for p in range(lo, hi)]


def pad_block_tables(tables: list[list[int]]) -> list[list[int]]:
    """-1 padded rectangular page table.  NV/engine/model_runner.py:121-125."""
    width = max(len(t) for t in tables)
    return [list(t) + [-1] * (width - len(t)) for t in tables]


def staircase_limit(i: int, seq_len: int, stairs: int) -> int:
    """Last key index (inclusive) query row ``i`` may attend in a sequence of
    ``seq_len`` tokens.  block_prefill_attention_v2.py:52-53,94-102: stairs are
    right-aligned, pad = ceil(T/S)*S - T, limit = ((i+pad)//S + 1)*S - 1 - pad.
    """
    blocks = (seq_len + stairs - 1) // stairs
    pad = blocks * stairs - seq_len
    return ((i + pad) // stairs + 1) * stairs - 1 - pad


def staircase_mask(seq_len: int, stairs: int) -> torch.Tensor:
    """Boolean [T, T] visibility matrix of the prefill staircase."""
    i = torch.arange(seq_len)
    blocks = (seq_len + stairs - 1) // stairs
    pad = blocks * stairs - seq_len
    limit = ((i + pad) // stairs + 1) * stairs - 1 - pad
    j = torch.arange(seq_len)
    return j[None, :] <= limit[:, None]


# --------------------------------------------------------------------------
# element-wise layers
# --------------------------------------------------------------------------
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """NV/layers/layernorm.py:16-26: fp32 normalise, round to the input dtype,
    then multiply by the weight in that dtype."""
    dt = x.dtype
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(dt) * weight.to(dt)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float):
    """NV/layers/layernorm.py:28-40: fp32 sum, residual = rounded sum, norm of
    the un-rounded fp32 sum."""
    dt = x.dtype
    xf = x.float() + residual.float()
    new_residual = xf.to(dt)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(dt) * weight.to(dt), new_residual


def rope_table(max_pos: int, head_dim: int, base: float) -> torch.Tensor:
    """fp32 [max_pos, head_dim] table, cos in the first half of each row and
    sin in the second.  NV/layers/rotary_embedding.py:19-35."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    t = torch.arange(max_pos, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x [..., heads, D] with positions [...]; NeoX half split in fp32.
    NV/layers/rotary_embedding.py:6-15,43-48."""
    cs = table[positions].unsqueeze(-2)
    cos, sin = cs.chunk(2, dim=-1)
    x1, x2 = torch.chunk(x.float(), 2, dim=-1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1).to(x.dtype)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """liger SiLU*mul as the reference calls it (NV/layers/activation.py:12-15):
    silu of the gate half in fp32, rounded to the storage dtype, times the up
    half in the storage dtype."""
    gate, up = gate_up.chunk(2, dim=-1)
    g = gate.float()
    return (g * torch.sigmoid(g)).to(gate_up.dtype) * up


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x W^T with fp32 accumulation and one rounding to the storage dtype
    (NV/layers/linear.py:72-73,153-154 through cuBLAS)."""
    return (x.float() @ w.float().t()).to(x.dtype)


# --------------------------------------------------------------------------
# paged KV cache
# --------------------------------------------------------------------------
def store_kvcache(key, value, k_cache, v_cache, slot_mapping) -> None:
    """Scatter rows of key/value [N, Hkv, D] into caches [pages, PAGE, Hkv, D]
    at ``slot_mapping`` [N]; -1 skips the row.  NV/layers/attention.py:10-40."""
    n, h, d = key.shape
    kc = k_cache.view(-1, h * d)
    vc = v_cache.view(-1, h * d)
    slots = slot_mapping.reshape(-1).tolist()
    kf = key.reshape(n, h * d)
    vf = value.reshape(n, h * d)
    for i, s in enumerate(slots):
        if s == -1:
            continue
        kc[s] = kf[i]
        vc[s] = vf[i]


def gather_pages(cache: torch.Tensor, table_row: torch.Tensor, ctx: int) -> torch.Tensor:
    """[ctx, Hkv, D] view of one request's cached rows through its page table."""
    pages = (ctx + PAGE - 1) // PAGE
    idx = table_row[:pages].long()
    return cache[idx].reshape(pages * PAGE, *cache.shape[2:])[:ctx]


def attn_paged(q, k_cache, v_cache, context_lens, block_tables, scale, round_p: bool = False):
    """Decode-form block attention: q [bs, B, Hq, D]; every query row sees
    keys [0, ctx) of its request, no other mask (``causal=False``).
    Restates flash_attn_with_kvcache as called at
    NV/layers/sdar_attention.py:50-55.  ``round_p`` mirrors flash-attn's
    rounding of the probabilities to bf16 before the PV product (its fp32
    row-sum uses the un-rounded values)."""
    bs, b, hq, d = q.shape
    hkv = k_cache.shape[2]
    g = hq // hkv
    out = torch.zeros_like(q)
    for r in range(bs):
        ctx = int(context_lens[r])
        if ctx <= 0:
            continue
        k = gather_pages(k_cache, block_tables[r], ctx).float()  # [ctx, Hkv, D]
        v = gather_pages(v_cache, block_tables[r], ctx).float()
        qf = q[r].float()  # [B, Hq, D]
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        s = torch.einsum("bhd,nhd->hbn", qf, k) * scale
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        l = p.sum(dim=-1, keepdim=True)
        if round_p:
            p = p.to(q.dtype).float()
        o = torch.einsum("hbn,nhd->bhd", p, v) / l.permute(1, 0, 2)
        out[r] = o.to(q.dtype)
    return out


def attn_staircase_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, stairs: int, mirror_rounding: bool = True):
    """Prefill staircase attention over packed sequences: q [N, Hq, D],
    k/v [N, Hkv, D].  block_prefill_attention_v2.py:17-166.  With
    ``mirror_rounding`` the two roundings of the Triton kernel are kept: q is
    multiplied by log2(e)/sqrt(D) and rounded to the storage dtype (:80), and
    probabilities are rounded to the storage dtype before PV (:152) while the
    row sum stays fp32 (:147-149)."""
    n, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    out = torch.zeros_like(q)
    q_scale = 1.0 / math.sqrt(d) * LOG2E
    nseq = cu_seqlens_q.numel() - 1
    for b in range(nseq):
        qs, qe = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        ks, ke = int(cu_seqlens_k[b]), int(cu_seqlens_k[b + 1])
        t = ke - ks
        if qe - qs == 0:
            continue
        assert qe - qs == t, "the reference kernel assumes self-attention lengths"
        mask = staircase_mask(t, stairs)
        if mirror_rounding:
            qf = (q[qs:qe] * q_scale).to(q.dtype).float()
        else:
            qf = q[qs:qe].float() * q_scale
        kf = k[ks:ke].float().repeat_interleave(g, dim=1)
        vf = v[ks:ke].float().repeat_interleave(g, dim=1)
        s = torch.einsum("ihd,jhd->hij", qf, kf)  # base-2 logits
        s = torch.where(mask[None], s, torch.full_like(s, -1.0e6))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp2(s - m)
        l = p.sum(dim=-1, keepdim=True)
        l = torch.where(l == 0, torch.ones_like(l), l)
        if mirror_rounding:
            p = p.to(q.dtype).float()
        o = torch.einsum("hij,jhd->ihd", p, vf) / l.permute(1, 0, 2)
        out[qs:qe] = o.to(q.dtype)
    return out


# --------------------------------------------------------------------------
# sampler
# --------------------------------------------------------------------------
def sampler_prepare(logits: torch.Tensor, temperatures: torch.Tensor, gumbel: torch.Tensor | None):
    """NV/layers/sampler.py:11-22 with the Gumbel noise made an explicit input
    (the reference draws it from torch's generator; ``None`` means zero noise,
    i.e. plain argmax).  logits [bs, B, V] (storage dtype), temperatures [bs, 1].
    Returns x0 [bs, B] int64 and x0_p [bs, B] fp32."""
    lf = logits.float() / temperatures.unsqueeze(1)
    gl = lf if gumbel is None else lf + gumbel
    x0 = gl.argmax(dim=-1)
    probs = torch.softmax(lf, dim=-1)
    x0_p = probs.gather(-1, x0.unsqueeze(-1)).squeeze(-1)
    return x0, x0_p


def unmask_decision(blocks: torch.Tensor, x0: torch.Tensor, x0_p: torch.Tensor, mask_id: int, threshold: float,
                    quotas=None):
    """NV/layers/sampler.py:28-54.  blocks [bs, B] int64 current block ids.
    Returns (new blocks, transfer mask [bs, B] bool).  ``quotas`` (one int per request) switches a request to
    the HF twin's rule (mineru_diffusion/modeling_mineru_diffusion.py:518-532): the positions above the
    threshold if at least ``quota`` of them, else the ``quota`` most confident masked positions (all masked
    positions when fewer are left -- below that the reference's topk picks among -inf entries in an order
    torch leaves unspecified)."""
    mask_index = blocks == mask_id
    confidence = torch.where(mask_index, x0_p, torch.full_like(x0_p, -torch.inf))
    transfer = torch.zeros_like(x0, dtype=torch.bool)
    for j in range(confidence.shape[0]):
        if not mask_index[j].any():
            continue
        quota = 1 if quotas is None else int(quotas[j])
        hi = confidence[j] > threshold
        if int(hi.sum()) >= quota:
            transfer[j] = hi
        else:
            # top-quota by confidence; the lowest index wins an exact tie
            order = sorted(range(confidence.shape[1]), key=lambda i: (-float(confidence[j, i]), i))
            for i in order[:quota]:
                if bool(mask_index[j, i]):
                    transfer[j, i] = True
    out = blocks.clone()
    out[transfer] = x0[transfer]
    return out, transfer


def num_transfer_tokens(block_length: int, steps: int) -> list[int]:
    """Quota of each denoising step of a block, mineru_diffusion/modeling_mineru_diffusion.py:617-623."""
    base, rem = divmod(block_length, steps)
    return [base + (1 if s < rem else 0) for s in range(steps)]


# --------------------------------------------------------------------------
# decoder
# --------------------------------------------------------------------------
@dataclass
class DecoderConfig:
    """Dimensions of the SDAR decoder (mineru_diffusion/configuration_mineru_diffusion.py:12-32)."""
    vocab_size: int = 151936
    hidden_size: int = 2048
    intermediate_size: int = 6144
    num_hidden_layers: int = 28
    num_attention_heads: int = 16
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    max_position_embeddings: int = 32768


@dataclass
class LayerWeights:
    input_ln: torch.Tensor
    qkv: torch.Tensor       # [(Hq+2Hkv)*D, H], rows q|k|v  (NV/layers/linear.py:114-128)
    q_norm: torch.Tensor    # [D]
    k_norm: torch.Tensor    # [D]
    o: torch.Tensor         # [H, Hq*D]
    post_ln: torch.Tensor
    gate_up: torch.Tensor   # [2I, H], rows gate|up  (NV/layers/linear.py:87-93)
    down: torch.Tensor      # [H, I]


@dataclass
class DecoderWeights:
    embed: torch.Tensor     # [V, H]
    layers: list[LayerWeights]
    final_ln: torch.Tensor
    lm_head: torch.Tensor   # [V, H] (untied, configuration_mineru_diffusion.py:24)


def make_weights(cfg: DecoderConfig, seed: int, dtype=torch.bfloat16, std: float = 0.02) -> DecoderWeights:
    """Seeded N(0, std) matrices drawn in fp32 and rounded to ``dtype``; every
    RMSNorm weight is 1 (mineru_diffusion/modeling_mineru_diffusion.py:317-328)."""
    g = torch.Generator().manual_seed(seed)

    def mat(r, c):
        return (torch.randn(r, c, generator=g, dtype=torch.float32) * std).to(dtype)

    h, i, d = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads
    embed = mat(cfg.vocab_size, h)
    layers = []
    for _ in range(cfg.num_hidden_layers):
        layers.append(LayerWeights(
            input_ln=torch.ones(h, dtype=dtype),
            qkv=mat((hq + 2 * hkv) * d, h),
            q_norm=torch.ones(d, dtype=dtype),
            k_norm=torch.ones(d, dtype=dtype),
            o=mat(h, hq * d),
            post_ln=torch.ones(h, dtype=dtype),
            gate_up=mat(2 * i, h),
            down=mat(h, i),
        ))
    final_ln = torch.ones(h, dtype=dtype)
    lm_head = mat(cfg.vocab_size, h)
    return DecoderWeights(embed, layers, final_ln, lm_head)


@dataclass
class StepContext:
    """Per-step metadata, the fields of NV/utils/context.py:5-15."""
    is_prefill: bool
    slot_mapping: torch.Tensor            # int32, [N] prefill / [bs, B] decode
    cu_seqlens_q: torch.Tensor | None = None
    cu_seqlens_k: torch.Tensor | None = None
    context_lens: torch.Tensor | None = None
    block_tables: torch.Tensor | None = None
    block_size: int = 32


class Decoder:
    """Restates SDARModel.forward / SDARDecoderLayer.forward / SDARAttention.forward
    (NV/models/sdar.py:68-85,109-113,141-154,167-181) and Attention.forward
    (NV/layers/sdar_attention.py:34-57) over a paged cache laid out as
    kv_cache[2, L, pages, PAGE, Hkv, D] (NV/engine/model_runner.py:113)."""

    def __init__(self, cfg: DecoderConfig, weights: DecoderWeights, num_pages: int, dtype=torch.bfloat16):
        self.cfg = cfg
        self.w = weights
        self.dtype = dtype
        self.kv_cache = torch.zeros(2, cfg.num_hidden_layers, num_pages, PAGE,
                                    cfg.num_key_value_heads, cfg.head_dim, dtype=dtype)
        self.rope = rope_table(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta)
        self.scale = cfg.head_dim ** -0.5
        self.round_p = True              # decode attention rounds probabilities to bf16 before PV, as flash-attn does
        self.trace: dict | None = None   # filled with intermediates when set to {}

    def embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.w.embed[input_ids]

    def forward(self, inputs_embeds: torch.Tensor, positions: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """inputs_embeds [N, H] (prefill, packed) or [bs, B, H] (decode);
        positions of matching leading shape.  Returns final-norm hidden states."""
        cfg = self.cfg
        hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        eps = cfg.rms_norm_eps
        hidden = inputs_embeds
        residual = None
        lead = positions.shape
        for li, lw in enumerate(self.w.layers):
            if residual is None:
                x, residual = rms_norm(hidden, lw.input_ln, eps), hidden
            else:
                x, residual = add_rms_norm(hidden, residual, lw.input_ln, eps)
            qkv = linear(x, lw.qkv)
            q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
            q = q.reshape(*lead, hq, d)
            k = k.reshape(*lead, hkv, d)
            v = v.reshape(*lead, hkv, d)
            q = rms_norm(q, lw.q_norm, eps)
            k = rms_norm(k, lw.k_norm, eps)
            q = apply_rope(q, positions, self.rope)
            k = apply_rope(k, positions, self.rope)
            k_cache, v_cache = self.kv_cache[0, li], self.kv_cache[1, li]
            store_kvcache(k.reshape(-1, hkv, d), v.reshape(-1, hkv, d), k_cache, v_cache, ctx.slot_mapping)
            if ctx.is_prefill:
                o = attn_staircase_varlen(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.block_size)
                o = o.flatten(1)
            else:
                o = attn_paged(q, k_cache, v_cache, ctx.context_lens, ctx.block_tables, self.scale, round_p=self.round_p)
                o = o.flatten(2)
            if self.trace is not None and li == 0:
                self.trace.update(q0=q.clone(), k0=k.clone(), v0=v.clone(), attn0=o.clone())
            hidden = linear(o, lw.o)
            x, residual = add_rms_norm(hidden, residual, lw.post_ln, eps)
            gate_up = linear(x, lw.gate_up)
            act = silu_mul(gate_up)
            hidden = linear(act, lw.down)
            if self.trace is not None and li == 0:
                self.trace.update(layer0_out=hidden.clone(), layer0_res=residual.clone())
        hidden, _ = add_rms_norm(hidden, residual, self.w.final_ln, eps)
        return hidden

    def compute_rows(self, hidden: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """The rows the LM head sees (NV/layers/embed_head.py:63-66): in prefill the
        last B rows of every sequence, otherwise every row."""
        if ctx.is_prefill:
            b = ctx.block_size
            starts = ctx.cu_seqlens_q[1:].long() - b
            idx = starts.unsqueeze(1) + torch.arange(b)
            hidden = hidden[idx].contiguous()
        return hidden

    def compute_logits(self, hidden: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """NV/layers/embed_head.py:61-72: prefill keeps the last B rows of every
        sequence; logits are rounded to the storage dtype."""
        return linear(self.compute_rows(hidden, ctx), self.w.lm_head)


# --------------------------------------------------------------------------
# model runner (the reference's boundary, restated for CPU)
# --------------------------------------------------------------------------
class OracleModelRunner:
    """CPU stand-in for ModelRunner.run (NV/engine/model_runner.py:127-219) and
    Sampler.forward (NV/layers/sampler.py:24-61).  ``seqs`` are duck-typed
    Sequence objects (NV/engine/sequence.py).  ``noise_fn(step_index, shape)``
    returns the Gumbel noise tensor of a step, or None for plain argmax.
    ``prompt_embeds`` maps seq_id -> [num_prompt_tokens, H] rows that replace
    the token embeddings of the prompt (the synthetic visual embeddings)."""

    def __init__(self, cfg: DecoderConfig, weights: DecoderWeights, num_pages: int, block_size: int = 32,
                 mask_token_id: int = 151669, noise_fn=None, prompt_embeds: dict | None = None):
        self.decoder = Decoder(cfg, weights, num_pages)
        self.block_size = block_size
        self.mask_token_id = mask_token_id
        self.noise_fn = noise_fn
        self.prompt_embeds = prompt_embeds or {}
        self.step_index = 0
        self.last: dict = {}
        self._block_passes: dict = {}    # seq_id -> (length at block start, passes made on the block)

    # NV/engine/model_runner.py:127-167
    def prepare_prefill(self, seqs):
        b = self.block_size
        ids, pos, slots, cu = [], [], [], [0]
        for seq in seqs:
            seqlen = len(seq) + b
            ids.extend(list(seq[seq.num_cached_tokens:]) + seq.current_denoising_block.tolist())
            pos.extend(range(seq.num_cached_tokens, seqlen))
            cu.append(cu[-1] + seqlen - seq.num_cached_tokens)
            if not seq.block_table:
                continue
            slots.extend(get_slots(seq.block_table, seq.num_cached_tokens, len(seq)) + [-1] * b)
        cu_t = torch.tensor(cu, dtype=torch.int32)
        ctx = StepContext(True, torch.tensor(slots, dtype=torch.int32), cu_t, cu_t.clone(), block_size=b)
        return torch.tensor(ids, dtype=torch.int64), torch.tensor(pos, dtype=torch.int64), ctx

    # NV/engine/model_runner.py:169-185
    def prepare_decode(self, seqs):
        b = self.block_size
        ids = [seq.current_denoising_block.tolist() for seq in seqs]
        pos = [list(range(len(seq), len(seq) + b)) for seq in seqs]
        lens = [len(seq) + b for seq in seqs]
        slots = [get_slots(seq.block_table, len(seq), len(seq) + b) for seq in seqs]
        tables = pad_block_tables([seq.block_table for seq in seqs])
        ctx = StepContext(False, torch.tensor(slots, dtype=torch.int32),
                          context_lens=torch.tensor(lens, dtype=torch.int32),
                          block_tables=torch.tensor(tables, dtype=torch.int32), block_size=b)
        return torch.tensor(ids, dtype=torch.int64), torch.tensor(pos, dtype=torch.int64), ctx

    def _embed(self, seqs, ids, is_prefill):
        emb = self.decoder.embed(ids)
        if is_prefill and self.prompt_embeds:
            emb = emb.clone()
            off = 0
            for seq in seqs:
                n = len(seq) + self.block_size
                pe = self.prompt_embeds.get(seq.seq_id)
                if pe is not None:
                    emb[off:off + pe.shape[0]] = pe.to(emb.dtype)
                off += n
        return emb

    def run(self, seqs, is_prefill: bool) -> int:
        ids, pos, ctx = self.prepare_prefill(seqs) if is_prefill else self.prepare_decode(seqs)
        temps = torch.tensor([seq.temperature for seq in seqs], dtype=torch.float32).unsqueeze(1)
        hidden = self.decoder.forward(self._embed(seqs, ids, is_prefill), pos, ctx)
        logits = self.decoder.compute_logits(hidden, ctx)
        logits = logits.reshape(len(seqs), self.block_size, -1)
        noise = self.noise_fn(self.step_index, logits.shape) if self.noise_fn else None
        x0, x0_p = sampler_prepare(logits, temps, noise)
        blocks = torch.stack([seq.current_denoising_block for seq in seqs], dim=0)
        thr = seqs[0].sampling_params.dynamic_threshold
        quotas = None
        steps = getattr(seqs[0].sampling_params, "denoising_steps", None)
        if steps:
            # pass s of a block takes num_transfer_tokens[min(s, steps - 1)] (modeling_mineru_diffusion.py:712)
            table = num_transfer_tokens(self.block_size, int(steps))
            quotas = []
            for seq in seqs:
                at, done = self._block_passes.get(seq.seq_id, (-1, 0))
                if at != len(seq):
                    done = 0
                quotas.append(table[min(done, len(table) - 1)])
                self._block_passes[seq.seq_id] = (len(seq), done + 1)
        new_blocks, transfer = unmask_decision(blocks, x0, x0_p, seqs[0].mask_token_id, thr, quotas)
        for i, seq in enumerate(seqs):
            seq.current_denoising_block = new_blocks[i]
            seq.current_step_map[transfer[i]] = seq.current_denoise_step
            seq.current_denoise_step += 1
        self.last = dict(logits=logits, x0=x0, x0_p=x0_p, transfer=transfer, hidden=hidden, ctx=ctx,
                         input_ids=ids, positions=pos)
        self.step_index += 1
        return int(transfer.sum())


# --------------------------------------------------------------------------
# timing aid for the CPU baseline
# --------------------------------------------------------------------------
_NATIVE_LINEAR = False


def use_native_linear(flag: bool) -> None:
    """Parity tests keep the fp32 restatement of ``linear``.  The CPU baseline
    of the benchmark switches to ``torch.nn.functional.linear`` on the storage
    dtype, which is the call the reference itself makes on a CPU
    (NV/layers/linear.py:73,154), so that the timed work is the reference's."""
    global _NATIVE_LINEAR, linear
    _NATIVE_LINEAR = flag
    if flag:
        import torch.nn.functional as F
        linear = lambda x, w: F.linear(x, w)  # noqa: E731
    else:
        linear = _linear_fp32


_linear_fp32 = linear
