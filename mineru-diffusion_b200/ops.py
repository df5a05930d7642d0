"""Op-level interface of the decode hot path, named after the reference ops
they stand in for.  Each function takes CUDA tensors, checks what the C ABI
cannot (dtype, device, contiguity) and calls libmdb200 on the current stream.
torch is used for memory and streams only; no function here computes in torch
and none has a fallback.
"""
from __future__ import annotations


import torch

from . import _lib

_BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (libmdb200 has no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")


def _rows(t: torch.Tensor, name: str) -> int:
    """Row stride (elements) of a 2-D view whose last dim is dense."""
    if t.stride(-1) != 1:
        raise ValueError(f"{name}: last dimension must be contiguous")
    return t.stride(0)


OPT_PDL = 1             # programmatic dependent launch between kernels (default on)
OPT_GEMM_PAIR = 3       # many-row GEMMs on CTA pairs (tcgen05.mma.cta_group::2): 1 from 2048 rows (default), 2 from 256, 0 never
OPT_WAIT_LIMIT_US = 4   # bound of every in-kernel wait in microseconds (default 2 s); expiry raises status bit 16


def set_option(option: int, value: int) -> None:
    _lib.check(_lib.lib().mdb_set_option(option, value), "mdb_set_option")


def get_option(option: int) -> int:
    return int(_lib.lib().mdb_get_option(option))


def pick_ksplit(m: int, n: int, k: int) -> int:
    """Split-k factor suited to the kernel that (m, n, k) will run on."""
    return int(_lib.lib().mdb_gemm_pick_ksplit(m, n, k))


# --------------------------------------------------------------------------
def store_kvcache(key: torch.Tensor, value: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    """``store_kvcache`` of the reference (nanovllm/layers/attention.py:33-40):
    key/value [N, Hkv, D] (or [bs, B, Hkv, D]), caches [pages, 256, Hkv, D],
    slot_mapping int32 with -1 = skip."""
    if key.dim() == 4:
        key = key.reshape(-1, *key.shape[2:])
        value = value.reshape(-1, *value.shape[2:])
    slot_mapping = slot_mapping.reshape(-1)
    n, h, d = key.shape
    for t, nm in ((key, "key"), (value, "value"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _need(t, _BF16, nm)
    _need(slot_mapping, torch.int32, "slot_mapping")
    if not (key.stride(-1) == 1 and value.stride(-1) == 1 and key.stride(1) == d and value.stride(1) == d):
        raise ValueError("key/value heads must be densely packed")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("caches must be contiguous")
    if slot_mapping.numel() != n:
        raise ValueError("slot_mapping must have one entry per row")
    num_slots = k_cache.numel() // (h * d)
    _lib.check(_lib.lib().mdb_kv_commit(key.data_ptr(), key.stride(0), value.data_ptr(), value.stride(0),
                                        k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(), n, h * d,
                                        num_slots, _stream()), "mdb_kv_commit")


def default_nsplit(bs: int, block: int, hq: int, hkv: int, max_ctx: int) -> int:
    """Key-range parts per request.  Measured on B200 over 1..32 requests and
    contexts of 0.6K..8K: the best part count fills the 148 SMs once and no
    more (a second wave of parts costs more than it saves, and from about 16
    requests up any split loses), with at most 16 parts; the kernels
    themselves never make a part shorter than 256 keys."""
    group = hq // hkv
    tokens_per_cta = max(1, min(block, (64 if group * block <= 64 else 128) // group))
    ctas = max(1, bs * hkv * -(-block // tokens_per_cta))
    want = 148 // ctas
    parts = max(1, max_ctx // 256)
    return int(max(1, min(want, parts, 16)))


def attn_workspace_bytes(bs: int, block: int, hq: int, nsplit: int) -> int:
    """Scratch bytes ``block_attn_with_kvcache`` needs for ``nsplit`` key-range parts (0 for one part)."""
    return int(_lib.lib().mdb_attn_paged_workspace_bytes(bs, block, hq, nsplit))


def _block_attn_args(q, k_cache, v_cache, cache_seqlens, block_table, out):
    """Shape, type and layout checks shared by the two paged-attention wrappers:
    the kernels hard-code head size 128 and 256-token pages and index the page
    table with unit stride inside a row."""
    if q.dim() != 4 or k_cache.dim() != 4:
        raise ValueError("q must be [bs, block, Hq, 128] and the caches [pages, 256, Hkv, 128]")
    bs, block, hq, d = q.shape
    pages, page, hkv, d2 = k_cache.shape
    if d != 128 or d2 != 128 or page != 256:
        raise ValueError("head_dim must be 128 and pages 256 tokens")
    if v_cache.shape != k_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    tensors = [(q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache")]
    if out is not None:
        if out.shape != q.shape:
            raise ValueError("out must have the shape of q")
        tensors.append((out, "out"))
    for t, nm in tensors:
        _need(t, _BF16, nm)
        if not t.is_contiguous():
            raise ValueError(f"{nm} must be contiguous")
    _need(cache_seqlens, torch.int32, "cache_seqlens")
    _need(block_table, torch.int32, "block_table")
    if cache_seqlens.numel() < bs or not cache_seqlens.is_contiguous():
        raise ValueError("cache_seqlens must hold one contiguous int32 per request")
    if block_table.dim() != 2 or block_table.shape[0] < bs or (block_table.shape[1] > 1 and block_table.stride(1) != 1):
        raise ValueError("block_table must be [bs, pages per request] with unit stride inside a row")
    return bs, block, hq, hkv, pages, d


def block_attn_with_kvcache(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                            cache_seqlens: torch.Tensor, block_table: torch.Tensor, softmax_scale: float | None = None,
                            nsplit: int | None = None, workspace: torch.Tensor | None = None,
                            out: torch.Tensor | None = None, max_ctx: int | None = None) -> torch.Tensor:
    """Stands in for ``flash_attn_with_kvcache(..., causal=False)`` as the
    reference calls it (nanovllm/layers/sdar_attention.py:50-55).
    q [bs, B, Hq, 128]; caches [pages, 256, Hkv, 128]."""
    bs, block, hq, hkv, pages, d = _block_attn_args(q, k_cache, v_cache, cache_seqlens, block_table, out)
    if softmax_scale is None:
        softmax_scale = d ** -0.5
    if nsplit is None:
        nsplit = default_nsplit(bs, block, hq, hkv, max_ctx if max_ctx is not None else block_table.shape[1] * 256)
    if out is None:
        out = torch.empty_like(q)
    need = _lib.lib().mdb_attn_paged_workspace_bytes(bs, block, hq, nsplit)
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _lib.check(_lib.lib().mdb_attn_block_paged(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                               block_table.data_ptr(), block_table.stride(0), cache_seqlens.data_ptr(),
                                               bs, block, hq, hkv, pages, float(softmax_scale), nsplit,
                                               _ptr(workspace), ws_bytes, _stream()), "mdb_attn_block_paged")
    return out


def block_attn_with_kvcache_noalloc(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                                    cache_seqlens: torch.Tensor, block_table: torch.Tensor, out: torch.Tensor,
                                    softmax_scale: float | None = None, nsplit: int = 1) -> torch.Tensor:
    """``block_attn_with_kvcache`` for hosts that cannot hand over scratch memory
    (all device memory already given to the KV-cache pool, or a thread that must
    stay out of the allocator): the split partials use a fixed 8 MiB array
    inside the library, so neither this wrapper nor the call allocates -- the
    caller passes ``out``.  Raises ``MdbError`` when (bs, nsplit) need more than
    that array.  Calls share the array; keep them on one stream."""
    bs, block, hq, hkv, pages, d = _block_attn_args(q, k_cache, v_cache, cache_seqlens, block_table, out)
    if softmax_scale is None:
        softmax_scale = d ** -0.5
    _lib.check(_lib.lib().mdb_attn_block_paged_noalloc(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                       out.data_ptr(), block_table.data_ptr(), block_table.stride(0),
                                                       cache_seqlens.data_ptr(), bs, block, hq, hkv, pages,
                                                       float(softmax_scale), nsplit, _stream()),
               "mdb_attn_block_paged_noalloc")
    return out


def sparse_attn_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q: torch.Tensor,
                       cu_seqlens_k: torch.Tensor, staircase_size: int = 4, max_seqlen: int | None = None,
                       out: torch.Tensor | None = None) -> torch.Tensor:
    """``sparse_attn_varlen`` of the reference
    (nanovllm/kernels/triton/attention/block_prefill_attention_v2.py:201-202):
    q [N, Hq, 128], k/v [N, Hkv, 128] packed; cu_seqlens int32 [nseq+1]."""
    n, hq, d = q.shape
    hkv = k.shape[1]
    if d != 128:
        raise ValueError("head_dim must be 128")
    if staircase_size not in (1, 2, 4, 8, 16, 32, 64, 128):
        raise AssertionError("staircase_size must be a power of two up to 128")
    for t, nm in ((q, "q"), (k, "k"), (v, "v")):
        _need(t, _BF16, nm)
        if t.stride(-1) != 1 or t.stride(1) != d:
            raise ValueError(f"{nm}: heads must be densely packed")
    _need(cu_seqlens_q, torch.int32, "cu_seqlens_q")
    if cu_seqlens_k is not cu_seqlens_q and cu_seqlens_k.data_ptr() != cu_seqlens_q.data_ptr():
        # the reference kernel assumes q and k lengths agree (self-attention)
        if not torch.equal(cu_seqlens_q, cu_seqlens_k):
            raise ValueError("query and key lengths must agree")
    nseq = cu_seqlens_q.numel() - 1
    if max_seqlen is None:
        max_seqlen = int((cu_seqlens_q[1:] - cu_seqlens_q[:-1]).max().item()) if nseq > 0 else 0
    if out is None:
        out = torch.empty((n, hq, d), dtype=_BF16, device=q.device)
    _lib.check(_lib.lib().mdb_attn_staircase_varlen(q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(),
                                                    v.stride(0), out.data_ptr(), out.stride(0),
                                                    cu_seqlens_q.data_ptr(), nseq, max_seqlen, n, hq, hkv,
                                                    staircase_size, _stream()), "mdb_attn_staircase_varlen")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear(x, weight)`` without bias for bf16 [.., K] x [N, K]."""
    _need(x, _BF16, "x")
    _need(weight, _BF16, "weight")
    if not weight.is_contiguous():
        raise ValueError("weight must be contiguous")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    n = weight.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=_BF16, device=x.device)
    _lib.check(_lib.lib().mdb_gemm_bf16(x2.data_ptr(), _rows(x2, "x"), weight.data_ptr(), out.data_ptr(),
                                        _rows(out, "out"), m, n, k, _stream()), "mdb_gemm_bf16")
    return out.reshape(*lead, n)


def gemm_splitk_partials(x: torch.Tensor, weight: torch.Tensor, ksplit: int, partials: torch.Tensor | None = None):
    """fp32 split-k slices [ksplit, m, n] of x W^T (m <= 64)."""
    m, k = x.shape
    n = weight.shape[0]
    if partials is None:
        partials = torch.empty((ksplit, m, n), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().mdb_gemm_splitk_partials(x.data_ptr(), _rows(x, "x"), weight.data_ptr(), partials.data_ptr(),
                                                   m, n, k, ksplit, _stream()), "mdb_gemm_splitk_partials")
    return partials


def gateup_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """gate_up projection + SiLU*mul in one pass over the weight (m <= 64)."""
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    if out is None:
        out = torch.empty((m, inter), dtype=_BF16, device=x.device)
    _lib.check(_lib.lib().mdb_gemm_gateup_swiglu(x.data_ptr(), _rows(x, "x"), w_gate_up.data_ptr(), out.data_ptr(),
                                                 _rows(out, "out"), m, inter, k, _stream()), "mdb_gemm_gateup_swiglu")
    return out


def silu_and_mul(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``SiluAndMul`` of the reference (nanovllm/layers/activation.py:12-15)."""
    _need(x, _BF16, "x")
    x2 = x.reshape(-1, x.shape[-1])
    m, two_i = x2.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((m, inter), dtype=_BF16, device=x.device)
    _lib.check(_lib.lib().mdb_silu_mul(x2.data_ptr(), _rows(x2, "x"), out.data_ptr(), _rows(out, "out"), m, inter,
                                       _stream()), "mdb_silu_mul")
    return out.reshape(*x.shape[:-1], inter)


def add_rms_norm(x: torch.Tensor | None, residual: torch.Tensor | None, weight: torch.Tensor, eps: float,
                 partials: torch.Tensor | None = None, out: torch.Tensor | None = None,
                 residual_out: torch.Tensor | None = None):
    """``RMSNorm.forward`` of the reference (nanovllm/layers/layernorm.py:42-50).
    Input rows come from ``x`` (bf16 [m, h]) or from fp32 split-k ``partials``
    [s, m, h].  Returns (y, new_residual); without ``residual`` the new
    residual is the input row itself."""
    src = x if x is not None else partials
    m, h = src.shape[-2], src.shape[-1]
    dev = src.device
    if out is None:
        out = torch.empty((m, h), dtype=_BF16, device=dev)
    if residual_out is None:
        residual_out = torch.empty((m, h), dtype=_BF16, device=dev)
    nparts = 0 if partials is None else partials.shape[0]
    _lib.check(_lib.lib().mdb_add_rmsnorm(_ptr(x), _ptr(partials), nparts, _ptr(residual), weight.data_ptr(),
                                          float(eps), out.data_ptr(), residual_out.data_ptr(), m, h, _stream()),
               "mdb_add_rmsnorm")
    return out, residual_out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    y, _ = add_rms_norm(x.reshape(-1, x.shape[-1]), None, weight, eps)
    return y.reshape(x.shape)


def qknorm_rope_commit(qkv: torch.Tensor | None, positions: torch.Tensor, rope_table: torch.Tensor,
                       q_norm_w: torch.Tensor, k_norm_w: torch.Tensor, eps: float, hq: int, hkv: int,
                       slot_mapping: torch.Tensor | None = None, k_cache: torch.Tensor | None = None,
                       v_cache: torch.Tensor | None = None, partials: torch.Tensor | None = None,
                       q_out: torch.Tensor | None = None, k_out: torch.Tensor | None = None,
                       v_out: torch.Tensor | None = None, want_kv: bool = False):
    """q/k per-head RMSNorm, rotary embedding and KV store after qkv_proj
    (nanovllm/models/sdar.py:74-82, nanovllm/layers/sdar_attention.py:37-38)."""
    src = qkv if qkv is not None else partials
    m = src.shape[-2]
    dev = src.device
    d = 128
    _need(positions, torch.int64, "positions")
    _need(rope_table, torch.float32, "rope_table")
    if q_out is None:
        q_out = torch.empty((m, hq, d), dtype=_BF16, device=dev)
    if want_kv and k_out is None:
        k_out = torch.empty((m, hkv, d), dtype=_BF16, device=dev)
        v_out = torch.empty((m, hkv, d), dtype=_BF16, device=dev)
    num_slots = 0 if k_cache is None else k_cache.numel() // (hkv * d)
    if slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
    nparts = 0 if partials is None else partials.shape[0]
    _lib.check(_lib.lib().mdb_qknorm_rope_commit(_ptr(qkv), 0 if qkv is None else _rows(qkv, "qkv"), _ptr(partials),
                                                 nparts, positions.data_ptr(), rope_table.data_ptr(),
                                                 rope_table.shape[0], q_norm_w.data_ptr(), k_norm_w.data_ptr(),
                                                 float(eps), _ptr(slot_mapping), q_out.data_ptr(), _ptr(k_out),
                                                 _ptr(v_out), _ptr(k_cache), _ptr(v_cache), num_slots, m, hq, hkv,
                                                 _stream()), "mdb_qknorm_rope_commit")
    return q_out, k_out, v_out


def qkv_rope_commit_supported(m: int, k: int) -> bool:
    """Whether ``qkv_proj_rope_commit`` takes this step: many rows, on the tcgen05 kernels."""
    return m > 64 and k % 64 == 0


def qkv_proj_rope_commit(x: torch.Tensor, w_qkv: torch.Tensor, positions: torch.Tensor, rope_table: torch.Tensor,
                         q_norm_w: torch.Tensor, k_norm_w: torch.Tensor, eps: float, hq: int, hkv: int,
                         slot_mapping: torch.Tensor | None = None, k_cache: torch.Tensor | None = None,
                         v_cache: torch.Tensor | None = None, q_out: torch.Tensor | None = None,
                         k_out: torch.Tensor | None = None, v_out: torch.Tensor | None = None):
    """``qkv_proj`` + ``qknorm_rope_commit`` as one kernel for many rows
    (nanovllm/models/sdar.py:73-82, nanovllm/layers/sdar_attention.py:37-38):
    the projection output stays in tensor memory."""
    _need(x, _BF16, "x")
    _need(w_qkv, _BF16, "w_qkv")
    _need(positions, torch.int64, "positions")
    _need(rope_table, torch.float32, "rope_table")
    m, k = x.shape
    d = 128
    if w_qkv.shape[0] != (hq + 2 * hkv) * d or w_qkv.shape[1] != k:
        raise ValueError("w_qkv must be [(hq + 2 hkv) * 128, k]")
    if q_out is None:
        q_out = torch.empty((m, hq, d), dtype=_BF16, device=x.device)
    num_slots = 0 if k_cache is None else k_cache.numel() // (hkv * d)
    if slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
    _lib.check(_lib.lib().mdb_gemm_qkv_rope_commit(x.data_ptr(), _rows(x, "x"), w_qkv.data_ptr(), m, k,
                                                   positions.data_ptr(), rope_table.data_ptr(), rope_table.shape[0],
                                                   q_norm_w.data_ptr(), k_norm_w.data_ptr(), float(eps),
                                                   _ptr(slot_mapping), q_out.data_ptr(), _ptr(k_out), _ptr(v_out),
                                                   _ptr(k_cache), _ptr(v_cache), num_slots, hq, hkv, _stream()),
               "mdb_gemm_qkv_rope_commit")
    return q_out, k_out, v_out


def gather_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``F.embedding`` row gather for bf16 tables and int64 ids."""
    _need(table, _BF16, "table")
    _need(ids, torch.int64, "ids")
    ids = ids.reshape(-1)
    m, h = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((m, h), dtype=_BF16, device=table.device)
    _lib.check(_lib.lib().mdb_gather_rows(table.data_ptr(), table.shape[0], ids.data_ptr(), out.data_ptr(), m, h,
                                          _stream()), "mdb_gather_rows")
    return out


def lmhead_workspace_bytes(m: int, vocab: int) -> int:
    return int(_lib.lib().mdb_lmhead_workspace_bytes(m, vocab))


def lm_head_sample(hidden: torch.Tensor, weight: torch.Tensor, temperatures: torch.Tensor, block: int,
                   noise: torch.Tensor | None = None, seed: int | None = None, step: int = 0,
                   step_dev: torch.Tensor | None = None, workspace: torch.Tensor | None = None,
                   x0: torch.Tensor | None = None, conf: torch.Tensor | None = None):
    """LM head + ``Sampler.prepare`` fused (nanovllm/layers/embed_head.py:61-72,
    nanovllm/layers/sampler.py:11-22).  hidden [m, H]; weight [V, H];
    temperatures fp32 [m // block].  Noise: explicit fp32 [m, V] tensor, or a
    ``seed`` for the counter-based generator, or neither for plain argmax.
    Returns (x0 int32 [m], confidence fp32 [m])."""
    _need(hidden, _BF16, "hidden")
    _need(weight, _BF16, "weight")
    _need(temperatures, torch.float32, "temperatures")
    m, h = hidden.shape
    vocab = weight.shape[0]
    mode = 1 if noise is not None else (2 if seed is not None else 0)
    if noise is not None:
        _need(noise, torch.float32, "noise")
        if tuple(noise.shape) != (m, vocab) or not noise.is_contiguous():
            raise ValueError("noise must be a contiguous [m, vocab] tensor")
    need = lmhead_workspace_bytes(m, vocab)
    if workspace is None or workspace.numel() * workspace.element_size() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=hidden.device)
    if x0 is None:
        x0 = torch.empty(m, dtype=torch.int32, device=hidden.device)
    if conf is None:
        conf = torch.empty(m, dtype=torch.float32, device=hidden.device)
    _lib.check(_lib.lib().mdb_lmhead_sample(hidden.data_ptr(), _rows(hidden, "hidden"), weight.data_ptr(), m, vocab, h,
                                            temperatures.data_ptr(), block, mode, _ptr(noise), int(seed or 0) & 0xFFFFFFFF,
                                            int(step) & 0xFFFFFFFF, _ptr(step_dev), workspace.data_ptr(),
                                            workspace.numel() * workspace.element_size(), x0.data_ptr(),
                                            conf.data_ptr(), _stream()), "mdb_lmhead_sample")
    return x0, conf


def logits_sample(logits: torch.Tensor, temperatures: torch.Tensor, block: int, noise: torch.Tensor | None = None,
                  seed: int | None = None, step: int = 0):
    """``Sampler.prepare`` (nanovllm/layers/sampler.py:11-22) on bf16 logits [m, V]."""
    _need(logits, _BF16, "logits")
    m, vocab = logits.shape
    mode = 1 if noise is not None else (2 if seed is not None else 0)
    need = lmhead_workspace_bytes(m, vocab)
    workspace = torch.empty(need, dtype=torch.uint8, device=logits.device)
    x0 = torch.empty(m, dtype=torch.int32, device=logits.device)
    conf = torch.empty(m, dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().mdb_logits_sample(logits.data_ptr(), _rows(logits, "logits"), m, vocab,
                                            temperatures.data_ptr(), block, mode, _ptr(noise),
                                            int(seed or 0) & 0xFFFFFFFF, int(step) & 0xFFFFFFFF, None,
                                            workspace.data_ptr(), need, x0.data_ptr(), conf.data_ptr(), _stream()),
               "mdb_logits_sample")
    return x0, conf


def gumbel_noise(m: int, vocab: int, seed: int, step: int, device) -> torch.Tensor:
    """The noise the counter-based generator adds for (seed, step)."""
    out = torch.empty((m, vocab), dtype=torch.float32, device=device)
    _lib.check(_lib.lib().mdb_gumbel_noise(out.data_ptr(), m, vocab, seed & 0xFFFFFFFF, step & 0xFFFFFFFF, _stream()),
               "mdb_gumbel_noise")
    return out


def unmask_decide(block_ids: torch.Tensor, x0: torch.Tensor, conf: torch.Tensor, mask_id: int, threshold: float,
                  quota: int = 1, transfer: torch.Tensor | None = None, counts: torch.Tensor | None = None,
                  quotas: torch.Tensor | None = None, status_out: torch.Tensor | None = None):
    """The unmask rule of ``Sampler.forward`` (nanovllm/layers/sampler.py:28-54)
    applied in place to block_ids int64 [bs, B]; returns (transfer uint8
    [bs, B], counts int32 [bs]).  ``quotas`` int32 [bs] gives every request its own
    quota (the HF twin's schedule, mineru_diffusion/modeling_mineru_diffusion.py:617-623).  ``status_out``
    (int32 [1], device) receives the device status word and clears it."""
    _need(block_ids, torch.int64, "block_ids")
    _need(x0, torch.int32, "x0")
    _need(conf, torch.float32, "conf")
    bs, block = block_ids.shape
    if quotas is not None:
        _need(quotas, torch.int32, "quotas")
        if quotas.numel() < bs or not quotas.is_contiguous():
            raise ValueError("quotas must be a contiguous int32 tensor with one entry per request")
    if transfer is None:
        transfer = torch.empty((bs, block), dtype=torch.uint8, device=block_ids.device)
    if counts is None:
        counts = torch.empty(bs, dtype=torch.int32, device=block_ids.device)
    _lib.check(_lib.lib().mdb_unmask_decide(block_ids.data_ptr(), x0.data_ptr(), conf.data_ptr(), bs, block,
                                            int(mask_id), float(threshold), int(quota), _ptr(quotas),
                                            transfer.data_ptr(), counts.data_ptr(), _ptr(status_out), _stream()),
               "mdb_unmask_decide")
    return transfer, counts


def num_transfer_tokens(block_length: int, steps: int) -> list[int]:
    """Quota of every denoising step of a block, ``get_num_transfer_tokens`` of the HF twin
    (mineru_diffusion/modeling_mineru_diffusion.py:617-623): ``block_length // steps`` tokens per step and
    one more in each of the first ``block_length % steps`` steps.  Step ``s`` of a block uses entry
    ``min(s, steps - 1)`` (:712)."""
    if steps < 1:
        raise ValueError("denoising_steps must be positive")
    base, rem = divmod(block_length, steps)
    return [base + (1 if s < rem else 0) for s in range(steps)]


# -------------------------------------------------------------------------- tensor-parallel pair
def gemm_splitk_partials_tp(x: torch.Tensor, weight: torch.Tensor, ksplit: int, local_ptr: int, peer_ptr: int,
                            peer_flags_ptr: int, tag: int, epoch: torch.Tensor) -> None:
    """Split-k slices of x W^T written to this rank's slice range locally and, over
    NVLink, in the peer's buffer; then the peer's flag slots are raised."""
    m, k = x.shape
    n = weight.shape[0]
    _lib.check(_lib.lib().mdb_gemm_splitk_partials_tp(x.data_ptr(), _rows(x, "x"), weight.data_ptr(), local_ptr,
                                                      peer_ptr, m, n, k, ksplit, peer_flags_ptr, tag,
                                                      epoch.data_ptr(), _stream()), "mdb_gemm_splitk_partials_tp")


def linear_tp_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, peer_ptr: int, peer_flags_ptr: int,
                   tag: int, epoch: torch.Tensor) -> int:
    """Many-row x W^T stored into ``out`` and, over NVLink, into the peer's landing buffer at ``peer_ptr``
    (same leading dimension as ``out``); then the peer's flag slots are raised.  Returns the number of
    flag slots (= CTAs launched) the consumer has to wait for."""
    import ctypes as C
    m, k = x.shape
    n = weight.shape[0]
    grid = C.c_int(0)
    _lib.check(_lib.lib().mdb_gemm_bf16_tp(x.data_ptr(), _rows(x, "x"), weight.data_ptr(), out.data_ptr(), peer_ptr,
                                           _rows(out, "out"), m, n, k, peer_flags_ptr, tag, epoch.data_ptr(),
                                           C.byref(grid), _stream()), "mdb_gemm_bf16_tp")
    return int(grid.value)


def add_rms_norm_tp_rows(x: torch.Tensor, x_peer: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                         out: torch.Tensor, residual_out: torch.Tensor, wait_flags_ptr: int, wait_count: int, tag: int,
                         epoch: torch.Tensor) -> None:
    """``add_rms_norm`` of bf16(x + x_peer) after the peer's flag slots show this launch's number."""
    m, h = x.shape
    _lib.check(_lib.lib().mdb_add_rmsnorm_tp_rows(x.data_ptr(), x_peer.data_ptr(), residual.data_ptr(),
                                                  weight.data_ptr(), float(eps), out.data_ptr(), residual_out.data_ptr(),
                                                  m, h, wait_flags_ptr, wait_count, tag, epoch.data_ptr(), _stream()),
               "mdb_add_rmsnorm_tp_rows")


def tp_grid_size(m: int, n: int, k: int, ksplit: int) -> int:
    return int(_lib.lib().mdb_tp_grid_size(m, n, k, ksplit))


def add_rms_norm_tp(partials: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                    out: torch.Tensor, residual_out: torch.Tensor, wait_flags_ptr: int, wait_count: int, tag: int,
                    epoch: torch.Tensor) -> None:
    """``add_rms_norm`` over [2*S, m, h] slices of both ranks after the peer's flag slots show this launch's number."""
    m, h = partials.shape[-2], partials.shape[-1]
    _lib.check(_lib.lib().mdb_add_rmsnorm_tp(None, partials.data_ptr(), partials.shape[0], residual.data_ptr(),
                                             weight.data_ptr(), float(eps), out.data_ptr(), residual_out.data_ptr(),
                                             m, h, wait_flags_ptr, wait_count, tag, epoch.data_ptr(), _stream()),
               "mdb_add_rmsnorm_tp")


def lm_head_sample_tp(hidden: torch.Tensor, weight: torch.Tensor, temperatures: torch.Tensor, block: int,
                      workspace: torch.Tensor, peer_workspace_ptr: int, tile_begin: int, tile_count: int,
                      peer_flags_ptr: int, wait_flags_ptr: int, wait_count: int, tag: int, epoch: torch.Tensor,
                      x0: torch.Tensor, conf: torch.Tensor, noise: torch.Tensor | None = None,
                      seed: int | None = None, step: int = 0, step_dev: torch.Tensor | None = None):
    """LM head + sampler statistics with the vocabulary split by 128-row tiles between the two ranks."""
    m, h = hidden.shape
    vocab = weight.shape[0]
    mode = 1 if noise is not None else (2 if seed is not None else 0)
    _lib.check(_lib.lib().mdb_lmhead_sample_tp(hidden.data_ptr(), _rows(hidden, "hidden"), weight.data_ptr(), m, vocab,
                                               h, temperatures.data_ptr(), block, mode, _ptr(noise),
                                               int(seed or 0) & 0xFFFFFFFF, int(step) & 0xFFFFFFFF, _ptr(step_dev),
                                               workspace.data_ptr(), peer_workspace_ptr,
                                               workspace.numel() * workspace.element_size(), tile_begin, tile_count,
                                               peer_flags_ptr, wait_flags_ptr, wait_count, tag, epoch.data_ptr(),
                                               x0.data_ptr(), conf.data_ptr(), _stream()), "mdb_lmhead_sample_tp")
    return x0, conf
