"""Writes the golden fixtures of this directory by executing the reference's
own modules on seeded inputs.

Run in a container that has the reference checkout:

    TORCHDYNAMO_DISABLE=1 TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference [fixture ...]

The reference's nano_dvlm layers are imported unchanged and run on CPU.  What
cannot run on a CPU is replaced by a shim *in this script only*:

* ``torch.compile``            -> disabled (TORCHDYNAMO_DISABLE=1), same eager code runs
* ``flash_attn_with_kvcache``  -> page gather + torch SDPA (flash-attn is CUDA-only)
* ``sparse_attn_varlen`` bf16  -> torch SDPA under the staircase mask; the Triton
  kernel itself is run through the Triton interpreter in fp32/fp16 and both its
  output and the mask it implies are stored
* liger ``SiluAndMul`` bf16    -> bf16(silu(fp32(gate))) * up (the interpreter
  returns NaN for bf16)
* ``.cuda()`` / ``pin_memory`` -> no-ops so the reference's own
  ``prepare_prefill`` / ``prepare_decode`` build the step tensors

Fixtures are .npz files; bf16 tensors are stored as their uint16 bit patterns.
"""
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
os.environ.setdefault("TRITON_INTERPRET", "1")

import math
from types import SimpleNamespace

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MINERU_DIFFUSION_REFERENCE", "")
if not REF or not os.path.isdir(REF):
    raise SystemExit("usage: make_golden.py <checkout of the reference repository>  (or MINERU_DIFFUSION_REFERENCE=...)")
sys.path.insert(0, os.path.join(REF, "engines", "nano_dvlm"))
sys.path.insert(0, REF)
sys.path.insert(0, ROOT)


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit pattern array."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = bits(v) if v.dtype == torch.bfloat16 else v.numpy()
        out[k] = np.asarray(v)
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **out)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


# ---------------------------------------------------------------- environment shims
torch.Tensor.cuda = lambda self, *a, **k: self  # noqa: E731  (CPU container)

if not dist.is_initialized():
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29577", world_size=1, rank=0)

from nanovllm.engine import model_runner as ref_mr            # noqa: E402
from nanovllm.engine.block_manager import BlockManager        # noqa: E402
from nanovllm.engine.scheduler import Scheduler               # noqa: E402
from nanovllm.engine.sequence import Sequence, SequenceStatus # noqa: E402
from nanovllm.layers import sdar_attention as ref_attn        # noqa: E402
from nanovllm.layers.activation import SiluAndMul             # noqa: E402
from nanovllm.layers.attention import store_kvcache           # noqa: E402
from nanovllm.layers.layernorm import RMSNorm                 # noqa: E402
from nanovllm.layers.rotary_embedding import RotaryEmbedding  # noqa: E402
from nanovllm.layers.sampler import Sampler                   # noqa: E402
from nanovllm.models.sdar import SDARForCausalLM              # noqa: E402
from nanovllm.sampling_params import SamplingParams           # noqa: E402
from nanovllm.utils.context import get_context, reset_context  # noqa: E402
from nanovllm.kernels.triton.attention.block_prefill_attention_v2 import (  # noqa: E402
    _staircase_attn_fwd_kernel_varlen_v2)


class _TorchNoPin:
    """torch, except that torch.tensor ignores pin_memory."""

    def __getattr__(self, k):
        return getattr(torch, k)

    @staticmethod
    def tensor(data, dtype=None, pin_memory=False, **kw):
        return torch.tensor(data, dtype=dtype, **kw)


ref_mr.torch = _TorchNoPin()


def make_ref_runner(block_size):
    r = object.__new__(ref_mr.ModelRunner)
    r.config = SimpleNamespace(block_size=block_size)
    r.rank = 0
    return r


# ---------------------------------------------------------------- 1. index contract
def gen_index_contract():
    """Drives the reference Scheduler / BlockManager / Sequence with a fake
    sampler and records the tensors its ModelRunner.prepare_* build each step."""
    g = torch.Generator().manual_seed(11)
    B, MASK = 32, 151669
    cfg = SimpleNamespace(max_num_seqs=4, max_num_batched_tokens=4096, eos=-1, num_kvcache_blocks=12,
                          kvcache_block_size=256)
    sched = Scheduler(cfg)
    runner = make_ref_runner(B)
    prompt_lens = [300, 45, 256, 511, 17]
    max_new = [96, 64, 64, 96, 32]
    Sequence.counter = __import__("itertools").count()
    for pl, mn in zip(prompt_lens, max_new):
        ids = torch.randint(0, 150000, (pl,), generator=g).tolist()
        sp = SamplingParams(temperature=1.0, max_new_tokens=mn, ignore_eos=True, stop_token_ids=[])
        sched.add(Sequence(ids, sp, denoising_block_size=B, mask_token_id=MASK))
    rec = {}
    step = 0
    while not sched.is_finished() and step < 400:
        seqs, is_prefill = sched.schedule()
        if is_prefill:
            ids, pos, _, _ = runner.prepare_prefill(seqs)
        else:
            ids, pos, _, _ = runner.prepare_decode(seqs)
        ctx = get_context()
        p = f"s{step:03d}_"
        rec[p + "is_prefill"] = np.array(int(is_prefill))
        rec[p + "seq_ids"] = np.array([s.seq_id for s in seqs])
        rec[p + "input_ids"] = ids.numpy()
        rec[p + "positions"] = pos.numpy()
        rec[p + "slot_mapping"] = ctx.slot_mapping.numpy()
        if is_prefill:
            rec[p + "cu_seqlens_q"] = ctx.cu_seqlens_q.numpy()
            rec[p + "cu_seqlens_k"] = ctx.cu_seqlens_k.numpy()
        else:
            rec[p + "context_lens"] = ctx.context_lens.numpy()
            rec[p + "block_tables"] = ctx.block_tables.numpy()
        reset_context()
        # fake sampler: unmask 1..16 random masked positions with random ids
        n_unmask = []
        for s in seqs:
            masked = (s.current_denoising_block == MASK).nonzero().flatten()
            if masked.numel() == 0:
                n_unmask.append(0)
                continue
            k = int(torch.randint(1, 17, (1,), generator=g))
            pick = masked[torch.randperm(masked.numel(), generator=g)[:k]]
            s.current_denoising_block[pick] = torch.randint(0, 150000, (pick.numel(),), generator=g)
            n_unmask.append(int(pick.numel()))
        rec[p + "n_unmask"] = np.array(n_unmask)
        rec[p + "blocks_after"] = torch.stack([s.current_denoising_block for s in seqs]).numpy()
        sched.postprocess(seqs)
        rec[p + "status_after"] = np.array([s.status.value for s in seqs])
        rec[p + "num_tokens_after"] = np.array([s.num_tokens for s in seqs])
        step += 1
    rec["num_steps"] = np.array(step)
    rec["prompt_lens"] = np.array(prompt_lens)
    rec["max_new"] = np.array(max_new)
    # stand-alone get_slots cases incl. page straddles and page-aligned ends
    seq = Sequence(list(range(700)), SamplingParams(stop_token_ids=[]), denoising_block_size=B, mask_token_id=MASK)
    seq.block_table = [7, 3, 11, 5]
    cases = [(0, 10), (250, 260), (255, 257), (240, 272), (0, 256), (256, 512), (500, 768), (511, 513), (700, 732),
             (736, 768), (10, 10)]
    rec["slots_table"] = np.array(seq.block_table)
    rec["slots_cases"] = np.array(cases)
    for i, (lo, hi) in enumerate(cases):
        rec[f"slots_{i}"] = np.array(seq.get_slots(lo, hi), dtype=np.int64)
    save("index_contract.npz", **rec)


# ---------------------------------------------------------------- 2. element-wise layers
def gen_layers():
    g = torch.Generator().manual_seed(12)
    bf = torch.bfloat16
    torch.set_default_dtype(bf)
    norm = RMSNorm(256, eps=1e-6)
    head_norm = RMSNorm(128, eps=1e-6)
    torch.set_default_dtype(torch.float32)
    norm.weight.data = (1.0 + 0.1 * torch.randn(256, generator=g)).to(bf)
    head_norm.weight.data = (1.0 + 0.1 * torch.randn(128, generator=g)).to(bf)
    x = torch.randn(40, 256, generator=g).to(bf)
    res = (3.0 * torch.randn(40, 256, generator=g)).to(bf)
    y_plain = norm(x.clone())
    y_add, res_out = norm(x.clone(), res.clone())
    heads = torch.randn(40, 6, 128, generator=g).to(bf)
    heads_normed = head_norm(heads.clone())

    rope = RotaryEmbedding(128, 128, 4096, 1000000.0)
    pos = torch.randint(0, 4096, (40,), generator=g)
    q = torch.randn(40, 4, 128, generator=g).to(bf)
    k = torch.randn(40, 2, 128, generator=g).to(bf)
    q_rot, k_rot = rope(pos, q.clone(), k.clone())
    table_probe = rope.cos_sin_cache[[0, 1, 17, 4095], 0, :].clone()

    # KV store through the reference's Triton kernel (interpreter)
    kc = torch.zeros(3, 256, 2, 128, dtype=bf)
    vc = torch.zeros(3, 256, 2, 128, dtype=bf)
    kk = torch.randn(40, 2, 128, generator=g).to(bf)
    vv = torch.randn(40, 2, 128, generator=g).to(bf)
    slots = torch.tensor(list(range(250, 270)) + [-1] * 5 + list(range(600, 615)), dtype=torch.int32)
    store_kvcache(kk, vv, kc, vc, slots)
    touched = sorted(set(int(s) for s in slots.tolist() if s >= 0))

    # liger SiLU*mul: fp32 through the interpreter, bf16 restated
    gu32 = torch.randn(8, 256, generator=g)
    silu32 = SiluAndMul.forward.__wrapped__(SiluAndMul(), gu32) if hasattr(SiluAndMul.forward, "__wrapped__") \
        else SiluAndMul()(gu32)
    save("layers.npz", norm_w=norm.weight.data, head_norm_w=head_norm.weight.data, x=x, res=res, y_plain=y_plain,
         y_add=y_add, res_out=res_out, heads=heads, heads_normed=heads_normed, rope_pos=pos, rope_q=q, rope_k=k,
         rope_q_out=q_rot, rope_k_out=k_rot, rope_table_probe=table_probe, kv_k=kk, kv_v=vv, kv_slots=slots,
         kv_touched=np.array(touched), kv_kc_rows=kc.view(-1, 256)[touched], kv_vc_rows=vc.view(-1, 256)[touched],
         kv_kc_sum=np.array(float(kc.float().abs().sum())), silu_in=gu32, silu_out=silu32)


# ---------------------------------------------------------------- 3. staircase kernel (Triton interpreter)
def run_triton_staircase(q, k, v, cu, stairs, block_m=32, block_n=64):
    n, hq, d = q.shape
    hkv = k.shape[1]
    o = torch.empty_like(q)
    grid = (cu.numel() - 1, hq)
    _staircase_attn_fwd_kernel_varlen_v2.fn[grid](
        q, k, v, o, cu, cu,
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        v.stride(0), v.stride(1), v.stride(2), o.stride(0), o.stride(1), o.stride(2),
        hq, hkv, q_scale=1.0 / math.sqrt(d) * 1.44269504,
        BLOCK_M=block_m, BLOCK_N=block_n, BLOCK_DMODEL=d, LOG2_STAIRS=int(math.log2(stairs)),
        NUM_HEADS_PER_KV_GROUP=hq // hkv)
    return o


def gen_staircase():
    g = torch.Generator().manual_seed(13)
    lens = [45, 32, 70]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    n = int(cu[-1])
    hq, hkv, d = 2, 1, 128
    # inputs are fp16-representable so the fp32 and fp16 runs share them and they store in half the space
    q = torch.randn(n, hq, d, generator=g).half().float()
    k = torch.randn(n, hkv, d, generator=g).half().float()
    v = torch.randn(n, hkv, d, generator=g).half().float()
    rec = dict(lens=np.array(lens), q=q.half(), k=k.half(), v=v.half())
    for stairs in (32, 8):
        rec[f"out_fp32_s{stairs}"] = run_triton_staircase(q, k, v, cu, stairs)
    # fp16 run: shows where the kernel rounds (q*scale -> fp16, p -> fp16)
    qh, kh, vh = q.half(), k.half(), v.half()
    rec["out_fp16_s32"] = run_triton_staircase(qh, kh, vh, cu, 32).float()
    # the same kernel in fp32 on inputs that bf16 holds exactly (stored as bf16 bit patterns): what a bf16
    # implementation is compared with when the rounding of its inputs is not to count as its error
    g2 = torch.Generator().manual_seed(113)
    lens_b = [70, 97, 33]
    cu_b = torch.tensor([0] + list(np.cumsum(lens_b)), dtype=torch.int32)
    nb = int(cu_b[-1])
    qb = torch.randn(nb, 2, d, generator=g2).to(torch.bfloat16)
    kb = torch.randn(nb, 1, d, generator=g2).to(torch.bfloat16)
    vb = torch.randn(nb, 1, d, generator=g2).to(torch.bfloat16)
    rec.update(lens_bf=np.array(lens_b), q_bf=bits(qb), k_bf=bits(kb), v_bf=bits(vb))
    for stairs in (32, 8):
        rec[f"out_fp32_bf_s{stairs}"] = run_triton_staircase(qb.float(), kb.float(), vb.float(), cu_b, stairs)
    # the HF twin's mask for the same shapes (prompt P, one generation block)
    from mineru_diffusion.modeling_mineru_diffusion import SDARForCausalLM as HFModel
    for P, gen, B in ((45, 32, 32), (5, 8, 4), (64, 64, 32), (70, 16, 8)):
        mask = HFModel._build_full_attention_mask(HFModel, P, gen, B, torch.device("cpu"))
        rec[f"hf_mask_{P}_{gen}_{B}"] = mask.numpy()
    save("staircase.npz", **rec)


# ---------------------------------------------------------------- 4. sampler
def gen_sampler():
    g = torch.Generator().manual_seed(14)
    B, V, MASK = 32, 256, 250
    sampler = Sampler()
    rec = {}
    for case, (temp, peaked) in enumerate([(1.0, False), (0.7, True), (0.05, False)]):
        bs = 3
        logits = torch.randn(bs, B, V, generator=g)
        if peaked:
            # a few positions get a dominant logit so that softmax prob > 0.9
            for r in range(bs):
                for p in torch.randperm(B, generator=g)[:5].tolist():
                    logits[r, p, int(torch.randint(0, V, (1,), generator=g))] += 14.0
        logits = logits.to(torch.bfloat16)
        expo = torch.empty(bs, B, V).exponential_(generator=g)
        gumbel = -expo.log()
        orig = torch.Tensor.exponential_
        torch.Tensor.exponential_ = lambda self, *a, **k: self.copy_(expo)  # noqa: E731
        seqs = []
        for r in range(bs):
            sp = SamplingParams(temperature=temp, dynamic_threshold=0.9, stop_token_ids=[])
            s = Sequence([1, 2, 3], sp, denoising_block_size=B, mask_token_id=MASK)
            s.current_step_map = torch.full((B,), -1, dtype=torch.int32)
            if r == 1:   # partly unmasked block
                s.current_denoising_block[torch.randperm(B, generator=g)[:20]] = 7
            if r == 2 and case == 2:   # fully unmasked (CACHING) row
                s.current_denoising_block[:] = 9
            s.current_denoise_step = 5
            seqs.append(s)
        before = torch.stack([s.current_denoising_block.clone() for s in seqs])
        temps = torch.tensor([[temp]] * bs, dtype=torch.float32)
        x0, x0_p = sampler.prepare(logits, temps)
        n = sampler(logits, temps, seqs)
        torch.Tensor.exponential_ = orig
        after = torch.stack([s.current_denoising_block for s in seqs])
        transfer = torch.stack([s.current_step_map == 5 for s in seqs])
        p = f"c{case}_"
        rec.update({p + "logits": logits, p + "temp": np.array(temp), p + "gumbel": gumbel, p + "before": before,
                    p + "after": after, p + "transfer": transfer, p + "x0": x0, p + "x0_p": x0_p,
                    p + "count": np.array(n)})
    rec["mask_id"] = np.array(MASK)
    rec["threshold"] = np.array(0.9)
    save("sampler.npz", **rec)


# ---------------------------------------------------------------- 5. tiny decoder through the reference modules
def sdpa_paged(q, k_cache, v_cache, cache_seqlens=None, block_table=None, softmax_scale=None, causal=False):
    """CPU stand-in for flash_attn_with_kvcache (non-causal, paged)."""
    assert not causal
    bs = q.shape[0]
    out = torch.empty_like(q)
    for r in range(bs):
        ctx = int(cache_seqlens[r])
        pages = (ctx + 255) // 256
        idx = block_table[r, :pages].long()
        k = k_cache[idx].reshape(pages * 256, *k_cache.shape[2:])[:ctx]
        v = v_cache[idx].reshape(pages * 256, *v_cache.shape[2:])[:ctx]
        o = F.scaled_dot_product_attention(q[r].transpose(0, 1)[None], k.transpose(0, 1)[None],
                                           v.transpose(0, 1)[None], scale=softmax_scale, enable_gqa=True)
        out[r] = o[0].transpose(0, 1)
    return out


def sdpa_staircase(q, k, v, cu_seqlens_q=None, cu_seqlens_k=None, staircase_size=32):
    """CPU stand-in for the Triton staircase kernel in bf16: SDPA under the
    mask the kernel implements (checked against the kernel in fp32 below)."""
    out = torch.empty_like(q)
    S = staircase_size
    for b in range(cu_seqlens_q.numel() - 1):
        s, e = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        T = e - s
        pad = (T + S - 1) // S * S - T
        i = torch.arange(T)
        limit = ((i + pad) // S + 1) * S - 1 - pad
        mask = torch.arange(T)[None, :] <= limit[:, None]
        o = F.scaled_dot_product_attention(q[s:e].transpose(0, 1)[None], k[s:e].transpose(0, 1)[None],
                                           v[s:e].transpose(0, 1)[None], attn_mask=mask, enable_gqa=True)
        out[s:e] = o[0].transpose(0, 1)
    return out


def gen_decoder():
    from oracle import nano_oracle as orc
    bf = torch.bfloat16
    B, MASK = 32, 500
    cfg = orc.DecoderConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=2048)
    w = orc.make_weights(cfg, seed=21)
    ns = SimpleNamespace(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                         intermediate_size=cfg.intermediate_size, num_hidden_layers=cfg.num_hidden_layers,
                         num_attention_heads=cfg.num_attention_heads, num_key_value_heads=cfg.num_key_value_heads,
                         head_dim=cfg.head_dim, max_position_embeddings=cfg.max_position_embeddings,
                         rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, rope_scaling=None,
                         attention_bias=False, hidden_act="silu", tie_word_embeddings=False)
    torch.set_default_dtype(bf)
    model = SDARForCausalLM(ns)
    torch.set_default_dtype(torch.float32)
    model.lm_head.set_denoise_block_size(B)
    model.model.embed_tokens.weight.data.copy_(w.embed)
    model.lm_head.weight.data.copy_(w.lm_head)
    model.model.norm.weight.data.copy_(w.final_ln)
    for layer, lw in zip(model.model.layers, w.layers):
        layer.input_layernorm.weight.data.copy_(lw.input_ln)
        layer.post_attention_layernorm.weight.data.copy_(lw.post_ln)
        layer.self_attn.qkv_proj.weight.data.copy_(lw.qkv)
        layer.self_attn.o_proj.weight.data.copy_(lw.o)
        layer.self_attn.q_norm.weight.data.copy_(lw.q_norm)
        layer.self_attn.k_norm.weight.data.copy_(lw.k_norm)
        layer.mlp.gate_up_proj.weight.data.copy_(lw.gate_up)
        layer.mlp.down_proj.weight.data.copy_(lw.down)
    pages = 6
    kv_cache = torch.zeros(2, cfg.num_hidden_layers, pages, 256, cfg.num_key_value_heads, cfg.head_dim, dtype=bf)
    li = 0
    for module in model.modules():
        if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
            module.k_cache = kv_cache[0, li]
            module.v_cache = kv_cache[1, li]
            li += 1
    ref_attn.flash_attn_with_kvcache = sdpa_paged
    ref_attn.sparse_attn_varlen = sdpa_staircase
    SiluAndMul.forward = lambda self, x: (lambda g_, u_: (g_.float() * torch.sigmoid(g_.float())).to(x.dtype) * u_)(
        *x.chunk(2, -1))

    g = torch.Generator().manual_seed(22)
    sched_cfg = SimpleNamespace(max_num_seqs=4, max_num_batched_tokens=4096, eos=-1, num_kvcache_blocks=pages,
                                kvcache_block_size=256)
    sched = Scheduler(sched_cfg)
    # shuffle the free list so page ids are not the identity
    sched.block_manager.free_block_ids = __import__("collections").deque([4, 1, 5, 0, 3, 2])
    runner = make_ref_runner(B)
    sampler = Sampler()
    prompt_lens = [300, 45]
    prompts = []
    Sequence.counter = __import__("itertools").count()
    for pl in prompt_lens:
        ids = torch.randint(0, 490, (pl,), generator=g).tolist()
        prompts.append(ids)
        sp = SamplingParams(temperature=1.0, max_new_tokens=64, ignore_eos=True, stop_token_ids=[], dynamic_threshold=0.9)
        s = Sequence(ids, sp, denoising_block_size=B, mask_token_id=MASK)
        s.current_step_map = torch.full((B,), -1, dtype=torch.int32)
        sched.add(s)
    rec = dict(prompt0=np.array(prompts[0]), prompt1=np.array(prompts[1]), mask_id=np.array(MASK))
    orig_exp = torch.Tensor.exponential_
    nsteps = 3
    with torch.inference_mode():
        for step in range(nsteps):
            seqs, is_prefill = sched.schedule()
            if is_prefill:
                ids, pos, _, _ = runner.prepare_prefill(seqs)
            else:
                ids, pos, _, _ = runner.prepare_decode(seqs)
            hidden = model(ids, pos)
            logits = model.compute_logits(hidden)
            logits = logits.reshape(len(seqs), B, -1)
            expo = torch.empty(logits.shape).exponential_(generator=g)
            torch.Tensor.exponential_ = lambda self, *a, **k: self.copy_(expo)  # noqa: E731
            temps = torch.tensor([[s.temperature] for s in seqs], dtype=torch.float32)
            x0, x0_p = sampler.prepare(logits, temps)
            n = sampler(logits, temps, seqs)
            torch.Tensor.exponential_ = orig_exp
            reset_context()
            p = f"s{step}_"
            rec.update({p + "is_prefill": np.array(int(is_prefill)), p + "logits": logits.to(bf),
                        p + "gumbel": -expo.log(), p + "x0": x0, p + "x0_p": x0_p, p + "count": np.array(n),
                        p + "blocks_after": torch.stack([s.current_denoising_block for s in seqs]),
                        p + "block_tables": np.array([s.block_table + [-1] * (3 - len(s.block_table)) for s in seqs]),
                        p + "kv_abs_sum": np.array([float(kv_cache[0].float().abs().sum()),
                                                    float(kv_cache[1].float().abs().sum())])})
            if is_prefill:
                # layer-0 K rows of the first prompt as cached (norm + rope applied)
                tab = seqs[0].block_table
                rec[p + "k_l0_first_rows"] = kv_cache[0, 0, tab[0], :8].clone()
                rec[p + "v_l0_first_rows"] = kv_cache[1, 0, tab[0], :8].clone()
            sched.postprocess(seqs)
    rec["num_steps"] = np.array(nsteps)
    save("decoder_tiny.npz", **rec)


# ---------------------------------------------------------------- 6. HF twin: quota rule and schedule
def gen_hf_twin():
    """``_select_transfer_index`` and ``get_num_transfer_tokens`` of the HF twin
    (mineru_diffusion/modeling_mineru_diffusion.py:518-532,617-623) on seeded confidences.  Cases keep at
    least ``count`` masked positions and distinct confidences: below that the reference's ``topk`` picks among
    -inf entries in an unspecified order."""
    from mineru_diffusion.modeling_mineru_diffusion import SDARForCausalLM as HFModel
    g = torch.Generator().manual_seed(31)
    rec = {}
    sched = [(32, 32), (32, 8), (32, 5), (32, 3), (16, 5), (64, 48), (8, 3), (32, 64)]
    rec["sched_pairs"] = np.array(sched)
    for b, steps in sched:
        rec[f"sched_{b}_{steps}"] = HFModel.get_num_transfer_tokens(b, steps).numpy()
    cases = []
    for block, count, n_masked, boost in [(32, 1, 32, 0), (32, 4, 20, 0), (32, 7, 7, 0), (32, 4, 20, 6), (32, 4, 20, 2),
                                          (16, 3, 9, 0), (64, 2, 40, 1), (8, 3, 8, 0), (32, 6, 32, 6)]:
        bs = 5
        conf = torch.rand(bs, block, generator=g) * 0.85            # below the threshold
        masked = torch.zeros(bs, block, dtype=torch.bool)
        for r in range(bs):
            masked[r, torch.randperm(block, generator=g)[:n_masked]] = True
            if boost:
                idx = masked[r].nonzero().flatten()
                pick = idx[torch.randperm(idx.numel(), generator=g)[:boost]]
                conf[r, pick] = 0.9 + 0.09 * torch.rand(boost, generator=g) + 1e-3
        confidence = torch.where(masked, conf, torch.full_like(conf, -torch.inf))
        transfer = HFModel._select_transfer_index(None, confidence, 0.9, count)
        cases.append((block, count))
        i = len(cases) - 1
        rec[f"q{i}_conf"] = conf
        rec[f"q{i}_masked"] = masked
        rec[f"q{i}_count"] = np.array(count)
        rec[f"q{i}_transfer"] = transfer
    rec["num_cases"] = np.array(len(cases))
    rec["threshold"] = np.array(0.9)
    save("hf_twin.npz", **rec)


# ---------------------------------------------------------------- 7. attribute sets of the boundary's objects
def gen_api_surface():
    """What a caller that uses the reference's own classes hands to ``ModelRunner``: the attribute names of
    ``Sequence``, ``SamplingParams`` and ``Config`` (nanovllm/engine/sequence.py:19-60,
    nanovllm/sampling_params.py:4-15, nanovllm/config.py:33-60) with the defaults of the dataclasses."""
    import dataclasses
    import json
    from nanovllm.config import Config as RefConfig
    sp = SamplingParams()
    seq = Sequence([1, 2, 3], sp, denoising_block_size=32, mask_token_id=151669)
    out = {
        "sequence_attributes": sorted(vars(seq)),
        "sequence_class_attributes": sorted(k for k, v in vars(Sequence).items()
                                            if not k.startswith("__") and not callable(v) and not isinstance(v, property)),
        "sequence_properties": sorted(k for k, v in vars(Sequence).items() if isinstance(v, property)),
        "sequence_methods": sorted(k for k, v in vars(Sequence).items() if callable(v)),
        "sampling_params": {f.name: (None if f.default is dataclasses.MISSING else f.default)
                            for f in dataclasses.fields(SamplingParams)},
        "config": {f.name: (None if f.default is dataclasses.MISSING else f.default)
                   for f in dataclasses.fields(RefConfig)},
    }
    path = os.path.join(HERE, "api_surface.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print(f"api_surface.json: {os.path.getsize(path)} B")


GENERATORS = {"index_contract": gen_index_contract, "layers": gen_layers, "staircase": gen_staircase,
              "sampler": gen_sampler, "decoder": gen_decoder, "hf_twin": gen_hf_twin, "api_surface": gen_api_surface}

if __name__ == "__main__":
    # optional further arguments name the fixtures to (re)write; default: all
    for name in (sys.argv[2:] or list(GENERATORS)):
        GENERATORS[name]()
