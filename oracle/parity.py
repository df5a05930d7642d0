"""Teacher-forced comparison of the CUDA model runner with the CPU oracle (TEST INFRASTRUCTURE).

Checker harness, never the product: only the test-suite, the smoke entry and
the benchmark's CPU leg may import it.  It drives ``OracleModelRunner`` (the
restatement of ``engines/nano_dvlm/nanovllm/engine/model_runner.py:127-219`` and
``nanovllm/layers/sampler.py:24-61``) and the package's ``ModelRunner`` through
the same denoising passes of one request, from identical weights, identical
cache bytes and identical Gumbel noise.  The oracle's decisions are the ones
applied (teacher forcing), so every pass compares the two paths on the same
request state.

A prefix of ``context`` tokens is not prefilled on the CPU (a 28-layer prefill
of a thousand rows takes minutes there): both caches are seeded with the same
N(0, 1) bf16 rows instead, which is all a decode-form pass reads of the prefix.
"""
from __future__ import annotations

import math
import time

import torch

from . import nano_oracle as orc

LOGIT_TOL = 2e-2      # max-abs logits tolerance of the path (bf16 operands, fp32 accumulation)


def _robust(last, noise, before, mask_id: int, thr: float, temp: float, tol: float) -> bool:
    """True when no move of every logit by up to ``tol`` can change this pass's decision for the request:
    the sampled token's noisy margin at every position that matters, the ranking of the confidences under
    the top-1 rule and the distance of the confidences to the threshold all exceed 2 * tol / T."""
    lf = last["logits"][0].float() / temp
    top2 = (lf + noise[0]).topk(2, dim=-1).values
    margin = top2[:, 0] - top2[:, 1]
    logc = last["x0_p"][0].clamp_min(1e-30).log()
    eps = 2 * tol / temp
    masked = before == mask_id
    if not bool(masked.any()):
        return True
    near_thr = masked & ((logc - math.log(thr)).abs() <= eps)
    hi = masked & (last["x0_p"][0] > thr)
    if bool(hi.any()):
        return not bool(near_thr.any()) and bool((margin[hi] > eps).all())
    c = logc.masked_fill(~masked, -float("inf"))
    best = c.topk(min(2, int(masked.sum())))
    gap = float(best.values[0] - best.values[1]) if best.values.numel() > 1 else float("inf")
    return gap > eps and not bool(near_thr.any()) and bool((margin[masked] > eps).all())


def decode_parity(pkg, ocfg: "orc.DecoderConfig", weights: "orc.DecoderWeights", *, context: int, passes: int,
                  temperature: float, threshold: float = 0.9, seed: int = 7, device: str = "cuda:0",
                  eager: bool = False, mask_id: int | None = None, block: int = 32, native_linear: bool = False,
                  gpu_weights=None) -> dict:
    """Runs ``passes`` decode-form passes (denoising passes and the commit pass that ends a block) of one
    request whose committed prefix is ``context`` tokens long.  Returns the comparison figures:

    * ``decisions`` / ``decisions_agree``: positions that changed in either path, and how many of them hold
      the same token in both; ``robust_*``: the same over the passes whose decision a logits move of
      ``LOGIT_TOL`` cannot flip (fixed tolerance, not widened by the measured error); ``floor_robust_*``: the
      same with the oracle's own floor (below) as the tolerance where that is larger -- decisions that two
      equally valid implementations of the reference's arithmetic could already flip are left out, whatever
      the CUDA path's own error is;
    * ``x0_agree`` / ``x0_total``: sampled tokens over all rows of all passes;
    * ``logits_fp32_max_abs``: worst |CUDA - oracle| over the un-rounded fp32 logits implied by the two
      final-norm hidden states (both through the oracle's LM head); ``logits_bf16_max_abs``: the same after
      the reference's rounding of the logits to bf16 (one bf16 step at |logit| >= 4 is 0.031);
    * ``oracle_floor_logits_fp32_max_abs``: the same figure between the oracle and itself with the one rounding
      inside its attention left out (probabilities kept in fp32 instead of rounded to bf16 before PV, which
      flash-attn does per key tile against a running maximum and no restatement can place identically), on the
      first pass: what two equally valid implementations of the reference's arithmetic differ by at this depth
      and width;
    * ``conf_max_rel``: worst relative difference of the confidences where the sampled tokens agree;
    * ``kv_rows``: committed K/V rows compared after each commit pass, ``kv_max_abs`` their worst difference,
      ``kv_exact_frac`` the share of identical bf16 values;
    * ``disagreements``: one record per differing decision with the oracle's noisy top-2 margin at that
      position and its confidence gap, next to the logits error of that pass (a tie within the error of the
      path explains the difference); ``disagreements_unexplained`` counts those whose deciding margin is not
      below twice that error over the temperature.
    """
    if native_linear:
        orc.use_native_linear(True)
    try:
        return _decode_parity(pkg, ocfg, weights, context, passes, temperature, threshold, seed, device, eager,
                              mask_id, block, gpu_weights)
    finally:
        if native_linear:
            orc.use_native_linear(False)


def _decode_parity(pkg, ocfg, weights, context, passes, temperature, threshold, seed, device, eager, mask_id, block,
                   gpu_weights):
    t_start = time.perf_counter()
    vocab = ocfg.vocab_size
    if mask_id is None:
        mask_id = 151669 if vocab > 151669 else vocab - 12
    dcfg = pkg.DecoderConfig(vocab_size=ocfg.vocab_size, hidden_size=ocfg.hidden_size,
                             intermediate_size=ocfg.intermediate_size, num_hidden_layers=ocfg.num_hidden_layers,
                             num_attention_heads=ocfg.num_attention_heads, num_key_value_heads=ocfg.num_key_value_heads,
                             head_dim=ocfg.head_dim, rms_norm_eps=ocfg.rms_norm_eps, rope_theta=ocfg.rope_theta,
                             max_position_embeddings=ocfg.max_position_embeddings)
    total = context + (passes // 2 + 2) * block
    pages = (total + orc.PAGE - 1) // orc.PAGE
    max_len = pages * orc.PAGE
    cfg = pkg.Config(max_num_batched_tokens=max(max_len, 2048), max_num_seqs=1, max_model_len=max_len,
                     enforce_eager=eager, num_kvcache_blocks=pages, decoder_config=dcfg, mask_token_id=mask_id,
                     block_size=block)
    if gpu_weights is None:
        gpu_weights = pkg.DecoderWeights.from_reference_layout(weights, device)
    runner = pkg.ModelRunner(cfg, weights=gpu_weights, noise="gumbel", noise_seed=seed, device=device)
    runner.keep_last = True

    noise_store = {}

    def oracle_noise(step, shape):
        # exactly what the counter-based generator of the LM-head epilogue adds at this step
        z = pkg.ops.gumbel_noise(shape[0] * shape[1], shape[2], seed, step, device).cpu().view(shape)
        noise_store[step] = z
        return z

    oracle = orc.OracleModelRunner(ocfg, weights, num_pages=pages, block_size=block, mask_token_id=mask_id,
                                   noise_fn=oracle_noise)
    g = torch.Generator().manual_seed(seed)
    oracle.decoder.kv_cache.copy_(torch.randn(oracle.decoder.kv_cache.shape, generator=g).to(torch.bfloat16))
    runner.kv_cache.copy_(oracle.decoder.kv_cache)

    def make():
        sp = pkg.SamplingParams(temperature=temperature, max_new_tokens=total - context, ignore_eos=True,
                                dynamic_threshold=threshold)
        s = pkg.Sequence([1] * context, sp, denoising_block_size=block, mask_token_id=mask_id)
        s.block_table = list(range(pages))
        s.status = pkg.SequenceStatus.RUNNING
        return s

    ref_seq, got_seq = make(), make()
    # the yardstick: the oracle against itself with its attention's probability rounding left out, first pass
    twin = orc.OracleModelRunner(ocfg, weights, num_pages=pages, block_size=block, mask_token_id=mask_id, noise_fn=None)
    twin.decoder.kv_cache.copy_(oracle.decoder.kv_cache)
    twin.decoder.round_p = False
    twin.run([make()], False)
    twin_hidden = twin.last["hidden"].reshape(block, -1).float()
    del twin
    lm_w32 = weights.lm_head.float()
    out = dict(decisions=0, decisions_agree=0, robust_decisions=0, robust_agree=0, floor_robust_decisions=0,
               floor_robust_agree=0, x0_total=0, x0_agree=0,
               logits_fp32_max_abs=0.0, logits_bf16_max_abs=0.0, conf_max_rel=0.0, kv_rows=0, kv_max_abs=0.0,
               kv_exact_frac=1.0, passes=0, commit_passes=0, multi_token_passes=0, disagreements=[],
               oracle_floor_logits_fp32_max_abs=None)
    for _ in range(passes):
        before = ref_seq.current_denoising_block.clone()
        is_commit = not bool((before == mask_id).any())
        n_ref = oracle.run([ref_seq], False)
        runner.run([got_seq], False)
        last = oracle.last
        step = oracle.step_index - 1
        ref_block, got_block = ref_seq.current_denoising_block, got_seq.current_denoising_block
        # logits implied by the two hidden states, before and after the reference's rounding point
        h_ref = last["hidden"].reshape(block, -1).float()
        h_got = runner.last["hidden"].cpu().float()
        lf_ref, lf_got = h_ref @ lm_w32.t(), h_got @ lm_w32.t()
        if out["oracle_floor_logits_fp32_max_abs"] is None:
            out["oracle_floor_logits_fp32_max_abs"] = round(float((lf_ref - twin_hidden @ lm_w32.t()).abs().max()), 6)
        err = float((lf_ref - lf_got).abs().max())
        out["logits_fp32_max_abs"] = max(out["logits_fp32_max_abs"], err)
        out["logits_bf16_max_abs"] = max(out["logits_bf16_max_abs"],
                                         float((lf_ref.to(torch.bfloat16).float() - lf_got.to(torch.bfloat16).float()).abs().max()))
        if not is_commit:
            x0_ref = last["x0"].view(-1)
            x0_got = runner.last["x0"].cpu().long()
            same = x0_ref == x0_got
            out["x0_total"] += block
            out["x0_agree"] += int(same.sum())
            if bool(same.any()):
                p_ref, p_got = last["x0_p"].view(-1)[same], runner.last["conf"].cpu()[same]
                out["conf_max_rel"] = max(out["conf_max_rel"], float(((p_got - p_ref).abs() / p_ref.clamp_min(1e-30)).max()))
            decided = last["transfer"][0] | (got_block != ref_block)
            agree = decided & (got_block == ref_block)
            out["decisions"] += int(decided.sum())
            out["decisions_agree"] += int(agree.sum())
            if _robust(last, noise_store[step], before, mask_id, threshold, temperature, LOGIT_TOL):
                out["robust_decisions"] += int(decided.sum())
                out["robust_agree"] += int(agree.sum())
            if _robust(last, noise_store[step], before, mask_id, threshold, temperature,
                       max(LOGIT_TOL, out["oracle_floor_logits_fp32_max_abs"])):
                out["floor_robust_decisions"] += int(decided.sum())
                out["floor_robust_agree"] += int(agree.sum())
            out["multi_token_passes"] += int(n_ref > 1)
            if bool((decided & ~agree).any()):
                lf = last["logits"][0].float() / temperature
                top2 = (lf + noise_store[step][0]).topk(2, dim=-1).values
                logc = last["x0_p"][0].clamp_min(1e-30).log().masked_fill(before != mask_id, -float("inf"))
                best = logc.topk(min(2, int((before == mask_id).sum()))).values
                for pos in (decided & ~agree).nonzero().flatten().tolist():
                    out["disagreements"].append(dict(
                        step=step, position=pos, ref_token=int(ref_block[pos]), got_token=int(got_block[pos]),
                        noisy_top2_margin=round(float(top2[pos, 0] - top2[pos, 1]), 5),
                        confidence_log_gap=round(float(best[0] - best[1]), 5) if best.numel() > 1 else None,
                        pass_logits_err=round(err, 5), temperature=temperature))
        else:
            out["commit_passes"] += 1
            # the block's final K/V rows as both paths cached them, every layer
            lo = len(ref_seq)
            slots = torch.tensor(orc.get_slots(ref_seq.block_table, lo, lo + block))
            layers, hkv, d = ocfg.num_hidden_layers, ocfg.num_key_value_heads, ocfg.head_dim
            kv_ref = oracle.decoder.kv_cache.view(2, layers, -1, hkv * d)[:, :, slots]
            kv_got = runner.kv_cache.view(2, layers, -1, hkv * d)[:, :, slots.to(device)].cpu()
            diff = (kv_ref.float() - kv_got.float()).abs()
            out["kv_rows"] += 2 * layers * block
            out["kv_max_abs"] = max(out["kv_max_abs"], float(diff.max()))
            out["kv_exact_frac"] = min(out["kv_exact_frac"], float((diff == 0).float().mean()))
        out["passes"] += 1
        # teacher forcing: the CUDA side continues from the oracle's state
        got_seq.current_denoising_block = ref_block.clone()
        if is_commit:
            ref_seq.append_block()
            got_seq.append_block()
    status = pkg._lib.device_status(clear=True)
    runner.exit()
    del runner
    torch.cuda.empty_cache()
    out.update(device_status=status, context=context, temperature=temperature, threshold=threshold, block=block,
               layers=ocfg.num_hidden_layers, hidden=ocfg.hidden_size, vocab=vocab, graphs=not eager,
               logit_tol=LOGIT_TOL, seconds=round(time.perf_counter() - t_start, 1))
    for k in ("logits_fp32_max_abs", "logits_bf16_max_abs", "conf_max_rel", "kv_max_abs", "kv_exact_frac"):
        out[k] = round(out[k], 6)
    out["decision_agreement"] = round(out["decisions_agree"] / max(out["decisions"], 1), 5)
    out["robust_agreement"] = round(out["robust_agree"] / max(out["robust_decisions"], 1), 5)
    out["floor_robust_agreement"] = round(out["floor_robust_agree"] / max(out["floor_robust_decisions"], 1), 5)
    # a differing decision is explained when the margin that decided it (sampled token: the two best noisy logits;
    # position: the two best confidences, in log) is below twice the logits error of that pass over T
    unexplained = 0
    for d in out["disagreements"]:
        eps = 2 * max(d["pass_logits_err"], LOGIT_TOL) / temperature
        gap = d["confidence_log_gap"] if d["confidence_log_gap"] is not None else float("inf")
        if not (d["noisy_top2_margin"] <= eps or gap <= eps):
            unexplained += 1
    out["disagreements_unexplained"] = unexplained
    return out
