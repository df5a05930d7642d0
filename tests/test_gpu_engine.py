"""The whole decode path through the ModelRunner boundary: CUDA runner vs the
CPU oracle runner and vs the reference-module fixture, teacher-forced."""
import copy

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, load_golden
from oracle import nano_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _tiny_cfg(mdb, vocab=512, layers=2, hkv=2):
    return mdb.DecoderConfig(vocab_size=vocab, hidden_size=256, intermediate_size=512, num_hidden_layers=layers,
                             num_attention_heads=4, num_key_value_heads=hkv, head_dim=128,
                             max_position_embeddings=2048)


def _oracle_cfg(c):
    return orc.DecoderConfig(vocab_size=c.vocab_size, hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
                             num_hidden_layers=c.num_hidden_layers, num_attention_heads=c.num_attention_heads,
                             num_key_value_heads=c.num_key_value_heads, head_dim=c.head_dim,
                             max_position_embeddings=c.max_position_embeddings)


def _make_runner(mdb, dcfg, weights, pages, eager, noise="explicit", max_seqs=4, max_len=1024, fused=False):
    cfg = mdb.Config(max_num_batched_tokens=2048, max_num_seqs=max_seqs, max_model_len=max_len, enforce_eager=eager,
                     num_kvcache_blocks=pages, decoder_config=dcfg, mask_token_id=500)
    w = mdb.DecoderWeights.from_reference_layout(weights, DEV)
    return cfg, mdb.ModelRunner(cfg, weights=w, noise=noise, fused_step=fused)


def test_runner_matches_reference_fixture(mdb):
    """Same scenario as the fixture recorded from the reference's modules:
    prefill of two prompts, then decode steps, shared weights / pages / noise."""
    g = load_golden("decoder_tiny.npz")
    dcfg = _tiny_cfg(mdb)
    weights = orc.make_weights(_oracle_cfg(dcfg), seed=21)
    cfg, runner = _make_runner(mdb, dcfg, weights, pages=6, eager=True)
    runner.keep_last = True
    noise = {s: torch.from_numpy(g[f"s{s}_gumbel"]) for s in range(int(g["num_steps"]))}
    runner.noise_fn = lambda step, m, v: noise[step].reshape(m, v).contiguous().to(DEV)
    mask_id = int(g["mask_id"])
    seqs = []
    for i in range(2):
        sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=64, ignore_eos=True, dynamic_threshold=0.9)
        seqs.append(mdb.Sequence(g[f"prompt{i}"].tolist(), sp, denoising_block_size=32, mask_token_id=mask_id))
    for step in range(int(g["num_steps"])):
        p = f"s{step}_"
        for seq, row in zip(seqs, g[p + "block_tables"]):
            seq.block_table = [int(t) for t in row if t >= 0]
        n = runner.run(seqs, bool(g[p + "is_prefill"]))
        assert torch.equal(runner.last["x0"].cpu().long().view(2, 32), torch.from_numpy(g[p + "x0"]))
        assert torch.allclose(runner.last["conf"].cpu().view(2, 32), torch.from_numpy(g[p + "x0_p"]), rtol=3e-2)
        assert n == int(g[p + "count"])
        blocks = torch.stack([s.current_denoising_block for s in seqs])
        assert torch.equal(blocks, torch.from_numpy(g[p + "blocks_after"]))
        kv = runner.kv_cache
        sums = [float(kv[0].float().abs().sum()), float(kv[1].float().abs().sum())]
        assert np.allclose(sums, g[p + "kv_abs_sum"], rtol=2e-3)
    assert mdb._lib.device_status(clear=True) == 0


def _clone_seq(mdb, seq):
    c = copy.copy(seq)
    c.token_ids = list(seq.token_ids)
    c.block_table = list(seq.block_table)
    c.current_denoising_block = seq.current_denoising_block.clone()
    c.current_step_map = seq.current_step_map.clone()
    c.step_map = list(seq.step_map)
    return c


LOGIT_TOL = 2e-2      # max-abs logits tolerance of the path (bf16, fp32 accumulate)
E2E_LOGIT_TOL = 5e-2  # end-to-end bound checked below: three bf16 layers of a 256-wide model amplify the
                      # per-op rounding differences; the reference's own two code paths (prefill vs decode form)
                      # differ by 0.03 .. 0.09 over 4 .. 28 layers


def _robust_requests(last, noise, blocks_before, mask_id, thr, temps, tol=LOGIT_TOL):
    """Which requests' decisions this step cannot be flipped by moving every
    logit by up to LOGIT_TOL: the sampled token's noisy margin, the ranking of
    confidences (top-1 rule) and the distance of confidences to the threshold
    all exceed what such a move can change (2*LOGIT_TOL/T in log space); under
    the top-1 rule the sampled token of every masked position must be clear of
    a tie, since the confidence ranked is that of the sampled token."""
    lf = last["logits"].float() / temps[:, None, None]
    top2 = (lf + noise).topk(2, dim=-1).values
    token_margin = top2[..., 0] - top2[..., 1]
    logc = last["x0_p"].clamp_min(1e-30).log()
    eps = 2 * tol / temps
    masked = blocks_before == mask_id
    out = []
    for r in range(masked.shape[0]):
        if not bool(masked[r].any()):
            out.append(True)
            continue
        near_thr = masked[r] & ((logc[r] - float(np.log(thr))).abs() <= eps[r])
        hi = masked[r] & (last["x0_p"][r] > thr)
        if bool(hi.any()):
            ok = not bool(near_thr.any()) and bool((token_margin[r][hi] > eps[r]).all())
        else:
            c = logc[r].masked_fill(~masked[r], -float("inf"))
            best = c.topk(min(2, int(masked[r].sum())))
            gap = float(best.values[0] - best.values[1]) if best.values.numel() > 1 else float("inf")
            # a token tie at any masked position swaps in a token of another confidence and can reorder the ranking
            ok = gap > float(eps[r]) and not bool(near_thr.any()) and bool((token_margin[r][masked[r]] > eps[r]).all())
        out.append(ok)
    return out


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("temperature", [1.0, 0.05])
def test_teacher_forced_agreement(mdb, eager, temperature):
    """The oracle drives generation (its decisions are applied); at every step
    the CUDA runner is given the same request state and must commit the same
    tokens at the same positions.  Random-init weights give nearly flat
    distributions, so some decisions are ties within the logits tolerance of
    the path: agreement is asserted over the decisions that such a tolerance
    cannot flip (>= 99.5 %) and reported over all of them.  The lower
    temperature sharpens the distributions so that confidences cross the
    threshold and several tokens commit per step."""
    dcfg = _tiny_cfg(mdb, vocab=1024, layers=3)
    ocfg = _oracle_cfg(dcfg)
    weights = orc.make_weights(ocfg, seed=5)
    pages = 8
    cfg, runner = _make_runner(mdb, dcfg, weights, pages=pages, eager=eager, noise="gumbel" if not eager else "explicit")
    gen = torch.Generator().manual_seed(77)
    noise_store = {}

    def oracle_noise(step, shape):
        m = shape[0] * shape[1]
        if eager:
            z = -torch.empty(shape).exponential_(generator=gen).log()
        else:   # graphs use the counter-based generator: fetch exactly what the kernel will add
            z = mdb.ops.gumbel_noise(m, shape[2], runner.noise_seed, step, DEV).cpu().view(shape)
        noise_store[step] = z
        return z

    runner.noise_fn = lambda step, m, v: noise_store[step].reshape(m, v).contiguous().to(DEV)
    oracle = orc.OracleModelRunner(ocfg, weights, num_pages=pages, block_size=32, mask_token_id=500,
                                   noise_fn=oracle_noise)
    sched = mdb.Scheduler(cfg)
    embeds = {}
    for i, plen in enumerate([150, 40, 260]):
        ids = torch.randint(0, 490, (plen,), generator=gen).tolist()
        sp = mdb.SamplingParams(temperature=temperature, max_new_tokens=64, ignore_eos=True, dynamic_threshold=0.9)
        rows = torch.randn(plen - 8, dcfg.hidden_size, generator=gen).to(torch.bfloat16)   # synthetic visual rows
        seq = mdb.Sequence(ids, sp, denoising_block_size=32, mask_token_id=500, inputs_embeds=rows)
        embeds[seq.seq_id] = rows
        sched.add(seq)
    oracle.prompt_embeds = embeds
    runner.keep_last = True
    raw_total = raw_agree = rob_total = rob_agree = steps = multi = 0
    worst_logit_err = 0.0
    while not sched.is_finished() and steps < 300:
        seqs, is_prefill = sched.schedule()
        twins = [_clone_seq(mdb, s) for s in seqs]
        before = torch.stack([s.current_denoising_block.clone() for s in seqs])
        temps = torch.tensor([s.temperature for s in seqs])
        n_ref = oracle.run(seqs, is_prefill)
        runner.run(twins, is_prefill)
        ref_blocks = torch.stack([s.current_denoising_block for s in seqs])
        got_blocks = torch.stack([s.current_denoising_block for s in twins])
        # logits the CUDA path implies (its final-norm rows through the oracle's LM head) vs the oracle's
        got_logits = orc.linear(runner.last["hidden"].cpu(), weights.lm_head).view_as(oracle.last["logits"])
        step_err = float((got_logits.float() - oracle.last["logits"].float()).abs().max())
        worst_logit_err = max(worst_logit_err, step_err)
        robust = _robust_requests(oracle.last, noise_store[oracle.step_index - 1], before, 500, 0.9, temps,
                                  tol=max(LOGIT_TOL, step_err))
        decided = oracle.last["transfer"] | (got_blocks != ref_blocks)
        same = decided & (got_blocks == ref_blocks)
        for r, ok in enumerate(robust):
            raw_total += int(decided[r].sum())
            raw_agree += int(same[r].sum())
            if ok:
                rob_total += int(decided[r].sum())
                rob_agree += int(same[r].sum())
        multi += int(n_ref > len(seqs))
        sched.postprocess(seqs)
        steps += 1
    assert sched.is_finished()
    print(f"teacher-forced agreement T={temperature} eager={eager}: all decisions {raw_agree}/{raw_total}, "
          f"tolerance-robust decisions {rob_agree}/{rob_total}, steps {steps}, multi-token steps {multi}, "
          f"worst end-to-end logits max-abs {worst_logit_err:.4f}")
    assert worst_logit_err <= E2E_LOGIT_TOL
    assert rob_total > 0 and rob_agree / rob_total >= 0.995, f"committed-token agreement {rob_agree}/{rob_total}"
    if temperature >= 0.5:
        assert rob_total >= 0.2 * raw_total
        assert raw_agree / raw_total >= 0.9
    else:
        # dividing by a small temperature magnifies logit differences 20x, so few decisions stay outside
        # the tolerance band; what matters here is that the threshold branch ran and agreed where it must
        assert multi > 0
    assert mdb._lib.device_status(clear=True) == 0


@pytest.mark.parametrize("block", [8, 16, 64])
@pytest.mark.parametrize("eager", [True, False])
def test_block_size_sweep(mdb, block, eager):
    """The block sizes of the throughput sweep other than 32 (8, 16, 64), teacher-forced
    against the oracle through prefill, denoising passes and block commits: identical block
    states wherever the decision is not a tie within the logits tolerance, end-to-end logits
    within tolerance.  Block 64 with two query heads per KV head runs the 128-row units of
    the attention kernel, and 3 x 64 rows per step the many-row GEMM path."""
    dcfg = _tiny_cfg(mdb, vocab=1024, layers=2)
    ocfg = _oracle_cfg(dcfg)
    weights = orc.make_weights(ocfg, seed=block)
    pages = 8
    cfg = mdb.Config(max_num_batched_tokens=2048, max_num_seqs=4, max_model_len=1024, enforce_eager=eager,
                     num_kvcache_blocks=pages, decoder_config=dcfg, mask_token_id=500, block_size=block)
    runner = mdb.ModelRunner(cfg, weights=mdb.DecoderWeights.from_reference_layout(weights, DEV),
                             noise="explicit" if eager else "gumbel")
    gen = torch.Generator().manual_seed(block)
    noise_store = {}

    def oracle_noise(step, shape):
        m = shape[0] * shape[1]
        if eager:
            z = -torch.empty(shape).exponential_(generator=gen).log()
        else:
            z = mdb.ops.gumbel_noise(m, shape[2], runner.noise_seed, step, DEV).cpu().view(shape)
        noise_store[step] = z
        return z

    runner.noise_fn = lambda step, m, v: noise_store[step].reshape(m, v).contiguous().to(DEV)
    oracle = orc.OracleModelRunner(ocfg, weights, num_pages=pages, block_size=block, mask_token_id=500,
                                   noise_fn=oracle_noise)
    sched = mdb.Scheduler(cfg)
    for plen in (150, 40, 250):
        ids = torch.randint(0, 490, (plen,), generator=gen).tolist()
        sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=2 * block, ignore_eos=True, dynamic_threshold=0.9)
        sched.add(mdb.Sequence(ids, sp, denoising_block_size=block, mask_token_id=500))
    runner.keep_last = True
    rob_total = rob_agree = raw_total = raw_agree = steps = 0
    worst = 0.0
    while not sched.is_finished() and steps < 200:
        seqs, is_prefill = sched.schedule()
        twins = [_clone_seq(mdb, s) for s in seqs]
        before = torch.stack([s.current_denoising_block.clone() for s in seqs])
        temps = torch.tensor([s.temperature for s in seqs])
        oracle.run(seqs, is_prefill)
        runner.run(twins, is_prefill)
        ref_blocks = torch.stack([s.current_denoising_block for s in seqs])
        got_blocks = torch.stack([s.current_denoising_block for s in twins])
        got_logits = orc.linear(runner.last["hidden"].cpu(), weights.lm_head).view_as(oracle.last["logits"])
        step_err = float((got_logits.float() - oracle.last["logits"].float()).abs().max())
        worst = max(worst, step_err)
        robust = _robust_requests(oracle.last, noise_store[oracle.step_index - 1], before, 500, 0.9, temps,
                                  tol=max(LOGIT_TOL, step_err))
        decided = oracle.last["transfer"] | (got_blocks != ref_blocks)
        same = decided & (got_blocks == ref_blocks)
        for r, ok in enumerate(robust):
            raw_total += int(decided[r].sum())
            raw_agree += int(same[r].sum())
            if ok:
                rob_total += int(decided[r].sum())
                rob_agree += int(same[r].sum())
        sched.postprocess(seqs)
        steps += 1
    assert sched.is_finished()
    print(f"block {block} eager={eager}: decisions {raw_agree}/{raw_total}, tolerance-robust {rob_agree}/{rob_total}, "
          f"steps {steps}, worst logits max-abs {worst:.4f}")
    assert worst <= E2E_LOGIT_TOL
    assert rob_total > 0 and rob_agree / rob_total >= 0.995
    assert raw_agree / raw_total >= 0.9
    assert mdb._lib.device_status(clear=True) == 0


@pytest.mark.parametrize("eager", [True, False])
def test_one_kernel_step_matches_separate_kernels(mdb, eager):
    """The persistent one-kernel decode step against the chain of separate
    kernels: same requests, same counter-based noise, teacher-forced.  The two
    run the same arithmetic (only the RMSNorm row sum is ordered differently),
    so sampled tokens must agree and hidden rows stay within a few bf16 steps."""
    dcfg = _tiny_cfg(mdb, vocab=1024, layers=3)
    weights = orc.make_weights(_oracle_cfg(dcfg), seed=5)
    cfg_a, ra = _make_runner(mdb, dcfg, weights, pages=8, eager=eager, noise="gumbel", fused=True)
    cfg_b, rb = _make_runner(mdb, dcfg, weights, pages=8, eager=eager, noise="gumbel", fused=False)
    ra.keep_last = rb.keep_last = True
    gen = torch.Generator().manual_seed(3)
    sched = mdb.Scheduler(cfg_a)
    for plen in (150, 40, 260):
        sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=64, ignore_eos=True)
        sched.add(mdb.Sequence(torch.randint(0, 490, (plen,), generator=gen).tolist(), sp, denoising_block_size=32,
                               mask_token_id=500))
    steps = agree = total = 0
    worst = 0.0
    while not sched.is_finished() and steps < 300:
        seqs, is_prefill = sched.schedule()
        twins = [_clone_seq(mdb, s) for s in seqs]
        ra.run(seqs, is_prefill)
        rb.run(twins, is_prefill)
        same = ra.last["x0"] == rb.last["x0"]
        agree += int(same.sum())
        total += same.numel()
        worst = max(worst, float((ra.last["hidden"].float() - rb.last["hidden"].float()).abs().max()))
        assert torch.allclose(ra.last["conf"][same], rb.last["conf"][same], rtol=5e-2)
        sched.postprocess(seqs)
        steps += 1
    assert sched.is_finished()
    print(f"one-kernel step vs separate kernels (eager={eager}): sampled tokens {agree}/{total}, "
          f"hidden max-abs {worst:.4f}, steps {steps}")
    assert agree / total >= 0.99 and worst <= 0.05
    assert mdb._lib.device_status(clear=True) == 0


def test_engine_generates_and_frees_pages(mdb):
    """Full loop through LLMEngine with graphs: every request reaches its
    length, pages return to the pool, outputs contain no mask token."""
    dcfg = _tiny_cfg(mdb, vocab=1024, layers=2, hkv=2)
    weights = orc.make_weights(_oracle_cfg(dcfg), seed=9)
    cfg, runner = _make_runner(mdb, dcfg, weights, pages=10, eager=False, noise="gumbel", max_seqs=4)
    engine = mdb.LLMEngine(cfg, runner)
    gen = torch.Generator().manual_seed(3)
    seqs = []
    for plen, new in [(100, 64), (300, 96), (31, 32), (257, 64), (64, 64)]:
        sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=new, ignore_eos=True)
        seqs.append(mdb.Sequence(torch.randint(0, 490, (plen,), generator=gen).tolist(), sp, denoising_block_size=32,
                                 mask_token_id=500))
    done, _ = engine.generate(seqs)
    assert len(done) == 5
    for seq, (plen, new) in zip(seqs, [(100, 64), (300, 96), (31, 32), (257, 64), (64, 64)]):
        toks, step_map = done[seq.seq_id]
        assert len(toks) == new and 500 not in toks and len(step_map) == new
    assert len(engine.scheduler.block_manager.free_block_ids) == 10
    assert mdb._lib.device_status(clear=True) == 0


@pytest.mark.parametrize("eager", [True, False])
def test_fused_commit_pass(mdb, eager):
    """Config.fuse_commit_pass: the pass that writes a finished block's K/V also runs the first denoising pass of
    the next block.  One request, no sampling noise, low temperature (several tokens per step): the rows of a
    request do not depend on how many other rows share the step, so the tokens must be the same as with the
    reference's schedule, in fewer steps.  Several requests: everything completes and pages come back."""
    dcfg = _tiny_cfg(mdb, vocab=1024, layers=2, hkv=2)
    weights = orc.make_weights(_oracle_cfg(dcfg), seed=11)
    gen = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, 490, (120,), generator=gen).tolist()
    results = {}
    for fuse in (False, True):
        cfg = mdb.Config(max_num_batched_tokens=2048, max_num_seqs=1, max_model_len=1024, enforce_eager=eager,
                         num_kvcache_blocks=4, decoder_config=dcfg, mask_token_id=500, fuse_commit_pass=fuse)
        runner = mdb.ModelRunner(cfg, weights=mdb.DecoderWeights.from_reference_layout(weights, DEV), noise="none")
        engine = mdb.LLMEngine(cfg, runner)
        sp = mdb.SamplingParams(temperature=0.02, max_new_tokens=256, ignore_eos=True, dynamic_threshold=0.9)
        seq = mdb.Sequence(list(prompt), sp, denoising_block_size=32, mask_token_id=500)
        done, _ = engine.generate([seq])
        results[fuse] = (done[seq.seq_id][0], engine.num_decode_steps)
        assert len(engine.scheduler.block_manager.free_block_ids) == 4
        runner.exit()
    (plain_tokens, plain_steps), (fused_tokens, fused_steps) = results[False], results[True]
    assert len(plain_tokens) == 256 and 500 not in plain_tokens
    assert fused_tokens == plain_tokens
    # 8 blocks; the commit pass of every block but the last and the page-crossing ones rides with the next block
    assert fused_steps <= plain_steps - 5, (plain_steps, fused_steps)
    print(f"fused commit pass (eager={eager}): {plain_steps} -> {fused_steps} decode steps for 256 tokens")

    cfg = mdb.Config(max_num_batched_tokens=2048, max_num_seqs=3, max_model_len=1024, enforce_eager=eager,
                     num_kvcache_blocks=8, decoder_config=dcfg, mask_token_id=500, fuse_commit_pass=True)
    runner = mdb.ModelRunner(cfg, weights=mdb.DecoderWeights.from_reference_layout(weights, DEV), noise="gumbel")
    engine = mdb.LLMEngine(cfg, runner)
    seqs = []
    for plen, new in [(100, 96), (300, 64), (31, 128), (200, 64)]:
        sp = mdb.SamplingParams(temperature=0.05, max_new_tokens=new, ignore_eos=True)
        seqs.append(mdb.Sequence(torch.randint(0, 490, (plen,), generator=gen).tolist(), sp, denoising_block_size=32,
                                 mask_token_id=500))
    done, _ = engine.generate(seqs)
    for seq, new in zip(seqs, (96, 64, 128, 64)):
        toks, step_map = done[seq.seq_id]
        assert len(toks) == new and 500 not in toks and len(step_map) == new
    assert len(engine.scheduler.block_manager.free_block_ids) == 8
    assert mdb._lib.device_status(clear=True) == 0


def test_reused_step_inputs_change_nothing(mdb):
    """While the same requests stay on the same blocks the runner rewrites only the token ids of the pinned step
    inputs (taken from the previous step's result copy).  Forcing the full rebuild every step must give the same
    tokens and step maps."""
    dcfg = _tiny_cfg(mdb, vocab=1024, layers=2, hkv=2)
    weights = orc.make_weights(_oracle_cfg(dcfg), seed=13)
    outs = []
    for force_rebuild in (False, True):
        cfg, runner = _make_runner(mdb, dcfg, weights, pages=10, eager=False, noise="gumbel", max_seqs=4)
        if force_rebuild:
            plain = runner.prepare_decode

            def rebuild(seqs, copy=True, _plain=plain, _runner=runner):
                _runner._decode_key, _runner._last_rows = None, None
                return _plain(seqs, copy)

            runner.prepare_decode = rebuild
        engine = mdb.LLMEngine(cfg, runner)
        gen = torch.Generator().manual_seed(5)
        seqs = []
        for plen, new in [(100, 64), (300, 96), (31, 32), (250, 64), (64, 64)]:
            sp = mdb.SamplingParams(temperature=0.05, max_new_tokens=new, ignore_eos=True)
            seqs.append(mdb.Sequence(torch.randint(0, 490, (plen,), generator=gen).tolist(), sp,
                                     denoising_block_size=32, mask_token_id=500))
        done, _ = engine.generate(seqs)
        outs.append([done[s.seq_id] for s in seqs])
        runner.exit()
    for (tok_a, map_a), (tok_b, map_b) in zip(*outs):
        assert tok_a == tok_b and map_a == map_b
    assert mdb._lib.device_status(clear=True) == 0
