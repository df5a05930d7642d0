"""Host-side mirror of the reference's scheduler / sequence / page allocator and
the step-input builders, replayed against tensors recorded from the reference
(tests/golden/index_contract.npz).  Integer contracts: bit-exact."""
import itertools

import numpy as np
import pytest
import torch

from conftest import load_golden


def _replay(mdb, g):
    from types import SimpleNamespace
    eng = mdb.engine
    B, MASK = 32, 151669
    cfg = SimpleNamespace(max_num_seqs=4, max_num_batched_tokens=4096, eos=-1, num_kvcache_blocks=12,
                          kvcache_block_size=256)
    sched = mdb.Scheduler(cfg)
    mdb.Sequence.counter = itertools.count()
    gen = torch.Generator().manual_seed(11)
    for pl, mn in zip(g["prompt_lens"].tolist(), g["max_new"].tolist()):
        ids = torch.randint(0, 150000, (pl,), generator=gen).tolist()
        sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=mn, ignore_eos=True, stop_token_ids=[])
        sched.add(mdb.Sequence(ids, sp, denoising_block_size=B, mask_token_id=MASK))
    from importlib import import_module
    si = import_module("mineru-diffusion_b200.engine.step_inputs")
    nsteps = int(g["num_steps"])
    kinds = set()
    for step in range(nsteps):
        p = f"s{step:03d}_"
        seqs, is_prefill = sched.schedule()
        assert int(is_prefill) == int(g[p + "is_prefill"]), step
        assert [s.seq_id for s in seqs] == g[p + "seq_ids"].tolist()
        if is_prefill:
            inp = si.build_prefill_inputs(seqs, B)
            assert np.array_equal(inp["input_ids"], g[p + "input_ids"])
            assert np.array_equal(inp["positions"], g[p + "positions"])
            assert np.array_equal(inp["slot_mapping"], g[p + "slot_mapping"])
            assert np.array_equal(inp["cu_seqlens"], g[p + "cu_seqlens_q"])
            assert np.array_equal(inp["cu_seqlens"], g[p + "cu_seqlens_k"])
        else:
            inp = si.build_decode_inputs(seqs, B)
            for ours, theirs in (("input_ids", "input_ids"), ("positions", "positions"),
                                 ("slot_mapping", "slot_mapping"), ("context_lens", "context_lens"),
                                 ("block_tables", "block_tables")):
                assert np.array_equal(inp[ours], g[p + theirs]), (step, ours)
                assert inp[ours].dtype == g[p + theirs].dtype
            if (inp["slot_mapping"][:, 0] // 256 != inp["slot_mapping"][:, -1] // 256).any():
                kinds.add("straddle")
        # apply the recorded sampler outcome, then the scheduler's own post-processing
        for s, row in zip(seqs, g[p + "blocks_after"]):
            s.current_denoising_block = torch.from_numpy(row.copy())
        sched.postprocess(seqs)
        assert [s.status.value for s in seqs] == g[p + "status_after"].tolist()
        assert [s.num_tokens for s in seqs] == g[p + "num_tokens_after"].tolist()
    assert sched.is_finished()
    assert len(sched.block_manager.free_block_ids) == 12
    return kinds


def test_scheduler_and_step_inputs_match_reference(mdb):
    g = load_golden("index_contract.npz")
    kinds = _replay(mdb, g)
    assert "straddle" in kinds      # a block that crosses a page boundary was exercised


def test_get_slots_cases(mdb):
    g = load_golden("index_contract.npz")
    seq = mdb.Sequence(list(range(700)), mdb.SamplingParams(), denoising_block_size=32, mask_token_id=1)
    seq.block_table = g["slots_table"].tolist()
    for i, (lo, hi) in enumerate(g["slots_cases"].tolist()):
        assert seq.get_slots(lo, hi) == g[f"slots_{i}"].tolist()
    seq.block_table = []
    assert seq.get_slots(5, 9) == [-1] * 4


def test_decode_inputs_match_per_request_form(mdb):
    """The vectorised decode-step builder against the per-request statement of the same contract
    (NV/engine/model_runner.py:169-185): ids, positions, slots through get_slots, context lengths,
    for ragged lengths around page edges, several block sizes and a request that holds no page."""
    import numpy as np
    import torch
    si = mdb.engine.step_inputs if hasattr(mdb, "engine") else __import__("importlib").import_module(
        "mineru-diffusion_b200.engine.step_inputs")
    gen = torch.Generator().manual_seed(0)
    for block in (8, 32, 64):
        seqs = []
        for n in (1, 255, 256, 257, 511, 700, 1024 - block, 3000):
            sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=64, ignore_eos=True)
            seq = mdb.Sequence(torch.randint(0, 100, (n,), generator=gen).tolist(), sp, denoising_block_size=block,
                               mask_token_id=1000)
            pages = (n + block + 255) // 256
            seq.block_table = torch.randperm(64, generator=gen)[:pages].tolist()
            seqs.append(seq)
        seqs[3].block_table = []          # a warm-up style request: no pages, every slot -1
        got = si.build_decode_inputs(seqs, block)
        for i, seq in enumerate(seqs):
            n = len(seq)
            assert np.array_equal(got["input_ids"][i], seq.current_denoising_block.numpy())
            assert np.array_equal(got["positions"][i], np.arange(n, n + block))
            assert np.array_equal(got["slot_mapping"][i], np.asarray(seq.get_slots(n, n + block), dtype=np.int32))
            assert got["context_lens"][i] == n + block
        assert got["slot_mapping"].dtype == np.int32 and got["positions"].dtype == np.int64


def test_preemption_when_pages_run_out(mdb):
    from types import SimpleNamespace
    cfg = SimpleNamespace(max_num_seqs=4, max_num_batched_tokens=4096, eos=-1, num_kvcache_blocks=2,
                          kvcache_block_size=256)
    sched = mdb.Scheduler(cfg)
    a = mdb.Sequence([1] * 250, mdb.SamplingParams(max_new_tokens=64), denoising_block_size=32, mask_token_id=9)
    b = mdb.Sequence([1] * 250, mdb.SamplingParams(max_new_tokens=64), denoising_block_size=32, mask_token_id=9)
    sched.add(a)
    sched.add(b)
    seqs, is_prefill = sched.schedule()
    assert is_prefill and seqs == [a, b]
    # both need a second page for the block that spills over; only the first can be served
    seqs, is_prefill = sched.schedule()
    assert not is_prefill and seqs == [a]
    assert b.status is mdb.SequenceStatus.WAITING and not b.block_table
    assert len(a.block_table) == 2


def test_sampling_params_and_config_validation(mdb):
    with pytest.raises(AssertionError):
        mdb.SamplingParams(temperature=0.0)
    with pytest.raises(AssertionError):
        mdb.Config(kvcache_block_size=100)
    with pytest.raises(AssertionError):
        mdb.Config(max_num_batched_tokens=100, max_model_len=4096)
    c = mdb.Config()
    assert c.decoder_config.vocab_size == 151936 and c.block_size == 32 and c.mask_token_id == 151669


def test_model_runner_needs_cuda(mdb):
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    with pytest.raises(RuntimeError):
        mdb.ModelRunner(mdb.Config())


def _running_seqs(mdb, n, block=32, mask=1000):
    from types import SimpleNamespace
    cfg = SimpleNamespace(max_num_seqs=16, max_num_batched_tokens=8192, eos=-1, num_kvcache_blocks=64,
                          kvcache_block_size=256)
    sched = mdb.Scheduler(cfg)
    gen = torch.Generator().manual_seed(3)
    for i in range(n):
        sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=96, ignore_eos=True, stop_token_ids=[])
        sched.add(mdb.Sequence(torch.randint(0, 100, (20 + i,), generator=gen).tolist(), sp,
                               denoising_block_size=block, mask_token_id=mask))
    seqs, is_prefill = sched.schedule()
    assert is_prefill and len(seqs) == n
    for s in seqs:                         # what a prefill step leaves behind
        s.num_cached_tokens = len(s)
    return sched, seqs


def test_postprocess_batch_check_equals_per_request(mdb):
    """Scheduler.postprocess (NV/engine/scheduler.py:65-82) decides RUNNING -> CACHING per request from "any
    mask token left"; batches of more than four requests make that decision with one comparison."""
    for n in (3, 9):
        sched, seqs = _running_seqs(mdb, n)
        for i, s in enumerate(seqs):
            s.current_denoising_block = torch.full((32,), 7, dtype=torch.int64)
            if i % 3 != 0:
                s.current_denoising_block[5 + i] = 1000
        sched.postprocess(seqs)
        for i, s in enumerate(seqs):
            assert s.is_caching == (i % 3 == 0), (n, i)
        # the caching pass of the finished ones: block appended, a fresh masked block opened
        lens = [len(s) for s in seqs]
        sched.postprocess(seqs)
        for i, s in enumerate(seqs):
            if i % 3 == 0:
                assert len(s) == lens[i] + 32 and not s.is_caching
                assert bool((s.current_denoising_block == 1000).all())
            else:
                assert len(s) == lens[i]


def test_pending_first_step_applied_after_append(mdb):
    """Config.fuse_commit_pass: the result of the next block's first denoising pass, left on the request by the
    runner, becomes the state of the block opened by append_block; a block without masks goes straight to
    its own commit pass."""
    sched, seqs = _running_seqs(mdb, 2)
    a, b = seqs
    for s in seqs:
        s.current_denoising_block = torch.full((32,), 7, dtype=torch.int64)
    sched.postprocess(seqs)
    assert a.is_caching and b.is_caching
    first = torch.full((32,), 1000, dtype=torch.int64)
    first[3] = 55
    moved = np.zeros(32, dtype=bool)
    moved[3] = True
    a.pending_first_step = (first, moved)
    done = torch.arange(32, dtype=torch.int64)
    b.pending_first_step = (done, np.ones(32, dtype=bool))
    step_a, step_b = a.current_denoise_step, b.current_denoise_step
    sched.postprocess(seqs)
    assert a.pending_first_step is None and b.pending_first_step is None
    assert torch.equal(a.current_denoising_block, first) and not a.is_caching
    assert a.current_denoise_step == step_a + 1 and int(a.current_step_map[3]) == step_a
    assert torch.equal(b.current_denoising_block, done) and b.is_caching
    assert b.current_denoise_step == step_b + 1
    assert a.token_ids[-32:] == [7] * 32 and b.token_ids[-32:] == [7] * 32


def test_lm_head_split_covers_the_vocabulary():
    """The two ranks of a tensor-parallel pair scan disjoint column ranges that cover the vocabulary
    (the reference shards it evenly, NV/layers/embed_head.py:19-23); for steps of more than 64 rows rank 0's
    range ends on a 256-column boundary because a sampler record covers one 256-column tile."""
    import importlib
    tp = importlib.import_module("mineru-diffusion_b200.tp")
    for vocab in (151936, 1024, 32000, 128 * 7, 256, 128):
        for many in (False, True):
            b0, c0, p0 = tp.lm_head_split(vocab, 0, many)
            b1, c1, p1 = tp.lm_head_split(vocab, 1, many)
            assert b0 == 0 and b1 == c0 and (c0 + c1) * 128 == vocab
            assert p0 == c1 * 128 and p1 == c0 * 128
            if many and c1 > 0:
                assert (c0 * 128) % 256 == 0
            assert abs(c0 - c1) <= 2


def test_small_batch_fill_matches_vectorised_builder(mdb):
    """The direct fill used for up to four requests writes what the vectorised builder returns (ids, positions,
    slots, context lengths, the page-table prefix), including blocks that straddle two pages, page-aligned ends
    and a request without pages."""
    import importlib
    si = importlib.import_module("mineru-diffusion_b200.engine.step_inputs")
    gen = torch.Generator().manual_seed(1)
    for block in (8, 32, 64):
        lens = (1, 255, 256 - block, 257, 511, 700, 1024 - block, 3000, 240)
        for start in range(0, len(lens), 3):
            seqs = []
            for n in lens[start:start + 3]:
                sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=64, ignore_eos=True)
                seq = mdb.Sequence(torch.randint(0, 100, (n,), generator=gen).tolist(), sp, denoising_block_size=block,
                                   mask_token_id=1000)
                seq.block_table = torch.randperm(64, generator=gen)[:(n + block + 255) // 256].tolist()
                seq.current_denoising_block[::3] = 5
                seqs.append(seq)
            if start == 3:
                seqs[1].block_table = []
            want = si.build_decode_inputs(seqs, block)
            bs = len(seqs)
            ids = np.zeros((4, block), np.int64); pos = np.zeros((4, block), np.int64)
            slots = np.full((4, block), -1, np.int32); ctx = np.zeros(4, np.int32); tab = np.full((4, 16), -1, np.int32)
            longest = si.fill_decode_inputs_small(seqs, block, ids, pos, slots, ctx, tab)
            assert np.array_equal(ids[:bs], want["input_ids"]) and np.array_equal(pos[:bs], want["positions"])
            assert np.array_equal(slots[:bs], want["slot_mapping"]) and np.array_equal(ctx[:bs], want["context_lens"])
            width = want["block_tables"].shape[1]
            assert np.array_equal(tab[:bs, :width], want["block_tables"])
            assert longest == int(want["context_lens"].max())
    sp = mdb.SamplingParams(temperature=1.0, max_new_tokens=64, ignore_eos=True)
    seq = mdb.Sequence(list(range(250)), sp, denoising_block_size=32, mask_token_id=1000)
    seq.block_table = [3]                     # the block needs a second page
    with pytest.raises(IndexError):
        si.fill_decode_inputs_small([seq], 32, np.zeros((1, 32), np.int64), np.zeros((1, 32), np.int64),
                                    np.zeros((1, 32), np.int32), np.zeros(1, np.int32), np.full((1, 4), -1, np.int32))


def test_tensor_parallel_shards_recompose_the_layer(mdb):
    """tp.shard_weights cuts q|k|v rows by head, o_proj columns by head, gate|up rows and down_proj columns the
    way the reference's weight loaders do (NV/layers/linear.py:54-151): the column-parallel outputs of the two
    ranks are the matching columns of the full output, and the row-parallel outputs add up to it."""
    import importlib
    tp = importlib.import_module("mineru-diffusion_b200.tp")
    dec = importlib.import_module("mineru-diffusion_b200.decoder")
    cfg = mdb.DecoderConfig(vocab_size=256, hidden_size=64, intermediate_size=96, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=64)
    g = torch.Generator().manual_seed(0)
    h, d, hq, hkv, inter = 64, 16, 4, 2, 96
    rnd = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    layer = dec.LayerWeights(rnd(h), rnd((hq + 2 * hkv) * d, h), rnd(d), rnd(d), rnd(h, hq * d), rnd(h), rnd(2 * inter, h),
                             rnd(h, inter))
    full = dec.DecoderWeights(rnd(256, h), [layer], rnd(h), rnd(256, h))
    local = tp.shard_config(cfg, 2)
    assert (local.num_attention_heads, local.num_key_value_heads, local.intermediate_size) == (2, 1, 48)
    x = rnd(5, h)
    qkv = x @ layer.qkv.T
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=1)
    attn = rnd(5, hq * d)
    gate, up = (x @ layer.gate_up.T).split([inter, inter], dim=1)
    act = torch.nn.functional.silu(gate) * up
    o_sum, down_sum = torch.zeros(5, h, dtype=torch.float64), torch.zeros(5, h, dtype=torch.float64)
    for rank in range(2):
        w = tp.shard_weights(full, cfg, rank, 2).layers[0]
        lq, lk, lv = (x @ w.qkv.T).split([2 * d, d, d], dim=1)
        assert torch.equal(lq, q[:, rank * 2 * d:(rank + 1) * 2 * d])
        assert torch.equal(lk, k[:, rank * d:(rank + 1) * d]) and torch.equal(lv, v[:, rank * d:(rank + 1) * d])
        o_sum += attn[:, rank * 2 * d:(rank + 1) * 2 * d] @ w.o.T
        lg, lu = (x @ w.gate_up.T).split([48, 48], dim=1)
        lact = torch.nn.functional.silu(lg) * lu
        assert torch.equal(lact, act[:, rank * 48:(rank + 1) * 48])
        down_sum += lact @ w.down.T
    assert torch.allclose(o_sum, attn @ layer.o.T, rtol=1e-12, atol=1e-12)
    assert torch.allclose(down_sum, act @ layer.down.T, rtol=1e-12, atol=1e-12)
    with pytest.raises(ValueError):
        tp.shard_config(mdb.DecoderConfig(num_attention_heads=3, num_key_value_heads=3), 2)


def test_attention_part_policy(mdb):
    """ops.default_nsplit: key-range parts fill the 148 SMs once and no more, at most 16, none below 256 keys,
    and no split from 16 requests on (decoder shapes: 16 query / 8 KV heads, block 32)."""
    n = lambda bs, ctx, block=32, hq=16, hkv=8: mdb.ops.default_nsplit(bs, block, hq, hkv, ctx)
    assert n(1, 4096) == 16 and n(1, 1100) == 4 and n(1, 200) == 1
    assert n(2, 8192) == 9 and n(4, 8192) == 4 and n(8, 8192) == 2
    assert all(n(bs, 8192) == 1 for bs in (16, 19, 32, 64, 512))
    for bs in (1, 2, 3, 4, 6, 8, 12):
        for ctx in (300, 1000, 5000, 16416):
            parts = n(bs, ctx)
            assert 1 <= parts <= 16 and parts <= max(1, ctx // 256)
            assert parts == 1 or bs * 8 * parts <= 148
    # a block of 64 with two heads per KV head still is one 128-row CTA per (request, KV head)
    assert n(1, 4096, block=64) == 16
    # 8 query heads per KV head, block 32: 256 rows = two 128-row CTAs per (request, KV head)
    assert n(1, 4096, hq=16, hkv=2) == 16 and n(8, 4096, hq=16, hkv=2) == 4
