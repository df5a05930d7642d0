"""Pins the CPU oracle against outputs of the reference's own modules
(fixtures written by tests/golden/make_golden.py).  No GPU needed."""
import numpy as np
import torch

from conftest import bf16_from_bits, load_golden, ulp_diff_bf16
from oracle import nano_oracle as orc


def test_get_slots_matches_reference():
    g = load_golden("index_contract.npz")
    table = g["slots_table"].tolist()
    for i, (lo, hi) in enumerate(g["slots_cases"].tolist()):
        assert orc.get_slots(table, lo, hi) == g[f"slots_{i}"].tolist()
    assert orc.get_slots([], 3, 7) == [-1] * 4


def test_staircase_mask_matches_hf_builder():
    g = load_golden("staircase.npz")
    for key in [k for k in g if k.startswith("hf_mask_")]:
        p, gen, b = (int(x) for x in key.split("_")[2:])
        hf = torch.from_numpy(g[key])
        # prompt part: right-aligned staircase over the prompt alone
        assert torch.equal(orc.staircase_mask(p, b), hf[:p, :p]), key
        # prompt + first block: the last block sees everything, prompt rows unchanged
        t = p + b
        ours = orc.staircase_mask(t, b)
        assert torch.equal(ours[:p, :p], hf[:p, :p])
        assert bool(ours[p:, :].all())
        assert torch.equal(ours[p:t, :t], hf[p:t, :t])


def test_staircase_attention_matches_triton_kernel():
    g = load_golden("staircase.npz")
    lens = g["lens"].tolist()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    q = torch.from_numpy(g["q"]).float()
    k = torch.from_numpy(g["k"]).float()
    v = torch.from_numpy(g["v"]).float()
    for stairs in (32, 8):
        out = orc.attn_staircase_varlen(q, k, v, cu, cu, stairs, mirror_rounding=False)
        ref = torch.from_numpy(g[f"out_fp32_s{stairs}"])
        assert (out - ref).abs().max() < 5e-6
    # fp16 run of the kernel: the restatement with the kernel's two roundings must sit closer
    qh, kh, vh = q.half(), k.half(), v.half()
    ref16 = torch.from_numpy(g["out_fp16_s32"])
    mirrored = orc.attn_staircase_varlen(qh, kh, vh, cu, cu, 32, mirror_rounding=True).float()
    assert (mirrored - ref16).abs().max() < 2e-3
    # bf16 restatement on inputs that bf16 holds exactly against the kernel's fp32 run on the same values: only
    # the roundings inside (q * scale, P, the output) remain
    lens = g["lens_bf"].tolist()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    qb, kb, vb = (bf16_from_bits(g[x]) for x in ("q_bf", "k_bf", "v_bf"))
    for stairs in (32, 8):
        out = orc.attn_staircase_varlen(qb, kb, vb, cu, cu, stairs)
        ref = torch.from_numpy(g[f"out_fp32_bf_s{stairs}"])
        assert (out.float() - ref).abs().max() < 8e-3


def test_layers_match_reference_modules():
    g = load_golden("layers.npz")
    bf = bf16_from_bits
    w, x, res = bf(g["norm_w"]), bf(g["x"]), bf(g["res"])
    assert torch.equal(orc.rms_norm(x, w, 1e-6), bf(g["y_plain"]))
    y, r = orc.add_rms_norm(x, res, w, 1e-6)
    assert torch.equal(y, bf(g["y_add"]))
    assert torch.equal(r, bf(g["res_out"]))
    assert torch.equal(orc.rms_norm(bf(g["heads"]), bf(g["head_norm_w"]), 1e-6), bf(g["heads_normed"]))
    table = orc.rope_table(4096, 128, 1000000.0)
    assert torch.equal(table[[0, 1, 17, 4095]], torch.from_numpy(g["rope_table_probe"]))
    pos = torch.from_numpy(g["rope_pos"])
    assert torch.equal(orc.apply_rope(bf(g["rope_q"]), pos, table), bf(g["rope_q_out"]))
    assert torch.equal(orc.apply_rope(bf(g["rope_k"]), pos, table), bf(g["rope_k_out"]))
    # SiLU*mul against liger's kernel in fp32
    out = orc.silu_mul(torch.from_numpy(g["silu_in"]))
    assert (out - torch.from_numpy(g["silu_out"])).abs().max() < 1e-6


def test_store_kvcache_matches_triton_kernel():
    g = load_golden("layers.npz")
    bf = bf16_from_bits
    kc = torch.zeros(3, 256, 2, 128, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    orc.store_kvcache(bf(g["kv_k"]), bf(g["kv_v"]), kc, vc, torch.from_numpy(g["kv_slots"]))
    touched = g["kv_touched"].tolist()
    assert torch.equal(kc.view(-1, 256)[touched], bf(g["kv_kc_rows"]))
    assert torch.equal(vc.view(-1, 256)[touched], bf(g["kv_vc_rows"]))
    assert abs(float(kc.float().abs().sum()) - float(g["kv_kc_sum"])) < 1e-3   # nothing else written


def test_sampler_matches_reference():
    g = load_golden("sampler.npz")
    mask_id, thr = int(g["mask_id"]), float(g["threshold"])
    for case in range(3):
        p = f"c{case}_"
        logits = bf16_from_bits(g[p + "logits"])
        bs = logits.shape[0]
        temps = torch.full((bs, 1), float(g[p + "temp"]))
        x0, x0_p = orc.sampler_prepare(logits, temps, torch.from_numpy(g[p + "gumbel"]))
        assert torch.equal(x0, torch.from_numpy(g[p + "x0"]))
        assert torch.allclose(x0_p, torch.from_numpy(g[p + "x0_p"]), rtol=1e-6, atol=0)
        after, transfer = orc.unmask_decision(torch.from_numpy(g[p + "before"]), x0, x0_p, mask_id, thr)
        assert torch.equal(after, torch.from_numpy(g[p + "after"]))
        assert torch.equal(transfer, torch.from_numpy(g[p + "transfer"]))
        assert int(transfer.sum()) == int(g[p + "count"])
    # the threshold branch and the top-1 branch are both exercised
    assert int(g["c1_count"]) > 3 and int(g["c0_count"]) == 3


class _Seq:
    """Duck-typed request for OracleModelRunner."""
    def __init__(self, seq_id, ids, block, mask_id, table):
        from types import SimpleNamespace
        self.seq_id, self.token_ids, self.block_table = seq_id, list(ids), list(table)
        self.num_cached_tokens = 0
        self.temperature = 1.0
        self.mask_token_id = mask_id
        self.sampling_params = SimpleNamespace(dynamic_threshold=0.9)
        self.current_denoising_block = torch.full((block,), mask_id, dtype=torch.int64)
        self.current_step_map = torch.full((block,), -1, dtype=torch.int32)
        self.current_denoise_step = 0

    def __len__(self):
        return len(self.token_ids)

    def __getitem__(self, k):
        return self.token_ids[k]


def test_decoder_steps_match_reference_modules():
    """Prefill + decode steps of a 2-layer decoder through the reference's
    nano_dvlm modules vs the restatement: same weights, pages, noise."""
    g = load_golden("decoder_tiny.npz")
    cfg = orc.DecoderConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=2048)
    w = orc.make_weights(cfg, seed=21)
    mask_id = int(g["mask_id"])
    noise = {s: torch.from_numpy(g[f"s{s}_gumbel"]) for s in range(int(g["num_steps"]))}
    runner = orc.OracleModelRunner(cfg, w, num_pages=6, block_size=32, mask_token_id=mask_id,
                                   noise_fn=lambda step, shape: noise[step])
    tables0 = g["s0_block_tables"]
    seqs = [_Seq(0, g["prompt0"].tolist(), 32, mask_id, [t for t in tables0[0] if t >= 0]),
            _Seq(1, g["prompt1"].tolist(), 32, mask_id, [t for t in tables0[1] if t >= 0])]
    for step in range(int(g["num_steps"])):
        p = f"s{step}_"
        for seq, row in zip(seqs, g[p + "block_tables"]):
            seq.block_table = [int(t) for t in row if t >= 0]
        n = runner.run(seqs, bool(g[p + "is_prefill"]))
        ref_logits = bf16_from_bits(g[p + "logits"])
        got = runner.last["logits"]
        # bf16 logits: the two paths differ only in fp32 summation order
        diff = (got.float() - ref_logits.float()).abs()
        print(f"step {step}: logits max-abs {float(diff.max()):.4f} mean-abs {float(diff.mean()):.5f} "
              f"(logit std {float(ref_logits.float().std()):.3f})")
        assert float(diff.max()) <= 2e-2 and float(diff.mean()) <= 3e-3
        assert torch.equal(runner.last["x0"], torch.from_numpy(g[p + "x0"]))
        assert torch.allclose(runner.last["x0_p"], torch.from_numpy(g[p + "x0_p"]), rtol=2e-2)
        assert n == int(g[p + "count"])
        blocks = torch.stack([s.current_denoising_block for s in seqs])
        assert torch.equal(blocks, torch.from_numpy(g[p + "blocks_after"]))
        kv = runner.decoder.kv_cache
        sums = [float(kv[0].float().abs().sum()), float(kv[1].float().abs().sum())]
        assert np.allclose(sums, g[p + "kv_abs_sum"], rtol=2e-3)
        if step == 0:
            tab = seqs[0].block_table
            k_rows = bf16_from_bits(g[p + "k_l0_first_rows"])
            v_rows = bf16_from_bits(g[p + "v_l0_first_rows"])
            assert int(ulp_diff_bf16(kv[0, 0, tab[0], :8], k_rows).max()) <= 1
            assert int(ulp_diff_bf16(kv[1, 0, tab[0], :8], v_rows).max()) <= 1


def test_hf_twin_quota_rule_and_schedule():
    """The quota form of the unmask rule and the per-block quota schedule against the HF twin's own
    ``_select_transfer_index`` / ``get_num_transfer_tokens``
    (mineru_diffusion/modeling_mineru_diffusion.py:518-532,617-623)."""
    g = load_golden("hf_twin.npz")
    for b, steps in g["sched_pairs"].tolist():
        assert orc.num_transfer_tokens(b, steps) == g[f"sched_{b}_{steps}"].tolist()
    thr = float(g["threshold"])
    mask_id = 99999
    for i in range(int(g["num_cases"])):
        conf = torch.from_numpy(g[f"q{i}_conf"])
        masked = torch.from_numpy(g[f"q{i}_masked"])
        count = int(g[f"q{i}_count"])
        blocks = torch.where(masked, torch.full(masked.shape, mask_id, dtype=torch.int64),
                             torch.zeros(masked.shape, dtype=torch.int64))
        x0 = torch.arange(conf.numel(), dtype=torch.int64).view(conf.shape) + 1
        out, transfer = orc.unmask_decision(blocks, x0, conf, mask_id, thr, quotas=[count] * conf.shape[0])
        assert torch.equal(transfer, torch.from_numpy(g[f"q{i}_transfer"])), i
        assert torch.equal(out[transfer], x0[transfer]) and torch.equal(out[~transfer], blocks[~transfer])
