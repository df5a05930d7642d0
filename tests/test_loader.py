"""The safetensors loader on synthetic checkpoints written in the reference's parameter names (separate q/k/v
and gate/up tensors under ``language_model.``, tied and untied embeddings, vision tensors to skip), for one
GPU and for both ranks of a tensor-parallel pair.  No GPU needed: the weights are loaded onto the CPU."""
import os

import pytest
import torch


def _write_checkpoint(path, cfg, seed, tied, with_lm_head=True, drop=None, files=2):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)
    d, h, inter = cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
    hq, hkv = cfg.num_attention_heads, cfg.num_key_value_heads

    def mat(*shape):
        return torch.randn(*shape, generator=g).to(torch.bfloat16)

    t = {"language_model.model.embed_tokens.weight": mat(cfg.vocab_size, h),
         "language_model.model.norm.weight": mat(h),
         "vision_model.blocks.0.attn.qkv.weight": mat(8, 8),          # the vision tower is not ours to load
         "vision_abstractor.proj.weight": mat(4, 4)}
    if with_lm_head and not tied:
        t["language_model.lm_head.weight"] = mat(cfg.vocab_size, h)
    for li in range(cfg.num_hidden_layers):
        p = f"language_model.model.layers.{li}."
        t[p + "self_attn.q_proj.weight"] = mat(hq * d, h)
        t[p + "self_attn.k_proj.weight"] = mat(hkv * d, h)
        t[p + "self_attn.v_proj.weight"] = mat(hkv * d, h)
        t[p + "self_attn.o_proj.weight"] = mat(h, hq * d)
        t[p + "self_attn.q_norm.weight"] = mat(d)
        t[p + "self_attn.k_norm.weight"] = mat(d)
        t[p + "input_layernorm.weight"] = mat(h)
        t[p + "post_attention_layernorm.weight"] = mat(h)
        t[p + "mlp.gate_proj.weight"] = mat(inter, h)
        t[p + "mlp.up_proj.weight"] = mat(inter, h)
        t[p + "mlp.down_proj.weight"] = mat(h, inter)
    if drop:
        del t[drop]
    names = sorted(t)
    for i in range(files):                      # sharded over several files, as hub checkpoints are
        save_file({n: t[n].contiguous() for n in names[i::files]}, os.path.join(path, f"model-{i:05d}.safetensors"))
    return t


@pytest.mark.parametrize("tied", [False, True])
def test_loader_packs_and_shards_like_the_reference(mdb, tmp_path, tied):
    cfg = mdb.DecoderConfig(vocab_size=96, hidden_size=64, intermediate_size=48, num_hidden_layers=2,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16, tie_word_embeddings=tied)
    t = _write_checkpoint(str(tmp_path), cfg, seed=3, tied=tied)
    w = mdb.load_decoder_weights(str(tmp_path), cfg, "cpu")
    pre = "language_model.model.layers.1."
    assert torch.equal(w.layers[1].qkv, torch.cat([t[pre + "self_attn.q_proj.weight"], t[pre + "self_attn.k_proj.weight"],
                                                   t[pre + "self_attn.v_proj.weight"]]))
    assert torch.equal(w.layers[1].gate_up, torch.cat([t[pre + "mlp.gate_proj.weight"], t[pre + "mlp.up_proj.weight"]]))
    assert torch.equal(w.layers[1].o, t[pre + "self_attn.o_proj.weight"])
    assert torch.equal(w.layers[1].down, t[pre + "mlp.down_proj.weight"])
    assert torch.equal(w.layers[0].q_norm, t["language_model.model.layers.0.self_attn.q_norm.weight"])
    assert torch.equal(w.layers[0].post_ln, t["language_model.model.layers.0.post_attention_layernorm.weight"])
    assert torch.equal(w.embed, t["language_model.model.embed_tokens.weight"])
    assert torch.equal(w.final_ln, t["language_model.model.norm.weight"])
    if tied:
        assert w.lm_head.data_ptr() == w.embed.data_ptr()       # sdar.py:200-201
    else:
        assert torch.equal(w.lm_head, t["language_model.lm_head.weight"])
    # the two ranks of a pair: the same slices tp.shard_weights cuts out of the full set, which are the
    # reference's weight-loader slices (linear.py:65-70,87-93,114-128,142-151)
    tp = __import__("importlib").import_module("mineru-diffusion_b200.tp")
    for rank in (0, 1):
        got = mdb.load_decoder_weights(str(tmp_path), cfg, "cpu", tp_rank=rank, tp_size=2)
        want = tp.shard_weights(w, cfg, rank, 2)
        for a, b in zip(got.layers, want.layers):
            for f in ("input_ln", "qkv", "q_norm", "k_norm", "o", "post_ln", "gate_up", "down"):
                assert torch.equal(getattr(a, f), getattr(b, f)), (rank, f)
        assert torch.equal(got.embed, want.embed) and torch.equal(got.lm_head, want.lm_head)
    # per-shard slices straight from the reference's rule: k_proj rows chunk(2)[rank], o_proj columns narrow
    k = t["language_model.model.layers.0.self_attn.k_proj.weight"]
    o = t["language_model.model.layers.0.self_attn.o_proj.weight"]
    r1 = mdb.load_decoder_weights(str(tmp_path), cfg, "cpu", tp_rank=1, tp_size=2)
    q_rows = cfg.num_attention_heads * cfg.head_dim // 2
    kv_rows = cfg.num_key_value_heads * cfg.head_dim // 2
    assert torch.equal(r1.layers[0].qkv[q_rows:q_rows + kv_rows], k.chunk(2, 0)[1])
    assert torch.equal(r1.layers[0].o, o.narrow(1, q_rows, q_rows))


def test_loader_reports_missing_and_misshapen_tensors(mdb, tmp_path):
    cfg = mdb.DecoderConfig(vocab_size=96, hidden_size=64, intermediate_size=48, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    a = tmp_path / "a"
    a.mkdir()
    _write_checkpoint(str(a), cfg, seed=4, tied=False, drop="language_model.model.layers.0.mlp.up_proj.weight")
    with pytest.raises(KeyError, match="up_proj"):
        mdb.load_decoder_weights(str(a), cfg, "cpu")
    b = tmp_path / "b"
    b.mkdir()
    _write_checkpoint(str(b), cfg, seed=4, tied=False, with_lm_head=False)
    with pytest.raises(KeyError, match="lm_head"):
        mdb.load_decoder_weights(str(b), cfg, "cpu")
    wide = mdb.DecoderConfig(vocab_size=96, hidden_size=64, intermediate_size=64, num_hidden_layers=1,
                             num_attention_heads=4, num_key_value_heads=2, head_dim=16)
    c = tmp_path / "c"
    c.mkdir()
    _write_checkpoint(str(c), cfg, seed=4, tied=False)
    with pytest.raises(ValueError, match="does not fit"):
        mdb.load_decoder_weights(str(c), wide, "cpu")
    with pytest.raises(FileNotFoundError):
        mdb.load_decoder_weights(str(tmp_path / "a" / "none"), cfg, "cpu")
