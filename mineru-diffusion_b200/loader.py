"""Decoder weights from a safetensors checkpoint in the reference's parameter names.

Follows ``load_model`` of the reference (``nanovllm/utils/loader.py:12-28``) with the packed-module map of
``SDARForCausalLM`` (``nanovllm/models/sdar.py:185-191``): the checkpoint stores ``q_proj`` / ``k_proj`` /
``v_proj`` and ``gate_proj`` / ``up_proj`` separately, the engine keeps them as the row-concatenated ``qkv`` (q|k|v)
and ``gate_up`` (gate|up) matrices.  For a tensor-parallel pair each rank takes the slice the reference's weight
loaders take (``nanovllm/layers/linear.py:65-70,87-93,114-128,142-151``): q/k/v and gate/up row chunks,
o_proj / down_proj column ranges.  Embedding and LM head stay whole on every rank (the LM head is read by
vocabulary-tile range).  With ``tie_word_embeddings`` the LM head is the embedding (``sdar.py:200-201``) and the
checkpoint need not hold ``lm_head.weight``.

Only the language decoder is read: names under ``vision_model.`` / ``vision_abstractor.`` (the vision tower and
the projector, which stay with the reference) are skipped.
"""
from __future__ import annotations

import os
import re
from glob import glob

import torch

from .decoder import DecoderWeights, LayerWeights
from .engine.config import DecoderConfig

_LAYER = re.compile(r"^model\.layers\.(\d+)\.(.+)\.weight$")
_SKIPPED_PREFIXES = ("vision_model.", "vision_abstractor.", "visual.", "vision_tower.")


def _strip(name: str) -> str | None:
    """Parameter name relative to ``SDARForCausalLM``; None for tensors outside the decoder."""
    if name.startswith(_SKIPPED_PREFIXES):
        return None
    if name.startswith("language_model."):
        name = name[len("language_model."):]
    return name


def load_decoder_weights(path: str, cfg: DecoderConfig, device, tp_rank: int = 0, tp_size: int = 1,
                         dtype=torch.bfloat16) -> DecoderWeights:
    """Reads every ``*.safetensors`` file of ``path`` and returns this rank's ``DecoderWeights`` on ``device``.
    Raises ``KeyError`` for a missing tensor and ``ValueError`` for one of the wrong shape or an unknown name."""
    from safetensors import safe_open
    files = sorted(glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no *.safetensors file in {path}")
    if tp_size < 1 or not 0 <= tp_rank < tp_size:
        raise ValueError("tp_rank must be in [0, tp_size)")
    d, h, inter = cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
    hq, hkv, layers = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.num_hidden_layers
    if hq % tp_size or hkv % tp_size or inter % tp_size:
        raise ValueError("heads and intermediate size must divide by the tensor-parallel size")
    q_rows, kv_rows, i_rows = hq * d // tp_size, hkv * d // tp_size, inter // tp_size

    def empty(*shape):
        return torch.empty(shape, dtype=dtype, device=device)

    lw = [dict(input_ln=empty(h), qkv=empty(q_rows + 2 * kv_rows, h), q_norm=empty(d), k_norm=empty(d),
               o=empty(h, q_rows), post_ln=empty(h), gate_up=empty(2 * i_rows, h), down=empty(h, i_rows))
          for _ in range(layers)]
    top = dict(embed=empty(cfg.vocab_size, h), final_ln=empty(h),
               lm_head=None if cfg.tie_word_embeddings else empty(cfg.vocab_size, h))
    seen: set[str] = set()

    def put(dst: torch.Tensor, src: torch.Tensor, name: str):
        if tuple(dst.shape) != tuple(src.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} does not fit {tuple(dst.shape)}")
        dst.copy_(src.to(dtype))

    def row_chunk(t: torch.Tensor) -> torch.Tensor:          # ColumnParallel: this rank's rows
        return t.chunk(tp_size, 0)[tp_rank]

    def col_range(t: torch.Tensor, width: int) -> torch.Tensor:   # RowParallel: this rank's input columns
        return t.narrow(1, tp_rank * width, width)

    for file in files:
        with safe_open(file, "pt", "cpu") as f:
            for raw in f.keys():
                name = _strip(raw)
                if name is None:
                    continue
                m = _LAYER.match(name)
                if m:
                    li, what = int(m.group(1)), m.group(2)
                    if li >= layers:
                        raise ValueError(f"{raw}: the configuration has {layers} layers")
                    t, w = f.get_tensor(raw), lw[li]
                    if what == "self_attn.q_proj":
                        put(w["qkv"][:q_rows], row_chunk(t), raw)
                    elif what == "self_attn.k_proj":
                        put(w["qkv"][q_rows:q_rows + kv_rows], row_chunk(t), raw)
                    elif what == "self_attn.v_proj":
                        put(w["qkv"][q_rows + kv_rows:], row_chunk(t), raw)
                    elif what == "self_attn.o_proj":
                        put(w["o"], col_range(t, q_rows), raw)
                    elif what == "mlp.gate_proj":
                        put(w["gate_up"][:i_rows], row_chunk(t), raw)
                    elif what == "mlp.up_proj":
                        put(w["gate_up"][i_rows:], row_chunk(t), raw)
                    elif what == "mlp.down_proj":
                        put(w["down"], col_range(t, i_rows), raw)
                    elif what == "self_attn.q_norm":
                        put(w["q_norm"], t, raw)
                    elif what == "self_attn.k_norm":
                        put(w["k_norm"], t, raw)
                    elif what == "input_layernorm":
                        put(w["input_ln"], t, raw)
                    elif what == "post_attention_layernorm":
                        put(w["post_ln"], t, raw)
                    else:
                        raise ValueError(f"{raw}: not a parameter of the decoder layer")
                    seen.add(f"{li}.{what}")
                elif name == "model.embed_tokens.weight":
                    put(top["embed"], f.get_tensor(raw), raw)
                    seen.add("embed")
                elif name == "model.norm.weight":
                    put(top["final_ln"], f.get_tensor(raw), raw)
                    seen.add("final_ln")
                elif name == "lm_head.weight":
                    if top["lm_head"] is not None:       # tied: the embedding is the head, a stored copy is ignored
                        put(top["lm_head"], f.get_tensor(raw), raw)
                    seen.add("lm_head")
                else:
                    raise ValueError(f"{raw}: not a parameter of the decoder")
    per_layer = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "self_attn.q_norm",
                 "self_attn.k_norm", "input_layernorm", "post_attention_layernorm", "mlp.gate_proj", "mlp.up_proj",
                 "mlp.down_proj")
    missing = [f"model.layers.{li}.{p}.weight" for li in range(layers) for p in per_layer if f"{li}.{p}" not in seen]
    missing += [n for key, n in (("embed", "model.embed_tokens.weight"), ("final_ln", "model.norm.weight")) if key not in seen]
    if not cfg.tie_word_embeddings and "lm_head" not in seen:
        missing.append("lm_head.weight")
    if missing:
        raise KeyError(f"checkpoint lacks {len(missing)} tensors, first: {missing[:4]}")
    lm_head = top["embed"] if cfg.tie_word_embeddings else top["lm_head"]
    return DecoderWeights(top["embed"], [LayerWeights(**w) for w in lw], top["final_ln"], lm_head)


def has_checkpoint(path: str | None) -> bool:
    return bool(path) and os.path.isdir(path) and bool(glob(os.path.join(path, "*.safetensors")))
