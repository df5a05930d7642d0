"""Engine configuration.

Same fields and defaults as ``engines/nano_dvlm/nanovllm/config.py:33-60``.
``model`` may be a directory holding ``config.json`` (read like the reference
does) or ``None`` when ``decoder_config`` is passed directly, which is how the
synthetic-weight workloads are set up.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from types import SimpleNamespace


@dataclass
class DecoderConfig:
    """Decoder dimensions; defaults from
    ``mineru_diffusion/configuration_mineru_diffusion.py:12-32``."""
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
    tie_word_embeddings: bool = False

    @classmethod
    def from_namespace(cls, ns) -> "DecoderConfig":
        kw = {}
        for name in cls.__dataclass_fields__:
            if hasattr(ns, name):
                kw[name] = getattr(ns, name)
        if "head_dim" not in kw and hasattr(ns, "hidden_size") and hasattr(ns, "num_attention_heads"):
            kw["head_dim"] = ns.hidden_size // ns.num_attention_heads
        return cls(**kw)


@dataclass
class Config:
    model: str | None = None
    checkpoint: str | None = None
    max_num_batched_tokens: int = 16384
    max_num_seqs: int = 512
    max_model_len: int = 4096
    gpu_memory_utilization: float = 0.9
    tensor_parallel_size: int = 1
    enforce_eager: bool = False
    hf_config: SimpleNamespace | None = None
    eos: int = -1
    kvcache_block_size: int = 256
    num_kvcache_blocks: int = -1
    mask_token_id: int = 151669
    block_size: int = 32
    decoder_config: DecoderConfig | None = None
    # Not in the reference: a request whose block is complete runs the pass that writes the block's final K/V
    # and, in the same step, the first denoising pass of its next block (one pass per block saved; the tokens
    # are the ones the two separate passes would produce from the same noise).  Off: the reference's schedule.
    fuse_commit_pass: bool = False
    # Not in the reference: after a decode step whose requests all stay on their blocks, the runner launches the
    # next step at once (same requests, the block ids just produced) instead of waiting for the scheduler to ask
    # for it; when the scheduler then asks for exactly that step, only its results are collected, otherwise they
    # are thrown away and the step asked for runs.  Same tokens either way; the host's work between two steps
    # overlaps with the GPU's.
    launch_ahead: bool = True

    def __post_init__(self):
        if self.kvcache_block_size % 256 != 0:
            raise AssertionError("kvcache_block_size must be a multiple of 256")
        if not 1 <= self.tensor_parallel_size <= 8:
            raise AssertionError("tensor_parallel_size must be in 1..8")
        if self.model is not None:
            if not os.path.isdir(self.model):
                raise AssertionError(f"{self.model} is not a directory")
            path = self.model if self.checkpoint is None else os.path.join(self.model, self.checkpoint)
            with open(os.path.join(path, "config.json")) as f:
                raw = json.load(f)
            text = raw.get("language_model_config") or raw.get("text_config") or raw
            self.hf_config = SimpleNamespace(**raw)
            if self.decoder_config is None:
                self.decoder_config = DecoderConfig.from_namespace(SimpleNamespace(**text))
        if self.decoder_config is None:
            self.decoder_config = DecoderConfig()
        self.max_model_len = min(self.max_model_len, self.decoder_config.max_position_embeddings)
        if self.max_num_batched_tokens < self.max_model_len:
            raise AssertionError("max_num_batched_tokens must cover max_model_len")
