"""Per-request sampling knobs of the block-diffusion sampler.

Same fields, defaults and validation as the reference's
``engines/nano_dvlm/nanovllm/sampling_params.py:4-15``; ``denoising_steps`` is
the one addition (the HF twin has it at
``mineru_diffusion/modeling_mineru_diffusion.py:631``) and ``None`` keeps the
nano behaviour of a quota of one token per step.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    temperature: float = 1.0
    max_new_tokens: int = 64
    ignore_eos: bool = False
    denoising_strategy: str = "low_confidence_dynamic"
    dynamic_threshold: float = 0.9
    stop_tokens: list[str] | None = None
    stop_token_ids: list[int] | None = None
    denoising_steps: int | None = None

    def __post_init__(self):
        if not self.temperature > 1e-10:
            raise AssertionError("greedy sampling is not permitted")
        if self.stop_token_ids is None:
            self.stop_token_ids = []
