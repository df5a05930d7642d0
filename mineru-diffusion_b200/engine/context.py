"""Per-step metadata handed from the model runner to the ops.

Field-for-field the reference's module-global ``Context``
(``engines/nano_dvlm/nanovllm/utils/context.py:5-28``); here it is an explicit
object the runner passes down rather than a global.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Context:
    is_prefill: bool = False
    cu_seqlens_q: torch.Tensor | None = None
    cu_seqlens_k: torch.Tensor | None = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    slot_mapping: torch.Tensor | None = None
    context_lens: torch.Tensor | None = None
    block_tables: torch.Tensor | None = None
    block_size: int = 32
