"""Host-side request state for block-diffusion decoding.

Mirrors ``engines/nano_dvlm/nanovllm/engine/sequence.py`` (same attribute and
method names, same integer results) so the scheduler and the model runner read
like the reference's.  Token ids live in a python list; the block being
denoised is a CPU int64 tensor of ``denoising_block_size`` ids, all equal to
``mask_token_id`` when a block starts.
"""
from __future__ import annotations

from enum import Enum, auto
from itertools import count

import torch

from .sampling_params import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    CACHING = auto()    # block fully unmasked; next pass only commits its K/V
    FINISHED = auto()


class Sequence:
    kvcache_block_size = 256   # tokens per KV page (sequence.py:17 of the reference)
    counter = count()

    def __init__(self, token_ids, sampling_params: SamplingParams | None = None, pixel_values=None,
                 image_grid_thw=None, denoising_block_size: int | None = None, mask_token_id: int | None = None,
                 inputs_embeds: torch.Tensor | None = None):
        sampling_params = sampling_params or SamplingParams()
        self.seq_id = next(Sequence.counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.step_map: list[int] = []
        self.last_token = self.token_ids[-1]
        self.num_tokens = len(self.token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.num_cached_tokens = 0
        self.block_table: list[int] = []
        self.sampling_params = sampling_params
        self.temperature = sampling_params.temperature
        self.max_new_tokens = sampling_params.max_new_tokens
        self.ignore_eos = sampling_params.ignore_eos
        self.pixel_values = pixel_values
        self.image_grid_thw = image_grid_thw
        # rows that replace the token embeddings of the first positions of the
        # prompt (stand-in for the vision tower's output), [n, hidden] or None
        self.inputs_embeds = inputs_embeds
        self.denoising_block_size = denoising_block_size
        self.mask_token_id = mask_token_id
        self.current_denoising_block = self._fresh_block()
        # never-set entries are meaningless in the reference (torch.empty); zero here
        self.current_step_map = torch.zeros(denoising_block_size, dtype=torch.int32)
        self.current_denoise_step = 0
        # (block ids, moved positions) of the next block's first denoising pass when it ran together with this
        # block's commit pass (Config.fuse_commit_pass); applied by Scheduler.postprocess after append_block
        self.pending_first_step = None

    def _fresh_block(self) -> torch.Tensor:
        return torch.full((self.denoising_block_size,), self.mask_token_id, dtype=torch.int64)

    def __len__(self):
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def is_finished(self):
        return self.status is SequenceStatus.FINISHED

    @property
    def is_caching(self):
        return self.status is SequenceStatus.CACHING

    @property
    def num_completion_tokens(self):
        return self.num_tokens - self.num_prompt_tokens

    @property
    def prompt_token_ids(self):
        return self.token_ids[:self.num_prompt_tokens]

    @property
    def completion_token_ids(self):
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_cached_blocks(self):
        return self.num_cached_tokens // self.kvcache_block_size

    @property
    def num_blocks(self):
        return -(-self.num_tokens // self.kvcache_block_size)

    @property
    def last_block_num_tokens(self):
        return self.num_tokens - (self.num_blocks - 1) * self.kvcache_block_size

    def block(self, i: int):
        if not 0 <= i < self.num_blocks:
            raise AssertionError("page index out of range")
        p = self.kvcache_block_size
        return self.token_ids[i * p:(i + 1) * p]

    def append_block(self):
        """Commit the finished block to the sequence and open a new masked one."""
        self.token_ids.extend(self.current_denoising_block.tolist())
        self.step_map.extend(self.current_step_map.tolist())
        self.num_tokens += self.denoising_block_size
        self.last_token = self.token_ids[-1]
        self.current_denoising_block = self._fresh_block()

    def need_new_block(self) -> bool:
        """True when the block being denoised spills past the pages held."""
        return self.num_tokens + self.denoising_block_size > self.kvcache_block_size * len(self.block_table)

    def get_slots(self, lo: int, hi: int) -> list[int]:
        """Flat cache slot (page_id * page + offset) of positions [lo, hi);
        -1 for every position when no page is held (warm-up sequences)."""
        if not self.block_table:
            return [-1] * (hi - lo)
        p = self.kvcache_block_size
        table = self.block_table
        slots: list[int] = []
        pos = lo
        while pos < hi:
            page, off = divmod(pos, p)
            run = min(hi - pos, p - off)
            base = table[page] * p + off
            slots.extend(range(base, base + run))
            pos += run
        return slots
