"""Continuous-batching scheduler with the block-diffusion state machine.

Mirrors ``engines/nano_dvlm/nanovllm/engine/scheduler.py``: waiting requests
are prefetched into one prefill batch while pages and the token budget last;
otherwise every running request (RUNNING or CACHING alike) joins the decode
batch, pre-empting from the tail when pages run out.  ``postprocess`` moves a
request to CACHING once its block holds no mask, and after the CACHING pass
appends the block and either finishes the request or reopens a masked block.
"""
from __future__ import annotations

from collections import deque

import numpy as np
import torch

from .block_manager import BlockManager
from .sequence import Sequence, SequenceStatus


class Scheduler:

    def __init__(self, config):
        self.max_num_seqs = config.max_num_seqs
        self.max_num_batched_tokens = config.max_num_batched_tokens
        self.eos = config.eos
        self.block_manager = BlockManager(config.num_kvcache_blocks, config.kvcache_block_size)
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add(self, seq: Sequence):
        self.waiting.append(seq)

    def schedule(self) -> tuple[list[Sequence], bool]:
        picked: list[Sequence] = []
        budget = 0
        while self.waiting and len(picked) < self.max_num_seqs:
            seq = self.waiting[0]
            if budget + len(seq) > self.max_num_batched_tokens or not self.block_manager.can_allocate(seq):
                break
            self.block_manager.allocate(seq)
            budget += len(seq) - seq.num_cached_tokens
            seq.status = SequenceStatus.RUNNING
            self.running.append(self.waiting.popleft())
            picked.append(seq)
        if picked:
            return picked, True

        while self.running and len(picked) < self.max_num_seqs:
            seq = self.running.popleft()
            evicted_self = False
            while not self.block_manager.can_append(seq):
                if self.running:
                    self.preempt(self.running.pop())
                else:
                    self.preempt(seq)
                    evicted_self = True
                    break
            if not evicted_self:
                self.block_manager.may_append(seq)
                picked.append(seq)
        if not picked:
            raise AssertionError("no request could be scheduled")
        self.running.extendleft(reversed(picked))
        return picked, False

    def preempt(self, seq: Sequence):
        seq.status = SequenceStatus.WAITING
        self.block_manager.deallocate(seq)
        self.waiting.appendleft(seq)

    def postprocess(self, seqs: list[Sequence]):
        caching = [seq for seq in seqs if seq.is_caching]
        denoising = [seq for seq in seqs if not seq.is_caching]
        if len(denoising) > 4:
            # one comparison for the whole batch: a block with no masked position left goes to its caching pass
            ids = torch.stack([seq.current_denoising_block for seq in denoising]).numpy()
            mask_ids = np.fromiter((seq.mask_token_id for seq in denoising), dtype=np.int64, count=len(denoising))
            masked_left = (ids == mask_ids[:, None]).any(axis=1)
            for i in np.flatnonzero(~masked_left):
                denoising[i].status = SequenceStatus.CACHING
        else:
            for seq in denoising:
                if not bool((seq.current_denoising_block.numpy() == seq.mask_token_id).any()):   # numpy view: no dispatch cost
                    seq.status = SequenceStatus.CACHING
        for seq in caching:
            block_np = seq.current_denoising_block.numpy()
            hit_stop = any(bool((block_np == t).any()) for t in seq.sampling_params.stop_token_ids)
            seq.append_block()
            if (not seq.ignore_eos and hit_stop) or seq.num_completion_tokens >= seq.max_new_tokens:
                seq.status = SequenceStatus.FINISHED
                self.block_manager.deallocate(seq)
                self.running.remove(seq)
            else:
                seq.status = SequenceStatus.RUNNING
            pending, seq.pending_first_step = getattr(seq, "pending_first_step", None), None
            if pending is not None and seq.status is SequenceStatus.RUNNING:
                # the new block's first denoising pass already ran, together with the commit pass
                block, moved = pending
                seq.current_denoising_block = block
                if moved is not None:
                    seq.current_step_map.numpy()[moved] = seq.current_denoise_step
                seq.current_denoise_step += 1
                if not bool((block.numpy() == seq.mask_token_id).any()):
                    seq.status = SequenceStatus.CACHING
