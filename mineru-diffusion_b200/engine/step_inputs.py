"""Host-side construction of a step's integer inputs (no device work here).

These are the index contracts of the reference's ``ModelRunner.prepare_prefill``
/ ``prepare_decode`` / ``prepare_block_tables``
(``engines/nano_dvlm/nanovllm/engine/model_runner.py:121-185``): token ids,
positions, cache slots, sequence boundaries, context lengths and the -1 padded
page table.  They must be bit-exact, so they are plain integer code that the
CPU tests compare with tensors recorded from the reference.
"""
from __future__ import annotations

import numpy as np

from .sequence import Sequence


def pad_block_tables(seqs: list[Sequence]) -> np.ndarray:
    width = max(len(seq.block_table) for seq in seqs)
    out = np.full((len(seqs), max(width, 1)), -1, dtype=np.int32)
    for i, seq in enumerate(seqs):
        out[i, :len(seq.block_table)] = seq.block_table
    return out[:, :width] if width else out[:, :0]


def build_prefill_inputs(seqs: list[Sequence], block_size: int) -> dict:
    """Packed prompt(+committed blocks)+masked block of every request.
    The masked block's rows get slot -1: prefill does not cache them."""
    ids: list[int] = []
    pos: list[int] = []
    slots: list[int] = []
    cu = [0]
    max_len = 0
    for seq in seqs:
        seqlen = len(seq) + block_size
        ids.extend(seq[seq.num_cached_tokens:])
        ids.extend(seq.current_denoising_block.tolist())
        pos.extend(range(seq.num_cached_tokens, seqlen))
        cu.append(cu[-1] + seqlen - seq.num_cached_tokens)
        max_len = max(max_len, seqlen)
        if not seq.block_table:      # warm-up sequences hold no pages
            continue
        slots.extend(seq.get_slots(seq.num_cached_tokens, len(seq)))
        slots.extend([-1] * block_size)
    return dict(input_ids=np.asarray(ids, dtype=np.int64), positions=np.asarray(pos, dtype=np.int64),
                slot_mapping=np.asarray(slots, dtype=np.int32), cu_seqlens=np.asarray(cu, dtype=np.int32),
                max_seqlen=max_len)


def build_decode_inputs(seqs: list[Sequence], block_size: int) -> dict:
    """The block being denoised of every request against its cached prefix."""
    bs = len(seqs)
    ids = np.empty((bs, block_size), dtype=np.int64)
    pos = np.empty((bs, block_size), dtype=np.int64)
    slots = np.empty((bs, block_size), dtype=np.int32)
    ctx = np.empty(bs, dtype=np.int32)
    for i, seq in enumerate(seqs):
        n = len(seq)
        ids[i] = seq.current_denoising_block.numpy()
        pos[i] = np.arange(n, n + block_size, dtype=np.int64)
        slots[i] = seq.get_slots(n, n + block_size)
        ctx[i] = n + block_size
    return dict(input_ids=ids, positions=pos, slot_mapping=slots, context_lens=ctx,
                block_tables=pad_block_tables(seqs))
