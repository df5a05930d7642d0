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
    """The block being denoised of every request against its cached prefix.
    Vectorised over the requests (a step of 64 requests spends more host time
    here than anywhere else otherwise); slot = page_id * page + offset, -1
    where a request holds no page."""
    bs = len(seqs)
    lens = np.fromiter((len(seq) for seq in seqs), dtype=np.int64, count=bs)
    ids = np.stack([seq.current_denoising_block.numpy() for seq in seqs]).astype(np.int64, copy=False)
    pos = lens[:, None] + np.arange(block_size, dtype=np.int64)[None, :]
    tables = pad_block_tables(seqs)
    page = Sequence.kvcache_block_size
    if tables.shape[1] == 0:
        slots = np.full((bs, block_size), -1, dtype=np.int32)
    else:
        page_idx = pos // page
        held = np.fromiter((len(seq.block_table) for seq in seqs), dtype=np.int64, count=bs)
        if bool(((held > 0)[:, None] & (page_idx >= held[:, None])).any()):
            raise IndexError("block position beyond the request's page table")
        page_ids = np.take_along_axis(tables.astype(np.int64), np.minimum(page_idx, tables.shape[1] - 1), axis=1)
        slots = np.where(held[:, None] > 0, page_ids * page + pos % page, -1).astype(np.int32)
    ctx = (lens + block_size).astype(np.int32)
    return dict(input_ids=ids, positions=pos, slot_mapping=slots, context_lens=ctx, block_tables=tables)


_ARANGE64: dict[int, np.ndarray] = {}


def fill_decode_inputs_small(seqs: list[Sequence], block_size: int, ids: np.ndarray, pos: np.ndarray,
                             slots: np.ndarray, ctx: np.ndarray, tab: np.ndarray) -> int:
    """``build_decode_inputs`` for a handful of requests, written straight into the rows of the caller's
    (pinned) arrays: per request a few slice writes instead of a dozen array constructions for the whole batch.
    Same contract (NV/engine/model_runner.py:169-185, NV/engine/sequence.py:117-141): a block spans at most two
    pages; -1 slots for a request that holds no page; IndexError if a position lies beyond the page table.
    Returns the longest context."""
    ar = _ARANGE64.get(block_size)
    if ar is None:
        ar = _ARANGE64[block_size] = np.arange(block_size, dtype=np.int64)
    page = Sequence.kvcache_block_size
    longest = 0
    for i, seq in enumerate(seqs):
        n = len(seq)
        table = seq.block_table
        ids[i] = seq.current_denoising_block.numpy()
        np.add(ar, n, out=pos[i])
        ctx[i] = n + block_size
        longest = max(longest, n + block_size)
        held = len(table)
        if held == 0:
            slots[i] = -1
            tab[i] = -1
            continue
        if held > tab.shape[1]:
            raise AssertionError("page table wider than max_model_len allows")
        tab[i, :held] = table
        tab[i, held:] = -1
        first, off = divmod(n, page)
        run = min(block_size, page - off)
        last = first if run == block_size else first + 1
        if last >= held:
            raise IndexError("block position beyond the request's page table")
        np.add(ar[:run], table[first] * page + off, out=slots[i, :run], casting="unsafe")
        if run < block_size:
            np.add(ar[:block_size - run], table[last] * page, out=slots[i, run:], casting="unsafe")
    return longest
