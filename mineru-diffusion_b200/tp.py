"""Tensor-parallel pair (TP = 2): peer buffers, handle exchange, weight shards.

What ``RowParallelLinear`` does with ``dist.all_reduce`` in the reference
(nanovllm/layers/linear.py:153-157) is done here inside the o_proj / down_proj
GEMM: its epilogue stores the rank's fp32 k-slices into the peer GPU's slice
buffer over NVLink and raises a flag there; the consumer kernel waits for the
flag and sums both ranks' slices in a fixed order.  This module owns the
memory that makes that possible: one region per rank allocated with
``mdb_tp_alloc`` (so it can be exported as an IPC handle), laid out as

    [o slices  2*S_o*64*H fp32][down slices 2*S_d*64*H fp32][LM-head records][flag slots 3*256 u32]

Both ranks use the same offsets; rank r writes index r of every pair.
One process per GPU; the handles travel through ``torch.distributed``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import replace

import torch
import torch.distributed as dist

from . import _lib
from .engine.config import DecoderConfig

FLAG_SLOTS = 256


class _RawCuda:
    """CUDA-array-interface holder so torch can view memory it did not allocate."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _align(v: int, a: int = 256) -> int:
    return (v + a - 1) // a * a


def shard_config(cfg: DecoderConfig, world: int) -> DecoderConfig:
    """Per-rank decoder dimensions: heads and MLP columns divided, hidden size kept
    (nanovllm/models/sdar.py:26-32, nanovllm/layers/linear.py:54-151)."""
    if cfg.num_attention_heads % world or cfg.num_key_value_heads % world or cfg.intermediate_size % world:
        raise ValueError("heads and intermediate size must divide by the tensor-parallel size")
    return replace(cfg, num_attention_heads=cfg.num_attention_heads // world,
                   num_key_value_heads=cfg.num_key_value_heads // world,
                   intermediate_size=cfg.intermediate_size // world)


def shard_weights(full, cfg: DecoderConfig, rank: int, world: int):
    """The rank's slice of a full weight set, cut the way the reference's weight
    loaders cut it: q|k|v rows by head, o_proj columns by head, gate|up rows,
    down_proj columns.  Embedding and LM head stay whole (the LM head is read by
    vocabulary tile range)."""
    from .decoder import DecoderWeights, LayerWeights
    d = cfg.head_dim
    hq, hkv, inter = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    q_rows, kv_rows, i_rows = hq * d // world, hkv * d // world, inter // world
    layers = []
    for l in full.layers:
        q, k, v = l.qkv.split([hq * d, hkv * d, hkv * d], dim=0)
        qkv = torch.cat([q[rank * q_rows:(rank + 1) * q_rows], k[rank * kv_rows:(rank + 1) * kv_rows],
                         v[rank * kv_rows:(rank + 1) * kv_rows]], dim=0).contiguous()
        o = l.o[:, rank * q_rows:(rank + 1) * q_rows].contiguous()
        gate, up = l.gate_up.split([inter, inter], dim=0)
        gate_up = torch.cat([gate[rank * i_rows:(rank + 1) * i_rows], up[rank * i_rows:(rank + 1) * i_rows]],
                            dim=0).contiguous()
        down = l.down[:, rank * i_rows:(rank + 1) * i_rows].contiguous()
        layers.append(LayerWeights(l.input_ln, qkv, l.q_norm, l.k_norm, o, l.post_ln, gate_up, down))
    return DecoderWeights(full.embed, layers, full.final_ln, full.lm_head)


def lm_head_split(vocab: int, rank: int, many_rows: bool) -> tuple[int, int, int]:
    """Share of the LM head a rank of the pair scans, in 128-column tiles of the vocabulary:
    (first tile, tiles, columns the peer scans).  Short steps (at most 64 rows) split the tiles evenly; steps of
    more rows run a kernel whose records cover 256 columns, so rank 0's share ends on a 256-column boundary and
    rank 1 takes the rest up to the end of the vocabulary.  A share can be empty for a tiny vocabulary."""
    tiles = vocab // 128
    if many_rows:
        first = min(2 * ((-(-vocab // 256) + 1) // 2), tiles)
    else:
        first = (tiles + 1) // 2
    begin, count = (0, first) if rank == 0 else (first, tiles - first)
    return begin, count, (tiles - count) * 128


class TensorParallelPair:

    def __init__(self, rank: int, device, hidden: int, ks_o: int, ks_down: int, lm_ws_bytes: int, max_rows: int = 64,
                 many_rows: int = 0):
        if not dist.is_initialized() or dist.get_world_size() != 2:
            raise RuntimeError("TensorParallelPair needs an initialised process group of size 2")
        self.rank, self.peer_rank, self.device = rank, 1 - rank, torch.device(device)
        self.hidden, self.ks_o, self.ks_down = hidden, ks_o, ks_down
        lib = _lib.lib()
        self.off_o = 0
        self.off_down = _align(self.off_o + 2 * ks_o * max_rows * hidden * 4)
        self.off_lm = _align(self.off_down + 2 * ks_down * max_rows * hidden * 4)
        # many-row steps: one landing buffer per exchange of a layer (o_proj, down_proj), [many_rows, hidden] bf16,
        # that only the peer writes
        self.many_rows = many_rows
        self.off_land = _align(self.off_lm + lm_ws_bytes)
        self.off_flags = _align(self.off_land + 2 * many_rows * hidden * 2)
        self.lm_ws_bytes = lm_ws_bytes
        self.nbytes = self.off_flags + 3 * FLAG_SLOTS * 4
        base = C.c_void_p()
        _lib.check(lib.mdb_tp_alloc(self.nbytes, C.byref(base)), "mdb_tp_alloc")
        self.base = int(base.value)
        self.local = torch.as_tensor(_RawCuda(self.base, self.nbytes), device=self.device)
        handle = (C.c_ubyte * 64)()
        _lib.check(lib.mdb_tp_export(self.base, handle), "mdb_tp_export")
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
        both = [torch.empty_like(mine) for _ in range(2)]
        dist.all_gather(both, mine)
        peer_handle = (C.c_ubyte * 64)(*both[self.peer_rank].cpu().tolist())
        peer = C.c_void_p()
        _lib.check(lib.mdb_tp_import(peer_handle, C.byref(peer)), "mdb_tp_import")
        self.peer_base = int(peer.value)
        dist.barrier()

    # --- addresses -------------------------------------------------------------
    def _slices(self, off: int, ks: int, m: int):
        """(local [2*ks, m, H] fp32 view, my local pointer, my pointer in the peer's region)."""
        n = self.hidden
        view = self.local[off:off + 2 * ks * m * n * 4].view(torch.float32).view(2 * ks, m, n)
        mine = self.rank * ks * m * n * 4
        return view, self.base + off + mine, self.peer_base + off + mine

    def o_slices(self, m: int):
        return self._slices(self.off_o, self.ks_o, m)

    def down_slices(self, m: int):
        return self._slices(self.off_down, self.ks_down, m)

    def landing(self, which: int, m: int):
        """(local [m, H] bf16 view the peer's GEMM stores into, the matching address in the peer's region)."""
        off = self.off_land + which * self.many_rows * self.hidden * 2
        view = self.local[off:off + m * self.hidden * 2].view(torch.bfloat16).view(m, self.hidden)
        return view, self.peer_base + off

    def flags(self, which: int) -> tuple[int, int]:
        """(local slots the peer writes, slots in the peer's region this rank writes)."""
        off = self.off_flags + which * FLAG_SLOTS * 4
        return self.base + off, self.peer_base + off

    def lm_workspace(self) -> tuple[torch.Tensor, int]:
        return self.local[self.off_lm:self.off_lm + self.lm_ws_bytes], self.peer_base + self.off_lm

    def close(self):
        lib = _lib.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier()
        lib.mdb_tp_release(self.peer_base)
        dist.barrier()
        self.local = None
        lib.mdb_tp_free(self.base)
