"""Varlen row-tile descriptors and task-space sizes for the fused prefill path.

Host-side mirror of the reference module ``src/mega_attention/metadata/row_desc.py``
(symbols and argument meaning are the same so callers can switch imports):

* ``cu_seqlens_from_seqlens``  — reference ``row_desc.py:47-52``
* ``RowDescMeta`` / ``build_row_desc`` — reference ``row_desc.py:72-141``
* ``oproj_task_counts``        — reference ``row_desc.py:144-153``
* ``active_counts``            — reference ``row_desc.py:156-174``
* ``decode_oproj_slot``        — reference ``row_desc.py:177-185``
* ``oscratch_numel`` / ``csym_numel`` — reference ``row_desc.py:189-206``

Every function returns the same values *and dtypes* as the reference (int32 arrays,
Python ints), which the parity tests check array for array.  The arithmetic is
written with vectorised numpy instead of per-tile Python loops.

One 128-row tile is the unit of work shared by the three stages: a FlashAttention
task is ``row_tile * H_local + head``, an O_proj / AllReduce slot is
``row_tile * num_super_groups + n_super_group``.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

ROW_M_TILE = 128
FA_M_TILE = ROW_M_TILE
OPROJ_M_TILE = ROW_M_TILE
AR_M_TILE = ROW_M_TILE


def cdiv(a: int, b: int) -> int:
    """Ceiling division for non-negative ints."""
    return -(-a // b)


def cu_seqlens_from_seqlens(seqlens) -> np.ndarray:
    """``[B]`` lengths -> ``[B+1]`` exclusive prefix sum, int32, ``cu[0] == 0``.

    The running sum is taken in int64 and narrowed afterwards, like the reference.
    """
    lens = np.asarray(seqlens, dtype=np.int64)
    out = np.zeros(lens.shape[0] + 1, dtype=np.int32)
    out[1:] = np.cumsum(lens, dtype=np.int64).astype(np.int32)
    return out


@dataclass
class RowDescMeta:
    """Flattened 128-row tile schedule of one varlen batch.

    ``t`` below is a flattened row-tile id in ``[0, num_row_tiles)``; tile ``t`` belongs
    to sequence ``batch_idx[t]`` and is that sequence's ``m_block[t]``-th tile.
    """

    num_batch: int
    M_TILE: int
    cu_seqlens_q: np.ndarray
    cu_seqlens_k: np.ndarray
    num_row_tiles: int
    cu_m_blocks: np.ndarray
    batch_idx: np.ndarray
    m_block: np.ndarray

    def q_len(self, t: int) -> int:
        b = int(self.batch_idx[t])
        return int(self.cu_seqlens_q[b + 1]) - int(self.cu_seqlens_q[b])

    def k_len(self, t: int) -> int:
        b = int(self.batch_idx[t])
        return int(self.cu_seqlens_k[b + 1]) - int(self.cu_seqlens_k[b])

    def q_tile_start(self, t: int) -> int:
        b = int(self.batch_idx[t])
        return int(self.cu_seqlens_q[b]) + int(self.m_block[t]) * self.M_TILE

    def valid_m(self, t: int) -> int:
        return min(self.M_TILE, self.q_len(t) - int(self.m_block[t]) * self.M_TILE)


def build_row_desc(seqlens_q, M_TILE: int = ROW_M_TILE, seqlens_k=None) -> RowDescMeta:
    """Build the tile schedule from per-sequence lengths.

    Preconditions (``AssertionError`` otherwise, as in the reference): ``M_TILE == 128``;
    a non-empty 1-D batch; every ``q_len > 0``; ``k_len >= q_len`` per sequence.
    ``seqlens_k=None`` means a complete prompt (``k == q``); ``k > q`` is chunked /
    append prefill with the causal mask aligned bottom-right.  Tiles are counted on Q
    tokens only.
    """
    assert int(M_TILE) == ROW_M_TILE, "the three stages share one 128-row tile"
    lq = np.asarray(seqlens_q, dtype=np.int64)
    assert lq.ndim == 1 and lq.shape[0] > 0
    assert bool((lq > 0).all()), "q_len must be positive"
    lk = lq if seqlens_k is None else np.asarray(seqlens_k, dtype=np.int64)
    assert lk.shape == lq.shape
    assert bool((lk >= lq).all()), "q_len > k_len is not supported (bottom-right causal)"

    tiles_per_seq = (lq + (M_TILE - 1)) // M_TILE
    cu_m = np.zeros(lq.shape[0] + 1, dtype=np.int32)
    cu_m[1:] = np.cumsum(tiles_per_seq, dtype=np.int64).astype(np.int32)
    total = int(cu_m[-1])
    batch_idx = np.repeat(np.arange(lq.shape[0], dtype=np.int32), tiles_per_seq)
    m_block = (np.arange(total, dtype=np.int64)
               - np.repeat(cu_m[:-1].astype(np.int64), tiles_per_seq)).astype(np.int32)
    return RowDescMeta(
        num_batch=int(lq.shape[0]),
        M_TILE=int(M_TILE),
        cu_seqlens_q=cu_seqlens_from_seqlens(lq),
        cu_seqlens_k=cu_seqlens_from_seqlens(lk),
        num_row_tiles=total,
        cu_m_blocks=cu_m,
        batch_idx=batch_idx.astype(np.int32, copy=False),
        m_block=m_block,
    )


def oproj_task_counts(num_row_tiles: int, hidden: int, N_TILE: int,
                      super_group_n_tiles: int):
    """``(num_out_n_tiles, num_super_groups, total_oproj_tasks)`` of the O_proj/AR space."""
    num_out = cdiv(hidden, N_TILE)
    nsg = cdiv(num_out, super_group_n_tiles)
    return num_out, nsg, num_row_tiles * nsg


def active_counts(num_row_tiles: int, H_local: int, num_super_groups: int,
                  tp_size: int, rank: int) -> np.ndarray:
    """The six int32 run-time counts the kernel reads at start:

    ``[num_fa, total_oproj, num_row_tiles, owner_slots, owner_words, local_owned_ar]``.
    Slot ``s`` is owned (all-reduced) by rank ``s % tp_size`` as its
    ``s // tp_size``-th owned slot.
    """
    total = num_row_tiles * num_super_groups
    owner_slots = cdiv(total, tp_size)
    return np.array(
        [num_row_tiles * H_local, total, num_row_tiles, owner_slots,
         cdiv(owner_slots, 64), cdiv(max(total - rank, 0), tp_size)],
        dtype=np.int32)


def decode_oproj_slot(slot_id: int, num_super_groups: int, super_group_n_tiles: int,
                      hidden: int, N_TILE: int):
    """slot id -> ``(row_tile, n_super_group, base_out_n_tile, valid_n_tiles)``."""
    row_tile, nsg = divmod(slot_id, num_super_groups)
    base = nsg * super_group_n_tiles
    valid = min(super_group_n_tiles, cdiv(hidden, N_TILE) - base)
    return row_tile, nsg, base, valid


def oscratch_numel(num_row_tiles: int, H_local: int, D: int,
                   M_TILE: int = ROW_M_TILE) -> int:
    """Elements of the attention-output scratch ``[num_row_tiles, M_TILE, H_local, D]``."""
    return num_row_tiles * M_TILE * H_local * D


def csym_numel(num_row_tiles: int, hidden: int, N_TILE: int,
               M_TILE: int = ROW_M_TILE) -> int:
    """Elements of the tile-padded output ``[num_row_tiles, M_TILE, num_out, N_TILE]``.

    Padding rows (beyond ``valid_m``) and padding columns (beyond ``hidden``) still take
    address space; they are masked at store time.
    """
    return num_row_tiles * M_TILE * cdiv(hidden, N_TILE) * N_TILE
