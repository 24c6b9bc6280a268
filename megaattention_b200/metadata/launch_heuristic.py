"""Launch heuristic: role weights and super-group size from the FA / O_proj MAC ratio.

Mirror of the reference ``src/mega_attention/metadata/launch_heuristic.py``
(``estimate_work_ratio`` :21-25, ``LaunchConfig`` :28-33, ``choose_launch_config``
:36-47).  Outputs are bit-identical to the reference, including its two quirks:
the ratio counts ``m_block + 1`` KV blocks per tile and so ignores any KV prefix of
chunked prefill, and ``num_sms`` is accepted but unused.

``choose_launch_config_b200`` is an additional entry point (no reference counterpart)
that accounts for the KV prefix; the reference-compatible function is left untouched.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .row_desc import cdiv

# Ratio at which the table switches from the balanced row to the FA-heavy row.
_R_LO = 2.0
# (w_fa, w_oproj, sg) below / at-or-above the switch point.
_TABLE = ((2, 1, 4), (8, 1, 4))


def estimate_work_ratio(meta, hidden: int, N_TILE: int = 128) -> float:
    """``2 * sum(m_block + 1) / (num_row_tiles * ceil(hidden / N_TILE))``.

    The integer sum is taken in int64 and the quotient is one Python true division,
    which is what makes the value reproducible bit for bit.
    """
    kv_blocks = int(np.add.reduce(meta.m_block.astype(np.int64) + 1))
    return (2 * kv_blocks) / (meta.num_row_tiles * cdiv(hidden, N_TILE))


@dataclass
class LaunchConfig:
    w_fa: int
    w_oproj: int
    w_ar: int
    sg: int


def choose_launch_config(meta, hidden: int, tp_size: int,
                         N_TILE: int = 128, num_sms: int = 132) -> LaunchConfig:
    """Two-bucket table lookup on the work ratio; ``w_ar`` is 0 on a single rank."""
    row = _TABLE[0] if estimate_work_ratio(meta, hidden, N_TILE) < _R_LO else _TABLE[1]
    sg = max(1, min(row[2], cdiv(hidden, N_TILE)))
    return LaunchConfig(w_fa=row[0], w_oproj=row[1], w_ar=int(tp_size > 1), sg=sg)


def estimate_work_ratio_kv(meta, hidden: int, N_TILE: int = 128) -> float:
    """Work ratio that counts the KV blocks a tile really visits (prefix included)."""
    M = meta.M_TILE
    b = meta.batch_idx.astype(np.int64)
    lq = np.diff(meta.cu_seqlens_q.astype(np.int64))[b]
    lk = np.diff(meta.cu_seqlens_k.astype(np.int64))[b]
    last_row = (meta.m_block.astype(np.int64) + 1) * M + (lk - lq)
    nblk = np.minimum(-(-lk // M), -(-last_row // M))
    return (2 * int(nblk.sum())) / (meta.num_row_tiles * cdiv(hidden, N_TILE))


def choose_launch_config_b200(meta, hidden: int, tp_size: int,
                              N_TILE: int = 128) -> LaunchConfig:
    """Same table, indexed by the KV-aware ratio, on one rank.  Not part of the reference
    surface.  With tp > 1 the balanced row is kept whatever the ratio: in the 8-GPU sweep
    the attention-heavy row leaves too few CTAs that look for AllReduce work first (k = 4q
    benchmark shape, tp 8: (8,1,1) 1.115 ms against (2,1,1) 1.099 ms, and 1.061 against
    1.050 ms with "downstream work first"; on the q = k shapes it is the slowest row)."""
    kv_heavy = estimate_work_ratio_kv(meta, hidden, N_TILE) >= _R_LO
    row = _TABLE[1] if (kv_heavy and tp_size <= 1) else _TABLE[0]
    sg = max(1, min(row[2], cdiv(hidden, N_TILE)))
    return LaunchConfig(w_fa=row[0], w_oproj=row[1], w_ar=int(tp_size > 1), sg=sg)


def _allreduce_over_compute(meta, hidden: int, tp_size: int, H_local: int, D: int = 128) -> float:
    """Estimated AllReduce time over estimated tensor time of one rank: the AllReduce payload
    at the ~0.38 TB/s the in-switch reduction sustains on 8 B200s against the un-padded FLOPs
    at an effective 1.2 PFLOP/s.  0 on one rank."""
    if tp_size <= 1:
        return 0.0
    lq = np.diff(meta.cu_seqlens_q.astype(np.int64)).astype(np.float64)
    lk = np.diff(meta.cu_seqlens_k.astype(np.int64)).astype(np.float64)
    fa = float((H_local * 2.0 * (lq * (lk - lq) + lq * (lq + 1) / 2) * (2 * D)).sum())
    tot_q = float(lq.sum())
    flops = fa + 2.0 * tot_q * H_local * D * hidden
    return (tot_q * hidden * 2.0 / 0.38e12) / (flops / 1.2e15)


def fa_prime_tiles_b200(meta, hidden: int, tp_size: int, H_local: int, D: int = 128) -> int:
    """Attention claim order for the sm_100a kernel (``workspace.claim_order``; no reference
    counterpart): 0 = longest row tile first, -1 = long and short row tiles interleaved.

    Interleaved while O_proj is a sizeable share of the work (KV-aware ratio below the
    table's switch point): row tiles then finish at an even rate from the start, so O_proj
    (and AllReduce) work flows all along instead of piling up behind the attention.  Where
    attention dominates, the longest tasks have to start first and the interleaved order
    loses.  Measured, interleaved over longest-first: one GPU, ratio < 2 (the benchmark's c2
    shape, 2048 x 8, 1024 x 4, 4096 x 2): 0.92-0.98; ratio >= 2 (8192 and longer, k = 4q):
    1.01-1.20; c3 at tp 8: 0.95, tp 4: 0.976, tp 2: 1.004; k = 4q at tp 8: 1.09."""
    return -1 if estimate_work_ratio_kv(meta, hidden) < _R_LO else 0


def launch_flags_b200(meta, hidden: int, tp_size: int, H_local: int, D: int = 128) -> int:
    """Launch flags for the sm_100a kernel (no reference counterpart).

    Returns 2 ("drain first": CTAs probe O_proj before attention, AllReduce first on the
    AllReduce-role CTAs) when the launch is expected to be NVLink bound, and on 8 ranks
    always, else 0.  The estimate compares the un-padded FLOPs at an effective 1.2 PFLOP/s
    with the AllReduce payload at the ~0.38 TB/s the in-switch reduction sustains on 8
    B200s.  Measured: tp 8 — c3 0.648 against 0.672 ms, k = 4q shape (ratio 0.36) 1.050
    against 1.099 ms; tp 4, c3 (ratio 0.75): 0.944 against 0.940 ms, within noise.
    """
    if tp_size >= 8:
        return 2
    return 2 if _allreduce_over_compute(meta, hidden, tp_size, H_local, D) > 0.8 else 0


def num_ctas_b200(meta, hidden: int, tp_size: int, H_local: int, num_sms: int = 148) -> int:
    """CTA count for the sm_100a kernel (no reference counterpart; the reference hard-codes
    132).  One persistent CTA per SM: the calibration sweep
    (``metadata/sweep_launch_config.py``) found no shape on which leaving SMs idle won."""
    return int(num_sms)
