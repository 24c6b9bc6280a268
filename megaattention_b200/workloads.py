"""The benchmark / parity workloads and their seeded synthetic inputs.

The reference measures on synthetic random tensors (benchmarks/
bench_fused_fa_oproj_ar.py:158-200 builds them inline); c1-c5 are five configurations of
that kind (a CPU-sized case, the per-rank shape of an 8-way split 64-head model, its
tensor-parallel sweep, a large-hidden case and a chunked-prefill case), long16k / long32k
are the single-sequence shapes on which the reference's own sweep falls below its unfused
baseline (benchmarks/sweep_results.md:11-14).  Inputs are drawn on the CPU with a
seeded ``torch.Generator`` in fp32 and cast to bf16, so that a CPU checker and the GPU
see identical bits.

Layouts follow the reference: ``Q [tot_q, H_local, D]``, ``K/V [tot_k, H_kv, D]``,
``W_o [K_local, hidden]`` (input-major, i.e. ``nn.Linear.weight.T``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

D_HEAD = 128


@dataclass
class Workload:
    name: str
    seqlens_q: List[int]
    q_heads_global: int          # across all tensor-parallel ranks
    kv_heads_global: int
    hidden: int
    tp_sizes: List[int]
    kv_mult: int = 1             # k_len = kv_mult * q_len (chunked prefill when > 1)
    w_fan_in: Optional[int] = None   # std of W_o is w_fan_in ** -0.5
    per_rank_seed: bool = False  # shapes given per rank: draw each rank independently
    note: str = ""
    seqlens_k: List[int] = field(init=False)

    def __post_init__(self):
        self.seqlens_k = [self.kv_mult * s for s in self.seqlens_q]
        if self.w_fan_in is None:
            self.w_fan_in = self.q_heads_global * D_HEAD

    @property
    def tot_q(self):
        return sum(self.seqlens_q)

    @property
    def tot_k(self):
        return sum(self.seqlens_k)

    def heads_local(self, tp):
        assert self.q_heads_global % tp == 0
        h = self.q_heads_global // tp
        hkv = max(1, self.kv_heads_global // tp)
        return h, hkv


_SWEEP = [7500, 4100, 3300, 2600, 2000, 1500, 1000, 600]
_SMALL = [6800, 2900, 1700, 1100, 600, 300]

WORKLOADS = {
    # CPU-runnable case: B=3, 8 q heads / 1 kv head, hidden 1024, one rank.
    "c1": Workload("c1", [64, 200, 256], 8, 1, 1024, [1]),
    # One GPU, the per-rank shape of an 8-way split 64q/8kv model, hidden 4096.
    "c2": Workload("c2", _SMALL, 8, 1, 4096, [1]),
    # Tensor-parallel sweep over a fixed global model (64 q / 8 kv heads).
    "c3": Workload("c3", _SWEEP, 64, 8, 4096, [1, 2, 4, 8]),
    # Large hidden, AllReduce bound: per rank 16 q / 1 kv heads, hidden 16384, 8 ranks.
    "c4": Workload("c4", _SWEEP, 128, 8, 16384, [8], per_rank_seed=True),
    # Chunked prefill, k = 4 q, per rank 8 q / 1 kv heads, 8 ranks.
    "c5": Workload("c5", _SMALL, 64, 8, 4096, [8], kv_mult=4, w_fan_in=1024,
                   per_rank_seed=True),
    # One long sequence, 8 q / 1 kv heads, hidden 2048, one rank: the tail of the launch is
    # one chain of ever longer attention tasks per head.
    # c2 with a kv head per q head: attention tasks pair heads that share no K/V.
    "c2_mha": Workload("c2_mha", _SMALL, 8, 8, 4096, [1]),
    "long16k": Workload("long16k", [16384], 8, 1, 2048, [1]),
    "long32k": Workload("long32k", [32768], 8, 1, 2048, [1]),
}


def _randn(shape, seed, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    x = torch.randn(shape, generator=g, dtype=torch.float32)
    if std != 1.0:
        x *= std
    return x.to(torch.bfloat16)


def make_rank_inputs(wl: Workload, tp: int, rank: int, seed: int = 0):
    """``(Q, K, V, W_o)`` bf16 CPU tensors of one rank.

    Global-model workloads draw the whole model once per tensor (seeds
    ``seed*1000 + {0,1,2,3}``) and slice contiguous head ranges, which keeps
    ``kv_head = q_head // q_per_kv`` consistent across tp sizes and makes every tp size
    comparable with one checker run.  Per-rank workloads add ``10 * rank`` to the seed.
    """
    h, hkv = wl.heads_local(tp)
    k_local = h * D_HEAD
    std_w = float(wl.w_fan_in) ** -0.5
    base = seed * 1000
    if wl.per_rank_seed:
        base += 10 * rank
        Q = _randn((wl.tot_q, h, D_HEAD), base + 0)
        K = _randn((wl.tot_k, hkv, D_HEAD), base + 1)
        V = _randn((wl.tot_k, hkv, D_HEAD), base + 2)
        W = _randn((k_local, wl.hidden), base + 3, std_w)
        return Q, K, V, W
    Qg = _randn((wl.tot_q, wl.q_heads_global, D_HEAD), base + 0)
    Kg = _randn((wl.tot_k, wl.kv_heads_global, D_HEAD), base + 1)
    Vg = _randn((wl.tot_k, wl.kv_heads_global, D_HEAD), base + 2)
    Wg = _randn((wl.q_heads_global * D_HEAD, wl.hidden), base + 3, std_w)
    Q = Qg[:, rank * h:(rank + 1) * h].contiguous()
    kv_lo = (rank * wl.kv_heads_global) // tp if wl.kv_heads_global >= tp else 0
    K = Kg[:, kv_lo:kv_lo + hkv].contiguous()
    V = Vg[:, kv_lo:kv_lo + hkv].contiguous()
    W = Wg[rank * k_local:(rank + 1) * k_local].contiguous()
    return Q, K, V, W


def fa_flops(seqlens_q, H_local, D, seqlens_k=None):
    """Causal (bottom-right) QK^T + PV FLOPs, un-padded
    (benchmarks/bench_fused_fa_oproj_ar.py:113-123)."""
    sk = seqlens_q if seqlens_k is None else seqlens_k
    total = 0.0
    for lq, lk in zip(seqlens_q, sk):
        pairs = lq * (lk - lq) + lq * (lq + 1) / 2
        total += H_local * 2 * pairs * (2 * D)
    return float(total)


def oproj_flops(tot_q, K_local, hidden):
    """benchmarks/bench_fused_fa_oproj_ar.py:126-127."""
    return float(2 * tot_q * K_local * hidden)


def ar_bytes(tot_q, hidden, dtype_bytes=2):
    """benchmarks/bench_fused_fa_oproj_ar.py:130-131."""
    return float(tot_q * hidden * dtype_bytes)
