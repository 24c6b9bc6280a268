"""Rotary position embedding on the packed varlen Q and the new rows of K, in place.

The producer-side op of the fused launch: the reference lists the "QKV-proj / RoPE producer"
as a step it has not built (README.md:41-44 of the reference).  The projection is a plain
library GEMM; the rotation is one HBM-bound CUDA kernel behind the C ABI (``ma_rope_qk``)::

    qkv = x @ W_qkv                                   # library GEMM
    q, k_new, v_new = split(qkv)                      # packed [tot_q, H, 128] ...
    rope_qk_(q, k, cu_seqlens_q, cu_seqlens_k)        # k: [tot_k, H_kv, 128], new rows in place
    layer(q, k, v, cu_seqlens_q, cu_seqlens_k)        # FusedPrefillLayer

Query row ``i`` of sequence ``b`` sits at position ``(k_len_b - q_len_b) + i``; the K rows
rotated are the last ``q_len_b`` rows of the sequence (the prefix of a chunked prefill was
rotated when it was written).  Rotate-half convention, ``inv_freq = theta ** (-arange(0, 128,
2) / 128)`` in fp32 unless given, fp32 angles and products, one rounding
(``oracle/producer_oracle.py`` states the same arithmetic on the CPU).
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from .. import _cabi


def default_inv_freq(theta: float = 10000.0, device=None):
    return 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32, device=device) / 128.0))


def rope_meta(cu_seqlens_q, cu_seqlens_k=None, device="cuda"):
    """Device copy of the three small index arrays one step needs (cu_q | cu_k | sequence of
    every packed query row); build it once per step and pass it to every layer's call."""
    cu_q = np.asarray(cu_seqlens_q.cpu() if torch.is_tensor(cu_seqlens_q) else cu_seqlens_q, dtype=np.int64)
    cu_k = cu_q if cu_seqlens_k is None else np.asarray(
        cu_seqlens_k.cpu() if torch.is_tensor(cu_seqlens_k) else cu_seqlens_k, dtype=np.int64)
    lq, lk = np.diff(cu_q), np.diff(cu_k)
    assert cu_q[0] == 0 and cu_k[0] == 0 and lq.size == lk.size
    assert (lq > 0).all() and (lq <= lk).all(), "0 < q_len <= k_len per sequence"
    meta = np.concatenate([cu_q, cu_k, np.repeat(np.arange(lq.size), lq)]).astype(np.int32)
    return torch.from_numpy(meta).to(device), int(lq.size + 1), int(cu_q[-1]), int(cu_k[-1])


def rope_qk_(q, k, cu_seqlens_q=None, cu_seqlens_k=None, *, theta: float = 10000.0, inv_freq=None,
             meta=None):
    """In place on ``q [tot_q, H, 128]`` and ``k [tot_k, H_kv, 128]`` (bf16, contiguous, CUDA).
    ``cu_seqlens_*`` are host arrays or tensors (int), ``cu_seqlens_k=None`` means q = k; or
    pass ``meta=rope_meta(...)`` built once for the step.  Queued on the current stream."""
    assert q.is_cuda and k.is_cuda and q.device == k.device
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16
    assert q.dim() == 3 and k.dim() == 3 and q.shape[2] == 128 and k.shape[2] == 128
    assert q.is_contiguous() and k.is_contiguous()
    dev = q.device
    assert meta is not None or cu_seqlens_q is not None, "pass cu_seqlens_q (and _k) or meta=rope_meta(...)"
    meta_d, nb, tot_q, tot_k = meta if meta is not None else rope_meta(cu_seqlens_q, cu_seqlens_k, dev)
    assert tot_q == q.shape[0] and tot_k == k.shape[0] and meta_d.device == dev
    w = default_inv_freq(theta, dev) if inv_freq is None else inv_freq.to(dev, torch.float32).contiguous()
    assert tuple(w.shape) == (64,)
    st = torch.cuda.current_stream(dev)
    base = meta_d.data_ptr()
    a = _cabi.RopeArgs(q.data_ptr(), k.data_ptr(), base, base + 4 * nb, base + 8 * nb, w.data_ptr(),
                       int(q.shape[0]), int(q.shape[1]), int(k.shape[1]), 0)
    _cabi.check(_cabi.lib.ma_rope_qk(C.byref(a), C.c_void_p(st.cuda_stream)), "ma_rope_qk")
    return q, k      # (w was allocated on this stream: reuse after free is stream-ordered)


def _benchmark():
    import json
    import os
    from ..workloads import WORKLOADS
    dev = torch.device("cuda:0")
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                         "MEASURED_PEAKS.json")
    hbm = json.load(open(peaks)).get("hbm_gbs") if os.path.exists(peaks) else None
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    for name, H, Hkv in (("c2", 8, 1), ("c3", 16, 2), ("c3", 64, 8)):
        wl = WORKLOADS[name]
        cu = np.concatenate([[0], np.cumsum(wl.seqlens_q)])
        tot = int(cu[-1])
        q = torch.randn(tot, H, 128, device=dev, dtype=torch.bfloat16)
        k = torch.randn(tot, Hkv, 128, device=dev, dtype=torch.bfloat16)
        ms = []
        meta = rope_meta(cu, None, dev)
        w = default_inv_freq(10000.0, dev)
        for i in range(8):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            st = torch.cuda.current_stream(dev)
            a.record(st)
            rope_qk_(q, k, meta=meta, inv_freq=w)
            b.record(st)
            torch.cuda.synchronize()
            if i >= 3:
                ms.append(a.elapsed_time(b))
        t = sum(ms) / len(ms)
        gb = tot * (H + Hkv) * 128 * 2 * 2 / 1e9
        print(json.dumps({"op": "rope_qk", "workload": name, "tokens": tot, "heads": [H, Hkv], "ms": t,
                          "algorithmic_GB": gb, "GB/s": gb / t * 1e3,
                          "frac_of_measured_hbm": (gb / t * 1e3 / hbm) if hbm else None}))


if __name__ == "__main__":
    _benchmark()
