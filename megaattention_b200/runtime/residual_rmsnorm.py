"""Residual add + RMSNorm on the fused launch's output, read in place from ``ws.csym``.

The op that follows the attention output path in a transformer layer: the reference lists
it as the next step after its fused kernel (README.md:41-44 of the reference, "residual /
RMSNorm consumer") and has no code for it.  Here it is one HBM-bound CUDA kernel behind the
C ABI (``ma_residual_rmsnorm``) that takes the tile-padded ``csym`` buffer and the varlen
arrays the workspace already holds on the device, so no de-tiled copy of the attention
output is ever made::

    ws.launch()                                   # or FusedPrefillLayer(...)(...)
    normed, residual = residual_rmsnorm(ws, residual, weight, eps=1e-6)

``h = bf16(y + residual)`` is the new residual stream, ``normed = bf16(h * rsqrt(mean(h^2) +
eps) * weight)`` with the statistics in fp32 (``oracle/consumer_oracle.py`` states the same
arithmetic on the CPU).  Run as a script it times the kernel against the HBM copy rate.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _cabi


def residual_rmsnorm(ws, residual, weight, eps: float = 1e-6, *, out=None, inplace: bool = False,
                     meta=None):
    """``residual [tot_q, hidden]`` and ``weight [hidden]`` bf16 on the workspace's device.
    Returns ``(normed, new_residual)``; with ``inplace`` the residual is updated where it is.
    Queued on the workspace's stream behind the launch that filled ``ws.csym``."""
    meta = meta if meta is not None else ws._meta
    assert meta is not None, "no layer has been set on this workspace"
    tot_q = int(meta.cu_seqlens_q[-1])
    assert residual.is_cuda and residual.device == ws.dev and residual.dtype == torch.bfloat16
    assert tuple(residual.shape) == (tot_q, ws.hidden) and residual.is_contiguous()
    assert tuple(weight.shape) == (ws.hidden,) and weight.dtype == torch.bfloat16
    assert weight.device == ws.dev and weight.is_contiguous()
    normed = out if out is not None else torch.empty_like(residual)
    assert normed.shape == residual.shape and normed.dtype == residual.dtype and normed.is_contiguous()
    new_res = residual if inplace else torch.empty_like(residual)
    a = _cabi.RmsNormArgs(
        ws.csym.data_ptr(), residual.data_ptr(), weight.data_ptr(), new_res.data_ptr(),
        normed.data_ptr(), ws.cu_q.data_ptr(), ws.fa_b.data_ptr(), ws.fa_mb.data_ptr(),
        int(meta.num_row_tiles), int(ws.hidden), int(ws.num_out * 128), float(eps))
    _cabi.check(ws._lib.ma_residual_rmsnorm(C.byref(a), C.c_void_p(ws._stream().cuda_stream)),
                "ma_residual_rmsnorm")
    return normed, new_res


def _benchmark():
    import json
    import os
    from ..metadata import build_row_desc
    from ..workloads import WORKLOADS
    from . import FusedFaOprojArWorkspace
    dev = torch.device("cuda:0")
    peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                         "MEASURED_PEAKS.json")
    hbm = json.load(open(peaks)).get("hbm_gbs") if os.path.exists(peaks) else None
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    for name in ("c2", "c3", "c4"):
        wl = WORKLOADS[name]
        meta = build_row_desc(wl.seqlens_q, seqlens_k=wl.seqlens_k)
        ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, wl.hidden, 2, 128, q_per_kv=2,
                                            max_num_batch=meta.num_batch, max_tot_k=wl.tot_k, device=dev)
        ws.compile()
        ws.set_meta(meta)
        ws.csym.normal_()
        tot_q = int(meta.cu_seqlens_q[-1])
        res = torch.randn(tot_q, wl.hidden, device=dev, dtype=torch.bfloat16)
        w = torch.randn(wl.hidden, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(res)
        ms = []
        for i in range(8):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(ws._stream())
            residual_rmsnorm(ws, res, w, out=out, inplace=True)
            b.record(ws._stream())
            torch.cuda.synchronize()
            if i >= 3:
                ms.append(a.elapsed_time(b))
        t = sum(ms) / len(ms)
        gb = tot_q * wl.hidden * 2 * 4 / 1e9
        print(json.dumps({"op": "residual_rmsnorm", "workload": name, "tokens": tot_q, "hidden": wl.hidden,
                          "ms": t, "algorithmic_GB": gb, "GB/s": gb / t * 1e3,
                          "frac_of_measured_hbm": (gb / t * 1e3 / hbm) if hbm else None}))


if __name__ == "__main__":
    _benchmark()
