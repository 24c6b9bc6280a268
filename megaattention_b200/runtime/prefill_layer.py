"""Serving-engine-facing wrapper of one layer's attention output path.

The reference describes this layer in its design notes (docs/design/
causal_varlen_prefill_persistent_fa_oproj_ar_plan_zh.md:959-1048 "host wrapper and launch
metadata", :1266-1283 "serving-engine interface constraints") and calls the workspace "the
sglang-facing runtime resource contract" (src/mega_attention/runtime/workspace.py:5); it
ships no code for it.  The contract built here:

* one ``FusedPrefillLayer`` per transformer layer, created once: it keeps the layer's
  ``W_o`` on the device in the layout the kernel reads (``[K_local, width]`` with
  ``width % 64 == 0``, columns past ``hidden`` zero), so nothing about the weight moves per
  step;
* per step the engine hands over what it already has — packed ``q [tot_q, H_local, D]`` and
  either packed ``k / v [tot_k, H_kv, D]`` with ``cu_seqlens_k`` (contiguous variant) or
  its token-pool KV cache with ``page_table [batch, max_pages_per_seq] int32`` and
  ``cache_seqlens [batch] int32`` (paged variant, page size 128: the cache is viewed as
  ``[-1, 128, H_kv, D]``) — and the kernel reads all of it in place.  Only the varlen tile
  descriptors (a few KB) are uploaded;
* the two KV layouts are two workspaces (``create(paged=...)``); a layer object is tied to
  one of them and refuses the other's arguments, a page size other than 128, a page table
  that is too narrow for the longest sequence, or a wrong dtype, before anything is queued;
* many layers share one workspace (the kernel's exit path leaves the control state clean,
  so there is no host reset between layers);
* the launch flags and the attention claim order are chosen per step from the batch at hand
  by the workspace (``launch_flags_b200``, ``fa_prime_tiles_b200``) unless the caller passes
  ``flags`` or pins ``ws.default_flags`` / ``ws.fa_prime_tiles``.
"""
from __future__ import annotations

import numpy as np
import torch

from ..metadata.row_desc import build_row_desc


def _seqlens(cu):
    cu = np.asarray(cu.cpu() if torch.is_tensor(cu) else cu, dtype=np.int64)
    assert cu.ndim == 1 and cu.size >= 2 and cu[0] == 0, "cu_seqlens must start at 0"
    return np.diff(cu)


class FusedPrefillLayer:
    def __init__(self, workspace, W_o):
        """``W_o [K_local, hidden]`` (input-major, i.e. ``nn.Linear.weight.T``), host or
        device.  Copied to the device once, padded to a multiple of 64 columns."""
        ws = workspace
        assert ws._plan is not None, "compile() the workspace first"
        assert tuple(W_o.shape) == (ws.K_local, ws.hidden) and W_o.dtype == ws.dtype
        width = (ws.hidden + 63) // 64 * 64
        if W_o.is_cuda and W_o.device == ws.dev and width == ws.hidden and W_o.is_contiguous():
            self.W_o = W_o
        else:
            self.W_o = torch.zeros(ws.K_local, width, dtype=ws.dtype, device=ws.dev)
            self.W_o[:, :ws.hidden].copy_(W_o)
        self.ws = workspace
        self.meta = None

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_k=None, *, page_table=None,
                cache_seqlens=None, page_size=128, flags=None):
        """Queue one fused launch on the workspace's stream and return the tile-padded
        output ``csym [R, 128, num_out, 128]`` (valid until the workspace's next launch;
        ``output()`` gives the de-tiled ``[tot_q, hidden]`` copy).

        Contiguous variant: ``k, v [tot_k, H_kv, D]`` and ``cu_seqlens_k`` (None: same as q).
        Paged variant: ``k, v`` are the KV caches, either ``[num_pages, 128, H_kv, D]`` or
        the token pool ``[num_slots, H_kv, D]`` with ``num_slots % 128 == 0``.
        """
        ws = self.ws
        lens_q = _seqlens(cu_seqlens_q)
        if ws.paged:
            assert page_table is not None and cache_seqlens is not None, \
                "a paged workspace needs page_table and cache_seqlens"
            assert cu_seqlens_k is None, "paged KV takes its lengths from cache_seqlens"
            assert page_size == 128, f"page size {page_size}: only 128 (one key block) is supported"
            for name, t in (("page_table", page_table), ("cache_seqlens", cache_seqlens)):
                assert torch.is_tensor(t) and t.dtype == torch.int32, f"{name} must be int32"
            if k.dim() == 3:                     # token pool -> pages of 128 slots
                assert k.shape[0] % 128 == 0 and v.shape == k.shape
                k = k.view(-1, 128, ws.H_kv, ws.D)
                v = v.view(-1, 128, ws.H_kv, ws.D)
            lens_k = cache_seqlens.cpu().numpy().astype(np.int64)
            assert page_table.dim() == 2 and page_table.shape[0] == lens_q.size == lens_k.size
            assert page_table.shape[1] >= int((-(-lens_k // 128)).max()), \
                "page_table is narrower than the longest sequence needs"
        else:
            assert page_table is None and cache_seqlens is None, \
                "page_table / cache_seqlens need a workspace created with paged=True"
            lens_k = lens_q if cu_seqlens_k is None else _seqlens(cu_seqlens_k)
        meta = build_row_desc(lens_q, seqlens_k=lens_k)      # asserts 0 < q_len <= k_len
        ws.bind_inputs(meta, q, k, v, self.W_o, page_table=page_table, cache_seqlens=cache_seqlens)
        ws.launch(flags)
        self.meta = meta
        return ws.csym[:meta.num_row_tiles]

    __call__ = forward

    def output(self):
        """De-tiled ``[tot_q, hidden]`` copy of the last launch's result."""
        return self.ws.output(self.meta)
