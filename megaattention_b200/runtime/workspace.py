"""Long-lived workspace of the fused FlashAttention -> O_proj -> AllReduce kernel.

Same surface as the reference's ``FusedFaOprojArWorkspace``
(``src/mega_attention/runtime/workspace.py``): ``create`` (:46-150) allocates every buffer
once at a bucket capacity and, with ``tp_size > 1``, rendezvous-es the symmetric ones;
``compile`` (:174-194) fixes the launch configuration; ``set_layer`` (:197-235) fills the
active prefixes and the six active counts; ``launch`` (:237-240) runs one layer with no
host-side reset in between; ``debug_zero_all`` (:243-248) is for fault localisation only.

Differences a caller can observe:

* nothing is JIT-compiled: ``compile`` builds a plan through the C ABI
  (``ma_plan_create``) and the role weights / CTA count are launch arguments;
* ``set_layer`` validates *every* capacity before copying anything;
* device-side waits are bounded: ``check_status`` raises ``RuntimeError`` when one gave up;
* role weights and CTA count can change per ``compile`` without any rebuild.

torch is used for device memory, streams and (tp > 1) symmetric-memory bootstrap only.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from .. import _cabi
from ..metadata.launch_heuristic import fa_prime_tiles_b200, launch_flags_b200
from ..metadata.row_desc import active_counts, oproj_task_counts

NUM_CTRL = 8
NUM_SYNC = 3
NUM_STATUS = 8


def claim_order(meta, prime: int = 0) -> np.ndarray:
    """Row tiles sorted by the number of 128-key blocks their attention task visits,
    longest first (stable), so the biggest tasks are claimed first and the tail of the
    launch is filled with small ones.  Same on every rank.

    ``prime`` > 0 moves that many of the shortest row tiles to the front: their attention
    finishes within microseconds, so O_proj and AllReduce work exists almost from the start
    of the launch instead of only after the first long attention task (tens of
    microseconds) — worth it when the launch is bound by the AllReduce.  ``prime`` < 0
    interleaves long and short row tiles instead (see below)."""
    M = meta.M_TILE
    b = meta.batch_idx.astype(np.int64)
    lq = np.diff(meta.cu_seqlens_q.astype(np.int64))[b]
    lk = np.diff(meta.cu_seqlens_k.astype(np.int64))[b]
    last_row = (meta.m_block.astype(np.int64) + 1) * M + (lk - lq)
    nblk = np.minimum(-(-lk // M), -(-last_row // M))
    order = np.argsort(-nblk, kind="stable").astype(np.int32)
    if prime < 0:
        # interleaved: longest, shortest, second longest, second shortest, ...  Row tiles
        # then finish at an even rate from the start of the launch (steady O_proj and
        # AllReduce work) while the long tasks still start early; the last tasks claimed are
        # of middling length.
        out = np.empty_like(order)
        half = (order.size + 1) // 2
        out[0::2] = order[:half]
        out[1::2] = order[half:][::-1]
        return out
    prime = int(min(prime, order.size))
    if prime:
        order = np.concatenate([order[order.size - prime:][::-1], order[:order.size - prime]])
    return order


class FusedFaOprojArWorkspace:
    def __init__(self, **kw):
        self.__dict__.update(kw)
        self._plan = None
        self._lib = _cabi.lib
        self._args = None
        self._meta = None
        # Launch flags applied by launch() (OR of _cabi.MA_FLAG_*) and attention claim order
        # (see claim_order).  None = chosen for the batch at hand by the calibrated rules,
        # launch_flags_b200 / fa_prime_tiles_b200; an int pins the setting.
        self.default_flags = None
        self.fa_prime_tiles = None
        self._auto_flags = 0
        self.ar_p2p = True       # tp_size == 2: AllReduce through peer loads instead of multimem

    # ------------------------------------------------------------------ create
    @classmethod
    def create(cls, group_name, max_num_row_tiles, hidden, H_local, D,
               tp_size=1, rank=0, N_TILE=128, super_group_n_tiles=4, q_per_kv=1,
               max_num_batch=None, max_tot_k=None, dtype=torch.bfloat16, device=None,
               paged=False, page_size=128, max_num_pages=None,
               max_num_pages_per_seq=None):
        assert dtype == torch.bfloat16 and D == 128 and N_TILE == 128
        assert H_local % q_per_kv == 0
        assert 1 <= super_group_n_tiles <= 4, "a super-group is at most 512 TMEM columns"
        dev = torch.device(device if device is not None
                           else f"cuda:{torch.cuda.current_device()}")
        H_kv = H_local // q_per_kv
        K_local = H_local * D
        if max_num_batch is None:
            max_num_batch = max_num_row_tiles
        num_out, nsg, max_total = oproj_task_counts(
            max_num_row_tiles, hidden, N_TILE, super_group_n_tiles)
        hidden_pad = num_out * N_TILE
        tot_cap = max_num_row_tiles * 128
        if max_tot_k is None:
            max_tot_k = tot_cap
        # paged KV: K/V live in [num_pages, 128, H_kv, D] caches addressed through a page
        # table; one page is exactly one 128-key block (workspace.py:67-74 of the reference)
        if paged:
            assert page_size == N_TILE == 128, (page_size, N_TILE)
            if max_num_pages is None:
                max_num_pages = (max_tot_k + 127) // 128
            if max_num_pages_per_seq is None:
                max_num_pages_per_seq = (max_tot_k + 127) // 128
        max_owner_slots = (max_total + tp_size - 1) // tp_size
        max_owner_words = (max_owner_slots + 63) // 64

        def zeros(shape, dt):
            return torch.zeros(shape, dtype=dt, device=dev)

        handles = None
        if tp_size > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem

            def sym(shape, dt):
                t = symm_mem.empty(*shape, device=dev, dtype=dt)
                t.zero_()
                return t, symm_mem.rendezvous(t, group_name)

            csym, hC = sym((max_num_row_tiles, 128, num_out, N_TILE), dtype)
            assert hC.has_multicast_support, "NVLS multicast is required for tp_size > 1"
            rco, hRC = sym((max_owner_slots,), torch.uint32)
            rbits, hRB = sym((max_owner_words,), torch.int64)
            nvl, hN = sym((2,), torch.int32)
            csym_mc_ptr = int(hC.multicast_ptr)
            rc_ptrs = [int(hRC.buffer_ptrs[r]) for r in range(tp_size)]
            rb_ptrs = [int(hRB.buffer_ptrs[r]) for r in range(tp_size)]
            nvl_peer_ptrs = [int(hN.buffer_ptrs[r]) for r in range(tp_size)]
            csym_peer_ptrs = [int(hC.buffer_ptrs[r]) for r in range(tp_size)]
            handles = (hC, hRC, hRB, hN)
        else:
            csym = zeros((max_num_row_tiles, 128, num_out, N_TILE), dtype)
            rco = zeros(max_owner_slots, torch.uint32)
            rbits = zeros(max_owner_words, torch.int64)
            nvl = zeros(2, torch.int32)
            csym_mc_ptr = 0
            rc_ptrs, rb_ptrs, nvl_peer_ptrs, csym_peer_ptrs = [], [], [], []

        # varlen metadata: one device buffer, so a layer's descriptors arrive in one copy;
        # cu_q | cu_k | fa_b | fa_mb | fa_order | actv are views at fixed (capacity) offsets,
        # each 16-byte aligned
        def up4(n):
            return (n + 3) // 4 * 4
        sizes = (max_num_batch + 1, max_num_batch + 1, max_num_row_tiles, max_num_row_tiles,
                 max_num_row_tiles, 8)
        offs = [0]
        for n in sizes:
            offs.append(offs[-1] + up4(n))
        meta_dev = zeros(offs[-1], torch.int32)
        mviews = [meta_dev[offs[i]:offs[i] + sizes[i]] for i in range(6)]
        ws = cls(
            dev=dev, dtype=dtype, meta_dev=meta_dev, _meta_offs=offs, tp_size=tp_size, rank=rank, group_name=group_name,
            H_local=H_local, H_kv=H_kv, D=D, K_local=K_local, hidden=hidden,
            hidden_pad=hidden_pad, N_TILE=N_TILE, super_group_n_tiles=super_group_n_tiles,
            q_per_kv=q_per_kv, num_out=num_out, num_super_groups=nsg,
            max_num_row_tiles=max_num_row_tiles, max_num_batch=max_num_batch,
            max_total_oproj=max_total, tot_cap=tot_cap, max_tot_k=max_tot_k,
            paged=bool(paged), page_size=page_size,
            max_num_pages=max_num_pages, max_num_pages_per_seq=max_num_pages_per_seq,
            ctrl=zeros(NUM_CTRL, torch.uint32), sync_ctrl=zeros(NUM_SYNC, torch.uint32),
            actv=mviews[5][:6], status=zeros(NUM_STATUS, torch.uint32),
            head_ready=zeros(max_num_row_tiles, torch.uint32),
            oproj_queue=zeros(max_total, torch.uint32),
            ar_done_bits=zeros(max_owner_words, torch.int64),
            cu_q=mviews[0], cu_k=mviews[1], fa_b=mviews[2], fa_mb=mviews[3], fa_order=mviews[4],
            Q=zeros((tot_cap, H_local, D), dtype),
            K=(None if paged else zeros((max_tot_k, H_kv, D), dtype)),
            V=(None if paged else zeros((max_tot_k, H_kv, D), dtype)),
            K_cache=(zeros((max_num_pages, 128, H_kv, D), dtype) if paged else None),
            V_cache=(zeros((max_num_pages, 128, H_kv, D), dtype) if paged else None),
            page_table=(zeros((max_num_batch, max_num_pages_per_seq), torch.int32)
                        if paged else None),
            cache_seqlens=(zeros(max_num_batch, torch.int32) if paged else None),
            W_o=zeros((K_local, hidden_pad), dtype),
            Oscr=zeros((max_num_row_tiles, 128, H_local, D), dtype),
            csym=csym, rco=rco, rbits=rbits, nvl=nvl,
            csym_mc_ptr=csym_mc_ptr, nvl_peer_ptrs=nvl_peer_ptrs, csym_peer_ptrs=csym_peer_ptrs,
            rc_ptrs=rc_ptrs, rb_ptrs=rb_ptrs, _handles=handles,
        )
        # The first launch relies on every control word being zero on every rank before
        # any rank issues a remote control write.
        torch.cuda.synchronize(dev)
        if tp_size > 1:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.barrier()
        return ws

    # ------------------------------------------------------------------ compile
    def compile(self, w_fa=4, w_oproj=1, w_ar=1, num_ctas=None, kv_stages=2,
                K_CHUNK=64, oproj_stages=4, softmax_scale=None, wait_limit_ms=0, audit=False):
        """Fix the launch configuration and build the C-ABI plan.

        ``kv_stages``, ``K_CHUNK`` and ``oproj_stages`` are accepted for signature
        compatibility; the staging depths of the sm_100a kernel are fixed.
        ``num_ctas=None`` means one CTA per SM.  ``audit=True`` adds execution counters
        (``self.audit``: one per attention (row tile, head), per O_proj slot, per owned
        AllReduce slot; see ``audit_counts``) for exactly-once checks.
        """
        if self._plan is not None:
            self._lib.ma_plan_destroy(self._plan)
            self._plan = None
        # the execution counters exist in the audit build of the library only
        self._lib = _cabi.audit_lib() if audit else _cabi.lib
        d = _cabi.PlanDesc()
        d.device = self.dev.index if self.dev.index is not None else torch.cuda.current_device()
        d.tp_size, d.rank = self.tp_size, self.rank
        d.H_local, d.H_kv, d.D, d.hidden = self.H_local, self.H_kv, self.D, self.hidden
        d.super_group_n_tiles = self.super_group_n_tiles
        d.max_row_tiles, d.max_batch = self.max_num_row_tiles, self.max_num_batch
        d.max_tot_q = self.tot_cap
        d.max_tot_k = self.max_num_pages * 128 if self.paged else self.max_tot_k
        d.softmax_scale = float(softmax_scale) if softmax_scale is not None else 0.0
        d.wait_limit_ms = int(wait_limit_ms)
        kv = (self.K_cache, self.V_cache) if self.paged else (self.K, self.V)
        if self.paged:
            d.page_table = self.page_table.data_ptr()
            d.cache_seqlens = self.cache_seqlens.data_ptr()
            d.max_pages_per_seq = self.max_num_pages_per_seq
        for name, t in (("Q", self.Q), ("K", kv[0]), ("V", kv[1]), ("W_o", self.W_o),
                        ("o_scratch", self.Oscr), ("csym", self.csym), ("ctrl", self.ctrl),
                        ("sync_ctrl", self.sync_ctrl), ("actv", self.actv),
                        ("head_ready", self.head_ready), ("oproj_queue", self.oproj_queue),
                        ("ready_count", self.rco), ("ready_bits", self.rbits),
                        ("ar_done_bits", self.ar_done_bits), ("nvl_signal", self.nvl),
                        ("cu_q", self.cu_q), ("cu_k", self.cu_k), ("fa_b", self.fa_b),
                        ("fa_mb", self.fa_mb), ("status", self.status),
                        ("fa_order", self.fa_order)):
            setattr(d, name, t.data_ptr())
        self.audit = None
        if audit:
            owner_slots = (self.max_total_oproj + self.tp_size - 1) // self.tp_size
            self.audit = torch.zeros(self.max_num_row_tiles * self.H_local + self.max_total_oproj
                                     + owner_slots, dtype=torch.int32, device=self.dev)
            d.audit = self.audit.data_ptr()
        d.csym_multicast = self.csym_mc_ptr
        for r in range(self.tp_size if self.tp_size > 1 else 0):
            d.peer_ready_count[r] = self.rc_ptrs[r]
            d.peer_ready_bits[r] = self.rb_ptrs[r]
            d.peer_nvl_signal[r] = self.nvl_peer_ptrs[r]
            d.peer_csym[r] = self.csym_peer_ptrs[r]
        plan = C.c_void_p()
        _cabi.check(self._lib.ma_plan_create(C.byref(d), C.byref(plan)), "ma_plan_create")
        self._plan = plan
        self._args = _cabi.LaunchArgs(int(w_fa), int(w_oproj), int(w_ar),
                                      int(num_ctas) if num_ctas else 0, 0)
        self._ts = torch.cuda.current_stream(self.dev)
        return self

    # ------------------------------------------------------------------ per layer
    def set_layer(self, meta, Q, K, V, W_o, page_table=None, cache_seqlens=None):
        """Copy one layer's inputs and varlen metadata into the active prefixes.

        ``Q [tot_q,H_local,D]``, ``K/V [tot_k,H_kv,D]``, ``W_o [K_local,hidden]``; host
        (pinned) or device tensors.  With ``paged=True`` K/V are the caches
        ``[num_pages,128,H_kv,D]`` and ``page_table [B,pps]`` / ``cache_seqlens [B]`` (int32)
        are required.  Raises ``AssertionError`` on any capacity violation before touching
        the workspace.
        """
        R, nb = meta.num_row_tiles, meta.num_batch
        tq = Q.shape[0]
        assert R <= self.max_num_row_tiles and nb <= self.max_num_batch
        assert tq <= self.tot_cap
        assert tuple(Q.shape[1:]) == (self.H_local, self.D)
        assert tuple(W_o.shape) == (self.K_local, self.hidden)
        assert int(meta.cu_seqlens_q[-1]) == tq
        if self.paged:
            # K, V are caches [num_pages, 128, H_kv, D] (workspace.py:213-222 of the reference)
            assert page_table is not None and cache_seqlens is not None
            page_table = torch.as_tensor(page_table, dtype=torch.int32)
            cache_seqlens = torch.as_tensor(cache_seqlens, dtype=torch.int32)
            npg, pps = K.shape[0], page_table.shape[1]
            assert npg <= self.max_num_pages and pps <= self.max_num_pages_per_seq, (
                npg, self.max_num_pages, pps, self.max_num_pages_per_seq)
            assert tuple(K.shape[1:]) == (128, self.H_kv, self.D) == tuple(V.shape[1:])
            assert V.shape[0] == npg and page_table.shape[0] == nb == cache_seqlens.shape[0]
            lens_k = cache_seqlens.cpu().numpy().astype(np.int64)
            lens_q = np.diff(np.asarray(meta.cu_seqlens_q, dtype=np.int64))
            assert bool((lens_k >= lens_q).all()), "q_len > k_len is not supported"
            assert bool((-(-lens_k // 128) <= pps).all())
            assert int(page_table.max()) < npg and int(page_table.min()) >= 0
        else:
            assert page_table is None and cache_seqlens is None
            tk = K.shape[0]
            assert tk <= self.max_tot_k and V.shape[0] == tk
            assert tuple(K.shape[1:]) == (self.H_kv, self.D) == tuple(V.shape[1:])
            assert int(meta.cu_seqlens_k[-1]) == tk
        self._unbind()
        with torch.cuda.stream(self._stream()):
            self.Q[:tq].copy_(Q, non_blocking=True)
            self.W_o[:, :self.hidden].copy_(W_o, non_blocking=True)
            if self.paged:
                self.K_cache[:npg].copy_(K, non_blocking=True)
                self.V_cache[:npg].copy_(V, non_blocking=True)
                self.page_table[:nb, :pps].copy_(page_table.to(self.dev))
                self.cache_seqlens[:nb].copy_(cache_seqlens.to(self.dev))
            else:
                self.K[:tk].copy_(K, non_blocking=True)
                self.V[:tk].copy_(V, non_blocking=True)
            self._set_meta(meta)

    def bind_inputs(self, meta, Q, K, V, W_o, page_table=None, cache_seqlens=None):
        """Zero-copy alternative to ``set_layer``: the kernel reads the caller's device
        tensors in place (only the varlen metadata is uploaded).  ``W_o`` may be the plain
        ``[K_local, hidden]`` weight when ``hidden % 64 == 0``, else a zero-padded
        ``[K_local, hidden_pad]`` one.  The tensors must stay alive and unchanged until the
        launch has finished; a later ``set_layer`` goes back to the workspace's own buffers.
        """
        for t in (Q, K, V, W_o):
            assert t.is_cuda and t.device == self.dev and t.dtype == self.dtype
            assert t.is_contiguous() and t.data_ptr() % 16 == 0
        R, nb = meta.num_row_tiles, meta.num_batch
        assert R <= self.max_num_row_tiles and nb <= self.max_num_batch
        assert tuple(Q.shape[1:]) == (self.H_local, self.D) and Q.shape[0] <= self.tot_cap
        assert int(meta.cu_seqlens_q[-1]) == Q.shape[0]
        assert W_o.shape[0] == self.K_local and W_o.shape[1] >= self.hidden and W_o.shape[1] % 64 == 0
        if self.paged:
            assert page_table is not None and cache_seqlens is not None
            assert tuple(K.shape[1:]) == (128, self.H_kv, self.D) == tuple(V.shape[1:])
            tot_k = K.shape[0] * 128
            page_table = torch.as_tensor(page_table, dtype=torch.int32)
            cache_seqlens = torch.as_tensor(cache_seqlens, dtype=torch.int32)
            assert page_table.shape[1] <= self.max_num_pages_per_seq
            assert int(page_table.max()) < K.shape[0] and int(page_table.min()) >= 0
        else:
            assert tuple(K.shape[1:]) == (self.H_kv, self.D) == tuple(V.shape[1:])
            tot_k = K.shape[0]
            assert int(meta.cu_seqlens_k[-1]) == tot_k
        _cabi.check(self._lib.ma_plan_set_inputs(
            self._plan, Q.data_ptr(), K.data_ptr(), V.data_ptr(), W_o.data_ptr(),
            int(Q.shape[0]), int(tot_k), int(W_o.shape[1])), "ma_plan_set_inputs")
        self._bound = (Q, K, V, W_o)          # keep them alive
        with torch.cuda.stream(self._stream()):
            if self.paged:
                self.page_table[:nb, :page_table.shape[1]].copy_(page_table.to(self.dev))
                self.cache_seqlens[:nb].copy_(cache_seqlens.to(self.dev))
            self._set_meta(meta)

    def _unbind(self):
        if getattr(self, "_bound", None) is not None:
            kv = (self.K_cache, self.V_cache) if self.paged else (self.K, self.V)
            tot_k = self.max_num_pages * 128 if self.paged else self.max_tot_k
            _cabi.check(self._lib.ma_plan_set_inputs(
                self._plan, self.Q.data_ptr(), kv[0].data_ptr(), kv[1].data_ptr(),
                self.W_o.data_ptr(), self.tot_cap, tot_k, self.hidden_pad), "ma_plan_set_inputs")
            self._bound = None

    def set_meta(self, meta):
        """Metadata only (inputs already resident in ``self.Q/K/V/W_o``)."""
        assert meta.num_row_tiles <= self.max_num_row_tiles
        assert meta.num_batch <= self.max_num_batch
        assert int(meta.cu_seqlens_q[-1]) <= self.tot_cap
        assert self.paged or int(meta.cu_seqlens_k[-1]) <= self.max_tot_k
        with torch.cuda.stream(self._stream()):
            self._set_meta(meta)

    def _set_meta(self, meta):
        R = meta.num_row_tiles
        # ONE asynchronous H2D copy: the six arrays are packed at their capacity offsets into
        # a pinned staging buffer (a ring of four, so the host never rewrites a buffer whose
        # copy may still be in flight)
        if getattr(self, "_meta_ring", None) is None:
            self._meta_ring = [[torch.zeros(self._meta_offs[-1], dtype=torch.int32).pin_memory(), None]
                               for _ in range(4)]
            self._meta_i = 0
        slot = self._meta_ring[self._meta_i % 4]
        self._meta_i += 1
        if slot[1] is not None:
            slot[1].synchronize()
        buf = slot[0].numpy()
        o = self._meta_offs
        prime = self.fa_prime_tiles
        if prime is None:
            prime = fa_prime_tiles_b200(meta, self.hidden, self.tp_size, self.H_local)
        self._auto_flags = launch_flags_b200(meta, self.hidden, self.tp_size, self.H_local)
        for i, arr in enumerate((meta.cu_seqlens_q, meta.cu_seqlens_k, meta.batch_idx, meta.m_block,
                                 claim_order(meta, prime),
                                 active_counts(R, self.H_local, self.num_super_groups,
                                               self.tp_size, self.rank))):
            arr = np.asarray(arr, dtype=np.int32)
            buf[o[i]:o[i] + arr.size] = arr
        self.meta_dev.copy_(slot[0], non_blocking=True)
        slot[1] = torch.cuda.Event()
        slot[1].record(torch.cuda.current_stream(self.dev))
        self._meta = meta

    def _stream(self):
        return getattr(self, "_ts", None) or torch.cuda.current_stream(self.dev)

    def launch(self, flags=None):
        assert self._plan is not None, "call compile() first"
        if flags is None:
            flags = self._auto_flags if self.default_flags is None else self.default_flags
        if self.tp_size == 2 and self.ar_p2p:
            # two GPUs: reduce with peer loads/stores, not multimem (see MA_FLAG_AR_P2P)
            flags |= _cabi.MA_FLAG_AR_P2P
        args = _cabi.LaunchArgs(self._args.w_fa, self._args.w_oproj, self._args.w_ar,
                                self._args.num_ctas, int(flags))
        _cabi.check(self._lib.ma_launch(self._plan, C.byref(args),
                                        C.c_void_p(self._ts.cuda_stream)), "ma_launch")

    def launch_fa_only(self):
        """Attention stage alone (fills ``Oscr``); used by the unfused baseline."""
        self.launch(flags=_cabi.MA_FLAG_FA_ONLY)

    def launch_oproj_only(self):
        """O_proj stage alone (single rank): ``Oscr`` must hold a finished attention output."""
        assert self.tp_size == 1
        self.launch(flags=_cabi.MA_FLAG_OPROJ_ONLY)

    def launch_ar_only(self, extra_flags=0):
        """AllReduce stage alone over every slot of ``csym`` (tp > 1).  Every rank's partial
        must be complete before any rank launches (e.g. after a host barrier)."""
        assert self.tp_size > 1, "the AllReduce stage needs tp_size > 1"
        self.launch(flags=_cabi.MA_FLAG_AR_ONLY | extra_flags)

    def audit_counts(self, meta=None):
        """``(attention [R, H_local], o_proj [R * nsg], allreduce [owned])`` execution
        counts since the last ``audit.zero_()`` (``compile(audit=True)``)."""
        meta = meta or self._meta
        R = meta.num_row_tiles
        a = self.audit.cpu()
        n_fa, n_op = self.max_num_row_tiles * self.H_local, self.max_total_oproj
        total = R * self.num_super_groups
        owned = max(total - self.rank, 0)
        owned = (owned + self.tp_size - 1) // self.tp_size
        return (a[:R * self.H_local].view(R, self.H_local), a[n_fa:n_fa + total],
                a[n_fa + n_op:n_fa + n_op + owned])

    def check_status(self):
        """Synchronise the launch stream and raise if a device-side wait gave up."""
        st = _cabi.Status()
        rc = self._lib.ma_read_status(self._plan, C.c_void_p(self._ts.cuda_stream), C.byref(st))
        if rc != _cabi.MA_OK:
            raise RuntimeError(
                f"fused prefill kernel: {_cabi.strerror(rc)} "
                f"(code={st.code} site=0x{st.site:x} cta={st.cta} aux={st.aux}); "
                "the workspace control state is undefined — call debug_zero_all()")

    def output(self, meta=None):
        """De-tiled ``[tot_q, hidden]`` copy of the valid region of ``csym``."""
        meta = meta or self._meta
        flat = self.csym.view(self.max_num_row_tiles, 128, self.hidden_pad)
        tot = int(meta.cu_seqlens_q[-1])
        out = torch.empty(tot, self.hidden, dtype=self.dtype, device=self.dev)
        for t in range(meta.num_row_tiles):
            s, vm = meta.q_tile_start(t), meta.valid_m(t)
            out[s:s + vm] = flat[t, :vm, :self.hidden]
        return out

    # ------------------------------------------------------------------ debug
    def debug_zero_all(self):
        """Fault localisation only; never on the production / bench / test default path.
        With tp > 1 every rank must call it, followed by a host barrier."""
        for t in (self.ctrl, self.sync_ctrl, self.actv, self.head_ready, self.oproj_queue,
                  self.fa_order, self.rco, self.rbits, self.ar_done_bits, self.nvl, self.csym, self.Oscr,
                  self.status):
            t.zero_()

    def __del__(self):
        try:
            if self._plan is not None:
                self._lib.ma_plan_destroy(self._plan)
                self._plan = None
        except Exception:
            pass
