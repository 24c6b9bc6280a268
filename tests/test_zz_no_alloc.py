"""The allocation-free entry point, ``ma_fused_prefill_noalloc``, against the workspace
entry points on the same inputs.

Some users of this library run where they may not allocate device memory: a serving
engine whose memory pool was sized at start-up and already owns every free byte, a
latency-critical path that cannot take an allocation's implicit synchronisation, a
plug-in that is handed buffers but may not create any.  For them the library keeps one
fixed scratch array per GPU and the caller passes only inputs and the output buffer.

The test calls the entry point through the C ABI twice in a row (the second call finds
the array holding the first call's leftovers), and each time compares the output with
what ``ma_plan_create`` + ``ma_launch`` produce: both run the same kernel on the same
bits, so over the valid region the two must be equal bit for bit, and both must lie
within the tolerance the other fused tests use against the CPU oracle (abs 3e-2 on C_sym,
2e-3 / 8e-3 of the maximum beyond bf16 rounding on the chained output); padding rows and
columns of the caller's buffer must be left untouched.  It also checks that free device memory
does not move across the second call, and that sizes beyond the stated maximum are
refused.  It sits in a file that pytest collects last on purpose.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs

pytestmark = pytest.mark.gpu
SENT = -7.0


def _call(sq, sk, H, Hkv, hidden, Q, K, V, W, out, sg=4):
    from megaattention_b200 import _cabi
    a = _cabi.NoAllocArgs()
    a.H_local, a.H_kv, a.hidden, a.super_group_n_tiles = H, Hkv, hidden, sg
    a.num_batch = len(sq)
    a.w_fa, a.w_oproj, a.num_ctas = 2, 1, 0
    a.softmax_scale, a.wait_limit_ms = 0.0, 0
    q_arr = (C.c_int32 * len(sq))(*sq)
    k_arr = (C.c_int32 * len(sq))(*(sk or sq))
    a.seqlens_q, a.seqlens_k = q_arr, k_arr
    a.Q, a.K, a.V, a.W_o = Q.data_ptr(), K.data_ptr(), V.data_ptr(), W.data_ptr()
    a.out = out.data_ptr() if out is not None else 0
    st = _cabi.Status()
    a.status_out = C.pointer(st)
    rc = _cabi.lib.ma_fused_prefill_noalloc(
        C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, st


def _workspace_result(name):
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(
        None, meta.num_row_tiles, hidden, H, 128, q_per_kv=qpk,
        max_tot_k=int(meta.cu_seqlens_k[-1]), device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0)
    ws.csym.fill_(SENT)
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    ws.launch()
    ws.check_status()
    return meta, ws.csym[:meta.num_row_tiles].clone(), (Q, K, V, W)


@pytest.mark.parametrize("name", ["gqa_q2", "chunk_multiseq"])
def test_noalloc_matches_workspace_entry_points_twice(name):
    from megaattention_b200 import _cabi
    sq, H, hidden, qpk, sk, seed = CASES[name]
    meta, ref, (Q, K, V, W) = _workspace_result(name)
    Qd, Kd, Vd, Wd = Q.cuda(), K.cuda(), V.cuda(), W.cuda().contiguous()
    outs = [torch.full_like(ref, SENT) for _ in range(2)]
    torch.cuda.synchronize()
    free_before = None
    for i in range(2):
        if i == 1:
            free_before = torch.cuda.mem_get_info()[0]
        rc, st = _call(sq, sk, H, H // qpk, hidden, Qd, Kd, Vd, Wd, outs[i])
        assert rc == _cabi.MA_OK, (_cabi.strerror(rc), st.code, hex(st.site), st.cta)
        if i == 1:
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed free memory"
    from oracle.chain_oracle import full_chain_oracle, untile_csym, err_beyond_rounding
    _, Yp, _ = full_chain_oracle(Q, K, V, W, sq, sk)
    num_out = ref.shape[2]
    for out in outs:
        for t in range(meta.num_row_tiles):
            vm = meta.valid_m(t)
            for o in range(num_out):
                vn = min(128, hidden - o * 128)
                assert torch.equal(out[t, :vm, o, :vn], ref[t, :vm, o, :vn])
                assert bool((out[t, vm:, o, :] == SENT).all())
                assert bool((out[t, :, o, vn:] == SENT).all())
        got = untile_csym(out.cpu(), sq, hidden)
        assert float((got.float() - Yp).abs().max()) < 3e-2
        assert err_beyond_rounding(got, Yp) <= (8e-3 if sk is not None else 2e-3)


def test_noalloc_refuses_sizes_beyond_its_scratch():
    from megaattention_b200 import _cabi
    dummy = torch.zeros(64, dtype=torch.bfloat16, device="cuda:0")
    # 16 q heads and 80 row tiles need 80*128*2048*2 bytes of attention scratch: > 16 MiB
    rc, _ = _call([80 * 128], None, 16, 2, 256, dummy, dummy, dummy, dummy, dummy)
    assert rc == _cabi.MA_ERR_CAPACITY
    # more row tiles than the descriptor table holds
    rc, _ = _call([128] * 513, None, 1, 1, 128, dummy, dummy, dummy, dummy, dummy)
    assert rc == _cabi.MA_ERR_CAPACITY
    rc, _ = _call([128], None, 2, 1, 100, dummy, dummy, dummy, dummy, dummy)   # hidden % 64
    assert rc == _cabi.MA_ERR_INVALID
