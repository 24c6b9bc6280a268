"""Failure detection without a GPU fault: every device-side wait is bounded, and a launch
that can never finish returns with a status instead of hanging.

The launch is made unfinishable on the host side only: the active count of O_proj tasks is
set one too high, so the schedulers run out of work without ever reaching the done
condition.  After ``wait_limit_ms`` each CTA records the wait that gave up and leaves;
``check_status`` turns that into ``RuntimeError``.  Nothing traps, and after
``debug_zero_all`` the same workspace runs a normal layer again.  (The reference's waits
are unbounded: fused_fa_oproj_ar.py:90-95, 137-142, 263-268.)
"""
import pytest
import torch

from cases import CASES, make_inputs

pytestmark = pytest.mark.gpu


def test_unreachable_done_condition_times_out_and_workspace_recovers():
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    from oracle.chain_oracle import full_chain_oracle, err_beyond_rounding
    name = "gqa_q2"
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, hidden, H, 128, q_per_kv=qpk,
                                        device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0, num_ctas=8, wait_limit_ms=250)
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    ws.actv[1] += 1                      # one O_proj task more than will ever exist
    ws.launch()
    with pytest.raises(RuntimeError) as err:
        ws.check_status()
    assert "gave up" in str(err.value) and "code=" in str(err.value)
    st = ws.status.cpu()
    assert int(st[0]) != 0
    # recover: clear everything, run the same layer for real
    ws.debug_zero_all()
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    ws.launch()
    ws.check_status()
    _, Yp, _ = full_chain_oracle(Q, K, V, W, sq, sk)
    assert err_beyond_rounding(ws.output(meta).cpu(), Yp) <= 2e-3
    assert ws.ctrl.cpu().tolist() == [0] * 8


def test_host_side_rejections_leave_the_workspace_untouched():
    # tests/fused/test_fused_production.py:129-146 of the reference: over-capacity layers
    # raise AssertionError from set_layer and the workspace stays usable
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    ws = FusedFaOprojArWorkspace.create(None, 2, 256, 2, 128, max_tot_k=300, device="cuda:0")
    ws.compile()
    before = ws.Q.clone()
    big = build_row_desc([300])
    with pytest.raises(AssertionError):
        ws.set_layer(big, torch.zeros(300, 2, 128, dtype=torch.bfloat16),
                     torch.zeros(300, 2, 128, dtype=torch.bfloat16),
                     torch.zeros(300, 2, 128, dtype=torch.bfloat16),
                     torch.zeros(256, 256, dtype=torch.bfloat16))
    longk = build_row_desc([128], seqlens_k=[400])
    with pytest.raises(AssertionError):
        ws.set_layer(longk, torch.ones(128, 2, 128, dtype=torch.bfloat16),
                     torch.zeros(400, 2, 128, dtype=torch.bfloat16),
                     torch.zeros(400, 2, 128, dtype=torch.bfloat16),
                     torch.zeros(256, 256, dtype=torch.bfloat16))
    assert torch.equal(ws.Q, before)
