"""Single-GPU parity of the fused kernel (tp_size = 1, AllReduce = identity) through the
workspace / C ABI, against the CPU oracle and the reference-produced fixtures.

Mirrors the reference's tests/fused/test_fused_single_card.py:107-157: per launch it checks
O_scratch against the attention oracle, tail rows exactly zero, C_sym against the O_proj
oracle over the valid region, that a sentinel pre-filled into C_sym survives in every
masked row / column, and that the exit path left the control words zero.
Tolerances: abs 2e-2 on O_scratch and 3e-2 on C_sym (the reference's), and on the
chained output 2e-3 (q == k) / 8e-3 (q < k) of max|ref| beyond the rounding that a bf16
result carries by construction (half a bf16 ulp of the fp32 reference value; see
oracle.chain_oracle.err_beyond_rounding).  The raw err_rel values are recorded too.
"""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle.chain_oracle import (full_chain_oracle, o_scratch_oracle, tile_coords, err_rel,
                                 err_beyond_rounding)

pytestmark = pytest.mark.gpu
SENT = -7.0
GOLD = os.path.join(os.path.dirname(__file__), "golden")


# Head groupings the fixture matrix does not have: odd q_per_kv (MHA included) with three,
# six and eight heads, so that attention tasks pair two q heads that do NOT share a kv head
# (each with K/V stages of its own), plus the single head an odd head count leaves over.
# Same input recipe as the fixture cases; compared with the oracle only.
EXTRA_CASES = {
    "mha_h3":          ([300, 130],      3, 384, 1, None,            31),
    "q3_h3":           ([200, 64, 130],  3, 256, 3, None,            32),
    "q3_h6_chunk":     ([260],           6, 256, 3, [516],           33),
    "mha_h8":          ([300, 200],      8, 512, 1, None,            34),
    "mha_h1":          ([200],           1, 256, 1, None,            35),
}


def _case_inputs(name):
    if name in CASES:
        return CASES[name], make_inputs(name)
    from cases import _randn
    sq, H, hidden, qpk, sk, seed = EXTRA_CASES[name]
    skk = sq if sk is None else sk
    base = seed * 1000
    return EXTRA_CASES[name], (_randn((sum(sq), H, 128), base + 0),
                               _randn((sum(skk), H // qpk, 128), base + 1),
                               _randn((sum(skk), H // qpk, 128), base + 2),
                               _randn((H * 128, hidden), base + 3, float(H * 128) ** -0.5))


def run_case(name, w=(4, 1, 1), num_ctas=None, launches=1, audit=False):
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    (sq, H, hidden, qpk, sk, seed), (Q, K, V, W) = _case_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(
        None, max_num_row_tiles=meta.num_row_tiles, hidden=hidden, H_local=H, D=128,
        q_per_kv=qpk, max_tot_k=int(meta.cu_seqlens_k[-1]), device="cuda:0")
    ws.compile(w_fa=w[0], w_oproj=w[1], w_ar=w[2], num_ctas=num_ctas, audit=audit)
    for _ in range(launches):
        ws.csym.fill_(SENT)
        ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
        ws.launch()
        ws.check_status()
    if audit:
        # every attention (row tile, head), O_proj slot and (identity) AllReduce slot was
        # executed exactly once per launch, and nothing outside the active range was touched
        fa, op, ar = ws.audit_counts(meta)
        assert bool((fa == launches).all()) and bool((op == launches).all()), (fa, op)
        assert bool((ar == 0).all())        # one rank: the O_proj finisher accounts the slot
        assert int(ws.audit.sum()) == launches * (fa.numel() + op.numel())
    O, Yp, Yf = full_chain_oracle(Q, K, V, W, sq, sk)
    oscr_ref = o_scratch_oracle(O, sq)
    oscr = ws.Oscr.float().cpu()
    csym = ws.csym.cpu()
    tiles = tile_coords(sq)
    res = dict(o_err=float((oscr - oscr_ref).abs().max()), o_tail=0.0, c_err=0.0, leak=0.0)
    num_out = ws.num_out
    for t, (s, vm) in enumerate(tiles):
        if vm < 128:
            res["o_tail"] = max(res["o_tail"], float(oscr[t, vm:].abs().max()))
        for o in range(num_out):
            vn = min(128, hidden - o * 128)
            got = csym[t, :vm, o, :vn].float()
            res["c_err"] = max(res["c_err"], float(
                (got - Yp[s:s + vm, o * 128:o * 128 + vn]).abs().max()))
            if vm < 128:
                res["leak"] = max(res["leak"], float((csym[t, vm:, o, :] != SENT).float().max()))
            if vn < 128:
                res["leak"] = max(res["leak"], float((csym[t, :, o, vn:] != SENT).float().max()))
    out = ws.output(meta).cpu()
    res["err_rel_fp32"] = err_rel(out, Yp)
    res["err_rel_bf16"] = err_rel(out, Yf)
    res["ctrl"] = ws.ctrl.cpu().numpy().astype(np.int64).tolist()
    res["err_comp"] = err_beyond_rounding(out, Yp)
    if name in CASES:       # against the reference-produced fixture as well
        g = np.load(os.path.join(GOLD, f"chain_{name}.npz"))
        ref_yf = torch.from_numpy(g["y_final_bits"]).view(torch.bfloat16)
    else:
        ref_yf = Yf
    res["err_rel_fixture"] = err_rel(out, ref_yf)
    res["err_comp_fixture"] = err_beyond_rounding(out, ref_yf, extra_half_ulps=1.0)
    res["q_lt_k"] = sk is not None
    res["out"], res["oscr"], res["Yp"] = out, oscr, Yp
    return res


def check(res):
    res = {k: v for k, v in res.items() if not torch.is_tensor(v)}
    assert res["o_err"] < 2e-2, res
    assert res["o_tail"] == 0.0, res
    assert res["c_err"] < 3e-2, res
    assert res["leak"] == 0.0, res
    assert res["ctrl"] == [0] * 8, res
    tol = 8e-3 if res["q_lt_k"] else 2e-3
    assert res["err_comp"] <= tol, res
    # the fixture (the reference's own bf16 output) was rounded once already
    assert res["err_comp_fixture"] <= tol, res


@pytest.mark.parametrize("name", list(CASES))
def test_fused_matches_oracle(name):
    check(run_case(name))


@pytest.mark.parametrize("name", list(CASES))
def test_every_task_runs_exactly_once(name):
    """The audit build of the library (same sources, -DMA_AUDIT) counts every attention (row
    tile, head), O_proj slot and AllReduce slot the kernel finishes: each must read exactly
    one per launch, over three launches on one workspace, with few CTAs and with all."""
    check(run_case(name, audit=True, launches=3, num_ctas=5))
    check(run_case(name, audit=True))


@pytest.mark.parametrize("name", list(EXTRA_CASES))
def test_heads_that_do_not_share_kv_are_paired_too(name):
    check(run_case(name))
    check(run_case(name, launches=3, num_ctas=3))


@pytest.mark.parametrize("name", list(EXTRA_CASES))
def test_unshared_kv_pairs_run_exactly_once(name):
    check(run_case(name, audit=True, launches=2, num_ctas=5))


@pytest.mark.parametrize("w", [(4, 1, 1), (8, 2, 1), (6, 1, 0), (1, 1, 0), (2, 1, 1)])
def test_role_weights_do_not_change_results(w):
    # tests/fused/test_role_weights.py of the reference
    check(run_case("gqa_q2", w=w, num_ctas=8))
    check(run_case("chunk_multiseq", w=w, num_ctas=8))


def test_few_ctas_and_repeat_launches():
    check(run_case("multi_seq", num_ctas=1))
    check(run_case("chunk_gqa_q4", num_ctas=3, launches=3))


def test_stages_run_alone_give_the_fused_result():
    """Attention-only then O_proj-only launches (the pieces the unfused baseline times)
    reproduce the fused launch bit for bit."""
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    name = "chunk_gqa_q4"
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    outs = []
    for staged in (False, True):
        ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, hidden, H, 128, q_per_kv=qpk,
                                            max_tot_k=int(meta.cu_seqlens_k[-1]), device="cuda:0")
        ws.compile(w_fa=2, w_oproj=1, w_ar=0)
        ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
        if staged:
            ws.launch_fa_only(); ws.check_status()
            assert ws.ctrl.cpu().tolist() == [0] * 8
            ws.launch_oproj_only(); ws.check_status()
        else:
            ws.launch(); ws.check_status()
        assert ws.ctrl.cpu().tolist() == [0] * 8
        outs.append((ws.Oscr.clone(), ws.output(meta)))
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])


def test_bound_inputs_give_the_same_result_as_copied_inputs():
    """Zero-copy path (ma_plan_set_inputs): the kernel reads the caller's tensors in place,
    with an unpadded W_o, and gives the same bits as the copying set_layer path; going
    back to set_layer afterwards works too."""
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    name = "chunk_multiseq"                 # hidden 384: unpadded W_o is [256, 384]
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles + 3, hidden, H, 128, q_per_kv=qpk,
                                        max_tot_k=int(meta.cu_seqlens_k[-1]) + 100, device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0)
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    ws.launch(); ws.check_status()
    ref = ws.output(meta).clone()
    ws.csym.zero_(); ws.Q.zero_(); ws.K.zero_(); ws.V.zero_(); ws.W_o.zero_()
    Qd, Kd, Vd, Wd = Q.cuda(), K.cuda(), V.cuda(), W.cuda().contiguous()
    ws.bind_inputs(meta, Qd, Kd, Vd, Wd)
    ws.launch(); ws.check_status()
    assert torch.equal(ws.output(meta), ref)
    ws.csym.zero_()
    ws.set_layer(meta, Qd, Kd, Vd, Wd)
    ws.launch(); ws.check_status()
    assert torch.equal(ws.output(meta), ref)


def test_peer_load_allreduce_flag_is_refused_on_one_rank():
    """MA_FLAG_AR_P2P needs two ranks and their C_sym addresses: on one rank the launch is
    rejected on the host, nothing runs and the workspace stays usable."""
    from megaattention_b200 import _cabi
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    name = "multi_seq"
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, hidden, H, 128, q_per_kv=qpk,
                                        max_tot_k=int(meta.cu_seqlens_k[-1]), device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0)
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    with pytest.raises(RuntimeError):
        ws.launch(flags=_cabi.MA_FLAG_AR_P2P)
    ws.launch(); ws.check_status()
    assert ws.ctrl.cpu().tolist() == [0] * 8


@pytest.mark.parametrize("name", ["c1", "gqa_q2", "chunk_gqa_q4", "ragged_hidden"])
def test_kernel_error_is_the_floor_of_its_staging(name):
    """The tolerance above is stated beyond bf16 rounding; this pins it from the other side.
    ``oracle/numerics_model.py`` computes what a pipeline with the kernel's rounding points
    (bf16 P per key block, bf16 O_scratch, bf16 output) gives when everything in between is
    exact fp32.  The kernel's raw err_rel against the fp32 chain must not exceed 1.25x the
    model's, and kernel and model must give the very same bf16 value for most elements (both
    round nearly the same fp32 value) and never differ by more than one ulp of the top
    binade, for the attention output and for the final output."""
    from oracle.numerics_model import chain_model
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    res = run_case(name)
    Om, Ym = chain_model(Q, K, V, W, sq, sk)
    model_err = err_rel(Ym, res["Yp"])
    print(f"{name}: kernel err_rel={res['err_rel_fp32']:.3g} model err_rel={model_err:.3g}")
    assert res["err_rel_fp32"] <= 1.25 * model_err, (res["err_rel_fp32"], model_err)
    # O_scratch (valid rows) against the model's attention output
    tiles = tile_coords(sq)
    got_o = torch.cat([res["oscr"][t, :vm] for t, (s0, vm) in enumerate(tiles)])
    # (the kernel moves its reference maximum lazily, the model at every block: P is rounded
    # at a different scale, so equality of the bits is the common case, not a law)
    for got, want, what, min_equal in ((got_o, Om.float(), "O_scratch", 0.3),
                                       (res["out"].float(), Ym.float(), "output", 0.3)):
        d = (got - want).abs()
        equal = float((d == 0).float().mean())
        worst = float(d.max() / want.abs().max())
        print(f"  {what}: bit-equal to the model {equal:.3f}, worst difference {worst:.2e} of the maximum")
        # most elements are the same bf16 value; none is further off than one ulp of the top
        # binade (2^-7 of the maximum)
        assert equal >= min_equal and worst <= 2.0 ** -7, (what, equal, worst)


def test_stage_flags_that_do_not_fit_the_plan_are_refused():
    """Launch flags that would send the kernel down a path its buffers do not back are
    rejected on the host (nothing is launched): AllReduce-only on one rank, two stage
    selectors at once, unknown bits.  The workspace stays usable."""
    from megaattention_b200 import _cabi
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    name = "multi_seq"
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, hidden, H, 128, q_per_kv=qpk,
                                        max_tot_k=int(meta.cu_seqlens_k[-1]), device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0)
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    for flags in (_cabi.MA_FLAG_AR_ONLY, _cabi.MA_FLAG_FA_ONLY | _cabi.MA_FLAG_OPROJ_ONLY,
                  _cabi.MA_FLAG_NO_AR | _cabi.MA_FLAG_AR_ONLY, 1 << 20):
        with pytest.raises(RuntimeError):
            ws.launch(flags=flags)
    with pytest.raises(AssertionError):
        ws.launch_ar_only()
    ws.launch(flags=_cabi.MA_FLAG_DRAIN_FIRST)       # a valid flag still launches
    ws.check_status()
    assert ws.ctrl.cpu().tolist() == [0] * 8
