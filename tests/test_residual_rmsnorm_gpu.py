"""Residual add + RMSNorm consumer (``ma_residual_rmsnorm``) on the fused launch's output,
against the CPU oracle: the new residual stream bit for bit, the normalised output to one
bf16 ulp (the row statistics are summed in a different order)."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from cases import CASES, make_inputs  # noqa: E402
from oracle.consumer_oracle import residual_rmsnorm_oracle  # noqa: E402

pytestmark = pytest.mark.gpu


def _layer(name):
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(
        None, max_num_row_tiles=meta.num_row_tiles + 2, hidden=hidden, H_local=H, D=128,
        q_per_kv=qpk, max_tot_k=int(meta.cu_seqlens_k[-1]), device="cuda:0")
    ws.compile()
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    ws.launch()
    ws.check_status()
    return ws, meta, sum(sq), hidden


def _check(normed, new_res, y, res, w, eps):
    ref_out, ref_h = residual_rmsnorm_oracle(y, res, w, eps)
    assert torch.equal(new_res.cpu(), ref_h)
    d = (normed.cpu().float() - ref_out.float()).abs()
    assert bool((d <= ref_out.float().abs() * 2.0 ** -7 + 1e-30).all()), float(d.max())
    assert float((d == 0).float().mean()) > 0.98


@pytest.mark.parametrize("name", ["multi_seq", "ragged_hidden", "vm44_300", "chunk_multiseq", "c1"])
def test_consumer_reads_the_tile_padded_output_in_place(name):
    from megaattention_b200.runtime.residual_rmsnorm import residual_rmsnorm
    ws, meta, tot_q, hidden = _layer(name)
    g = torch.Generator().manual_seed(77)
    res = (torch.randn(tot_q, hidden, generator=g) * 2).to(torch.bfloat16)
    w = (1 + 0.2 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    y = ws.output(meta).cpu()
    res_d = res.cuda()
    normed, new_res = residual_rmsnorm(ws, res_d, w.cuda(), eps=1e-5)
    torch.cuda.synchronize()
    assert torch.equal(res_d.cpu(), res)                      # not in place unless asked
    _check(normed, new_res, y, res, w, 1e-5)
    normed2, same = residual_rmsnorm(ws, res_d, w.cuda(), eps=1e-5, inplace=True)
    torch.cuda.synchronize()
    assert same.data_ptr() == res_d.data_ptr()
    _check(normed2, res_d, y, res, w, 1e-5)


@pytest.mark.parametrize("hidden", [4096, 16384])
def test_consumer_at_the_benchmark_widths(hidden):
    """Row tiles of three ragged sequences filled with random values instead of a launch: the
    widths of the benchmark configurations (two and eight 16-byte chunks per thread)."""
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    from megaattention_b200.runtime.residual_rmsnorm import residual_rmsnorm
    sq = [300, 129, 64]
    meta = build_row_desc(sq)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, hidden, 2, 128, q_per_kv=2,
                                        max_tot_k=sum(sq), device="cuda:0")
    ws.compile()
    ws.set_meta(meta)
    g = torch.Generator().manual_seed(hidden)
    tiles = torch.randn(meta.num_row_tiles, 128, hidden, generator=g).to(torch.bfloat16)
    ws.csym.copy_(tiles.view(ws.csym.shape).cuda())
    res = torch.randn(sum(sq), hidden, generator=g).to(torch.bfloat16)
    w = (1 + 0.2 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    y = ws.output(meta).cpu()
    normed, new_res = residual_rmsnorm(ws, res.cuda(), w.cuda())
    torch.cuda.synchronize()
    _check(normed, new_res, y, res, w, 1e-6)
