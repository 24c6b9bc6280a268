"""Paged KV (page size 128) through the workspace / C ABI on one GPU.

Mirrors the reference's tests/fused/test_fused_paged_single_card.py: the packed K/V that
the attention oracle reads are scattered into shuffled physical pages (with spare pages
and random values in every slot that holds no token), and the fused output must match the
contiguous-KV oracle: MHA and GQA, q == k and q < k, a last Q tile and a last K page that
are not full, several sequences.  A page size other than 128 is refused.
"""
import pytest
import torch

from cases import CASES, make_inputs
from oracle.chain_oracle import (full_chain_oracle, o_scratch_oracle, make_paged_kv,
                                 err_beyond_rounding, tile_coords)

pytestmark = pytest.mark.gpu
SENT = -7.0
PAGED_CASES = ["varlen_200", "vm44_300", "multi_seq", "gqa_q2", "gqa_q4_vm44",
               "chunk_unaligned", "chunk_multitile", "chunk_multiseq", "chunk_gqa_q4"]


@pytest.mark.parametrize("name", PAGED_CASES)
def test_paged_matches_contiguous_oracle(name):
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    sq, H, hidden, qpk, sk, seed = CASES[name]
    sk = sq if sk is None else sk
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    pages = sum((s + 127) // 128 for s in sk) + 2
    Kc, Vc, table, lens = make_paged_kv(K, V, sk, num_pages=pages, shuffle=True, seed=seed + 7)
    ws = FusedFaOprojArWorkspace.create(
        None, meta.num_row_tiles, hidden, H, 128, q_per_kv=qpk, paged=True, page_size=128,
        max_num_pages=pages, max_num_pages_per_seq=table.shape[1], device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0, num_ctas=8)
    ws.csym.fill_(SENT)
    ws.set_layer(meta, Q.cuda(), Kc.cuda(), Vc.cuda(), W.cuda(), page_table=table,
                 cache_seqlens=lens)
    ws.launch()
    ws.check_status()
    O, Yp, _ = full_chain_oracle(Q, K, V, W, sq, sk)
    oscr = ws.Oscr.float().cpu()
    assert float((oscr - o_scratch_oracle(O, sq)).abs().max()) < 2e-2
    for t, (s, vm) in enumerate(tile_coords(sq)):
        if vm < 128:
            assert float(oscr[t, vm:].abs().max()) == 0.0
            assert bool((ws.csym[t, vm:] == SENT).all())
    tol = 8e-3 if sk != sq else 2e-3
    assert err_beyond_rounding(ws.output(meta).cpu(), Yp) <= tol
    assert ws.ctrl.cpu().tolist() == [0] * 8


def test_other_page_sizes_are_refused():
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    with pytest.raises(AssertionError):
        FusedFaOprojArWorkspace.create(None, 2, 256, 2, 128, paged=True, page_size=64,
                                       device="cuda:0")
