"""The per-layer serving wrapper (``FusedPrefillLayer``): weights bound once, Q/K/V read in
place, several layers on one workspace, both KV layouts, and the wrapper-side refusals the
reference's design notes list (docs/design/
causal_varlen_prefill_persistent_fa_oproj_ar_plan_zh.md:995-1003, 1266-1283)."""
import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle.chain_oracle import full_chain_oracle, make_paged_kv, err_beyond_rounding

pytestmark = pytest.mark.gpu


def _cu(lens):
    return torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)


def test_layers_share_a_workspace_and_match_the_copying_path():
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace, FusedPrefillLayer
    name = "chunk_multiseq"                       # hidden 384, q < k, three sequences
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles + 2, hidden, H, 128, q_per_kv=qpk,
                                        max_tot_k=int(meta.cu_seqlens_k[-1]) + 64, device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0)
    ws.set_layer(meta, Q.cuda(), K.cuda(), V.cuda(), W.cuda())
    ws.launch(); ws.check_status()
    ref = ws.output(meta).clone()
    # two "layers" with different weights on the same workspace, inputs stay where they are
    W2 = (W.float() * 0.5).to(torch.bfloat16)
    layers = [FusedPrefillLayer(ws, W), FusedPrefillLayer(ws, W2)]
    Qd, Kd, Vd = Q.cuda(), K.cuda(), V.cuda()
    outs = []
    for layer in layers:
        csym = layer(Qd, Kd, Vd, _cu(sq), _cu(sk))
        ws.check_status()
        assert csym.shape[0] == meta.num_row_tiles
        outs.append(layer.output().clone())
    assert torch.equal(outs[0], ref)
    _, Yp2, _ = full_chain_oracle(Q, K, V, W2, sq, sk)
    assert err_beyond_rounding(outs[1].cpu(), Yp2) <= 8e-3
    assert ws.ctrl.cpu().tolist() == [0] * 8
    # refusals happen before anything is queued
    with pytest.raises(AssertionError):
        layers[0](Qd, Kd, Vd, _cu(sq), None, page_table=torch.zeros(3, 4, dtype=torch.int32),
                  cache_seqlens=torch.tensor(sk, dtype=torch.int32))
    with pytest.raises(AssertionError):
        layers[0](Qd, Kd, Vd, _cu(sk), _cu(sq))                 # q longer than k
    layers[0](Qd, Kd, Vd, _cu(sq), _cu(sk)); ws.check_status()
    assert torch.equal(layers[0].output(), ref)


def test_paged_token_pool_cache():
    from megaattention_b200.runtime import FusedFaOprojArWorkspace, FusedPrefillLayer
    name = "chunk_gqa_q4"
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    pages = sum((s + 127) // 128 for s in sk) + 3
    Kc, Vc, table, lens = make_paged_kv(K, V, sk, num_pages=pages, shuffle=True, seed=5)
    ws = FusedFaOprojArWorkspace.create(
        None, sum((s + 127) // 128 for s in sq), hidden, H, 128, q_per_kv=qpk, paged=True,
        max_num_pages=pages, max_num_pages_per_seq=table.shape[1] + 1, device="cuda:0")
    ws.compile(w_fa=2, w_oproj=1, w_ar=0)
    layer = FusedPrefillLayer(ws, W)
    pool_k = Kc.cuda().view(-1, H // qpk, 128)          # the engine's token pool [slots, H_kv, D]
    pool_v = Vc.cuda().view(-1, H // qpk, 128)
    layer(Q.cuda(), pool_k, pool_v, _cu(sq), page_table=table.cuda(), cache_seqlens=lens.cuda())
    ws.check_status()
    _, Yp, _ = full_chain_oracle(Q, K, V, W, sq, sk)
    assert err_beyond_rounding(layer.output().cpu(), Yp) <= 8e-3
    with pytest.raises(AssertionError):                  # page size other than 128
        layer(Q.cuda(), pool_k, pool_v, _cu(sq), page_table=table.cuda(),
              cache_seqlens=lens.cuda(), page_size=64)
    with pytest.raises(AssertionError):                  # int64 page table
        layer(Q.cuda(), pool_k, pool_v, _cu(sq), page_table=table.cuda().long(),
              cache_seqlens=lens.cuda())
    with pytest.raises(AssertionError):                  # page table too narrow
        layer(Q.cuda(), pool_k, pool_v, _cu(sq), page_table=table[:, :1].contiguous().cuda(),
              cache_seqlens=lens.cuda())
