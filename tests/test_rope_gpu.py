"""Rotary embedding of the producer side (``ma_rope_qk``) against the CPU oracle, and the
rotated tensors through the fused layer."""
import numpy as np
import pytest
import torch

from oracle.producer_oracle import rope_oracle

pytestmark = pytest.mark.gpu


def _close(got, ref):
    d = (got.float() - ref.float()).abs()
    assert bool((d <= ref.float().abs() * 2.0 ** -7 + 1e-6).all()), float(d.max())
    assert float((d == 0).float().mean()) > 0.98


@pytest.mark.parametrize("sq,sk,H,Hkv,theta", [
    ([200, 64, 130], None, 8, 1, 10000.0),
    ([300], [700], 4, 2, 1000000.0),
    ([128, 1, 77], [384, 1, 333], 3, 3, 10000.0),
])
def test_rope_matches_the_oracle_and_leaves_the_prefix_alone(sq, sk, H, Hkv, theta):
    from megaattention_b200.runtime import rope_qk_
    skk = sq if sk is None else sk
    g = torch.Generator().manual_seed(sum(sq) + H)
    q = torch.randn(sum(sq), H, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(skk), Hkv, 128, generator=g).to(torch.bfloat16)
    qo, ko = rope_oracle(q, k, sq, skk, theta)
    qd, kd = q.cuda(), k.cuda()
    cu_q = np.concatenate([[0], np.cumsum(sq)])
    cu_k = np.concatenate([[0], np.cumsum(skk)])
    rope_qk_(qd, kd, cu_q, None if sk is None else cu_k, theta=theta)
    torch.cuda.synchronize()
    _close(qd.cpu(), qo)
    _close(kd.cpu(), ko)
    k0 = 0
    for lq, lk in zip(sq, skk):                      # cached prefix: not a bit changed
        assert torch.equal(kd[k0:k0 + lk - lq].cpu(), k[k0:k0 + lk - lq])
        k0 += lk


def test_rotated_tensors_feed_the_fused_layer():
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import FusedFaOprojArWorkspace, FusedPrefillLayer, rope_qk_
    from oracle.chain_oracle import full_chain_oracle, err_beyond_rounding
    sq, H, Hkv, hidden = [200, 130], 4, 2, 384
    g = torch.Generator().manual_seed(3)
    q = torch.randn(sum(sq), H, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(sq), Hkv, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(sq), Hkv, 128, generator=g).to(torch.bfloat16)
    W = (torch.randn(H * 128, hidden, generator=g) * (H * 128) ** -0.5).to(torch.bfloat16)
    meta = build_row_desc(sq)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, hidden, H, 128, q_per_kv=H // Hkv,
                                        max_tot_k=sum(sq), device="cuda:0")
    ws.compile()
    layer = FusedPrefillLayer(ws, W)
    cu = torch.tensor([0, 200, 330], dtype=torch.int32)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    with torch.cuda.stream(ws._stream()):
        rope_qk_(qd, kd, cu)
        layer(qd, kd, vd, cu)
    ws.check_status()
    qo, ko = rope_oracle(q, k, sq)
    _, yp, _ = full_chain_oracle(qo, ko, v, W, sq, sq)
    assert err_beyond_rounding(layer.output().cpu(), yp) <= 2e-3


def test_a_whole_layer_step_rope_attention_oproj_residual_norm():
    """The three pieces in the order a transformer layer runs them, on one stream with no
    host synchronisation in between, against the composition of their CPU oracles."""
    from megaattention_b200.metadata import build_row_desc
    from megaattention_b200.runtime import (FusedFaOprojArWorkspace, FusedPrefillLayer,
                                            residual_rmsnorm, rope_qk_)
    from oracle.chain_oracle import full_chain_oracle, err_rel
    from oracle.consumer_oracle import residual_rmsnorm_oracle
    sq, sk, H, Hkv, hidden = [150, 260], [150, 516], 4, 2, 512
    g = torch.Generator().manual_seed(11)
    q = torch.randn(sum(sq), H, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(sk), Hkv, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(sk), Hkv, 128, generator=g).to(torch.bfloat16)
    W = (torch.randn(H * 128, hidden, generator=g) * (H * 128) ** -0.5).to(torch.bfloat16)
    res = torch.randn(sum(sq), hidden, generator=g).to(torch.bfloat16)
    wn = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    meta = build_row_desc(sq, seqlens_k=sk)
    ws = FusedFaOprojArWorkspace.create(None, meta.num_row_tiles, hidden, H, 128, q_per_kv=H // Hkv,
                                        max_tot_k=sum(sk), device="cuda:0")
    ws.compile()
    layer = FusedPrefillLayer(ws, W)
    cu_q = torch.tensor([0, 150, 410], dtype=torch.int32)
    cu_k = torch.tensor([0, 150, 666], dtype=torch.int32)
    qd, kd, vd, resd = q.cuda(), k.cuda(), v.cuda(), res.cuda()
    with torch.cuda.stream(ws._stream()):
        rope_qk_(qd, kd, cu_q, cu_k, theta=1e6)
        layer(qd, kd, vd, cu_q, cu_k)
        normed, new_res = residual_rmsnorm(ws, resd, wn.cuda(), eps=1e-6, inplace=True)
    ws.check_status()
    torch.cuda.synchronize()
    qo, ko = rope_oracle(q, k, sq, sk, 1e6)
    _, _, yf = full_chain_oracle(qo, ko, v, W, sq, sk)
    ref_out, ref_res = residual_rmsnorm_oracle(yf, res, wn, 1e-6)
    assert err_rel(new_res.cpu(), ref_res) <= 8e-3
    assert err_rel(normed.cpu(), ref_out) <= 8e-3
