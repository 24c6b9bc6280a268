"""The CPU oracle against fixtures produced by the reference's own oracle module
(tests/golden/make_golden.py), and the fixtures' input digests against this machine's
generators."""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs, digest
from oracle.chain_oracle import (full_chain_oracle, o_scratch_oracle, tile_coords,
                                 untile_csym, err_rel, make_paged_kv)

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, f"chain_{name}.npz"))


@pytest.mark.parametrize("name", list(CASES))
def test_oracle_matches_reference_fixture(name):
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    g = _load(name)
    assert digest(Q, K, V, W) == bytes(g["input_sha256"]).decode(), "input generator drift"
    O, Yp, Yf = full_chain_oracle(Q, K, V, W, sq, sk)
    ref_yf = torch.from_numpy(g["y_final_bits"]).view(torch.bfloat16)
    # fp32 attention: same math, different summation order -> ~1e-6 relative
    if "o" in g:
        ref_o = torch.from_numpy(g["o"])
        assert err_rel(O, ref_o) < 2e-5
    else:
        assert np.allclose(O.double().sum(dim=2).numpy(), g["o_rowsum"], rtol=0, atol=2e-4)
        assert np.allclose(Yp.double().sum(dim=1).numpy(), g["yp_rowsum"], rtol=0, atol=2e-3)
    # chained bf16 output: identical except where fp32 noise crosses a rounding boundary
    diff = (Yf.float() - ref_yf.float()).abs()
    # (outputs near zero are cancellation results: allow the fp32 noise floor there)
    ulp = torch.clamp(ref_yf.float().abs() * 2.0 ** -7, min=2e-5)
    assert bool((diff <= ulp).all()), "more than one bf16 ulp away from the reference"
    assert float((diff > 0).float().mean()) < 2e-3


def test_tile_helpers_roundtrip():
    sq = [200, 64, 130]
    tiles = tile_coords(sq)
    assert tiles == [(0, 128), (128, 72), (200, 64), (264, 128), (392, 2)]
    O = torch.randn(sum(sq), 2, 128)
    scr = o_scratch_oracle(O, sq)
    assert scr.shape == (5, 128, 2, 128)
    assert float(scr[1, 72:].abs().max()) == 0.0
    assert torch.equal(scr[4, :2], O[392:394])
    hidden = 200
    Y = torch.randn(sum(sq), hidden)
    csym = torch.full((5, 128, 2, 128), -7.0)
    for t, (s, vm) in enumerate(tiles):
        csym.view(5, 128, 256)[t, :vm, :hidden] = Y[s:s + vm]
    assert torch.equal(untile_csym(csym, sq, hidden), Y)


def test_paged_packer_matches_reference_fixture():
    g = np.load(os.path.join(GOLD, "paged_golden.npz"))
    Q, K, V, W = make_inputs("chunk_gqa_q4")
    sk = CASES["chunk_gqa_q4"][4]
    pages = sum((s + 127) // 128 for s in sk) + 3
    Kc, Vc, table, lens = make_paged_kv(K, V, sk, num_pages=pages, shuffle=True, seed=5)
    assert (table.numpy() == g["page_table"]).all() and table.dtype == torch.int32
    assert (lens.numpy() == g["cache_seqlens"]).all()
    assert np.array_equal(Kc.double().sum(dim=(1, 2, 3)).numpy(), g["k_rowsum"])
    assert np.array_equal(Vc.double().sum(dim=(1, 2, 3)).numpy(), g["v_rowsum"])
    # gathering the pages back gives the packed tensors
    off = 0
    for b, lk in enumerate(sk):
        for i in range((lk + 127) // 128):
            n = min(128, lk - i * 128)
            assert torch.equal(Kc[int(table[b, i]), :n], K[off + i * 128: off + i * 128 + n])
        off += lk
