"""The numerics model (oracle/numerics_model.py) against the reference-made fixtures: how
far a bf16-staged pipeline that is exact between its rounding points sits from the fp32
chain.  This is the floor the GPU tests compare the kernel with; here it is pinned on the
CPU so that a change to the model shows up without a GPU."""
import os

import numpy as np
import pytest
import torch

from cases import CASES, make_inputs
from oracle.chain_oracle import full_chain_oracle, err_rel, err_beyond_rounding
from oracle.numerics_model import chain_model, allreduce_model

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", list(CASES))
def test_model_sits_at_the_bf16_rounding_floor(name):
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    O, Yp, Yf = full_chain_oracle(Q, K, V, W, sq, sk)
    Om, Ym = chain_model(Q, K, V, W, sq, sk)
    # attention output: one bf16 rounding of an O that is accurate to ~1e-3 relative
    assert float((Om.float() - O).abs().max()) < 2e-2
    raw = err_rel(Ym, Yp)
    g = np.load(os.path.join(GOLD, f"chain_{name}.npz"))
    ref_yf = torch.from_numpy(g["y_final_bits"]).view(torch.bfloat16)
    raw_fix = err_rel(Ym, ref_yf)
    beyond = err_beyond_rounding(Ym, Yp)
    print(f"{name}: model err_rel vs fp32 chain {raw:.3g}, vs the reference's bf16 output "
          f"{raw_fix:.3g}, beyond rounding {beyond:.3g}")
    # the literal err_rel of a correct bf16 pipeline: above 2e-3 on most cases, never above 8e-3
    assert 1e-3 < raw < 6e-3 and raw_fix < 8e-3
    assert beyond <= (8e-3 if sk is not None else 2e-3)


def test_two_rank_model_matches_the_summed_chain():
    name = "gqa_q2"
    sq, H, hidden, qpk, sk, seed = CASES[name]
    Q, K, V, W = make_inputs(name)
    _, Yp, _ = full_chain_oracle(Q, K, V, W, sq, sk)
    # split heads (kv head 0 / 1) and W_o rows over two ranks
    parts = []
    for r in range(2):
        hs = slice(r * 2, r * 2 + 2)
        parts.append(chain_model(Q[:, hs], K[:, r:r + 1], V[:, r:r + 1],
                                 W[r * 256:(r + 1) * 256], sq, sk)[1])
    y = allreduce_model(parts)
    assert 1e-3 < err_rel(y, Yp) < 6e-3
    assert err_beyond_rounding(y, Yp, partials=[p.float() for p in parts]) <= 2e-3
