"""Host metadata: the values the reference's CPU tests pin
(tests/metadata/test_row_desc.py, tests/metadata/test_launch_heuristic.py) and the
arrays the reference itself produced for the benchmark batches (meta_golden.npz)."""
import os

import numpy as np
import pytest

from megaattention_b200.metadata import (
    ROW_M_TILE, FA_M_TILE, OPROJ_M_TILE, AR_M_TILE, build_row_desc, cdiv,
    cu_seqlens_from_seqlens, oproj_task_counts, decode_oproj_slot, csym_numel,
    oscratch_numel, active_counts, LaunchConfig, choose_launch_config,
    estimate_work_ratio)
from megaattention_b200.metadata.launch_heuristic import (
    choose_launch_config_b200, estimate_work_ratio_kv)

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "meta_golden.npz"))


def test_one_shared_tile():
    assert ROW_M_TILE == FA_M_TILE == OPROJ_M_TILE == AR_M_TILE == 128
    with pytest.raises(AssertionError):
        build_row_desc([128], M_TILE=64)


def test_prefix_sums():
    cu = cu_seqlens_from_seqlens([3, 5, 2])
    assert cu.tolist() == [0, 3, 8, 10] and cu.dtype == np.int32


def test_tile_counts_and_roundtrip():
    m = build_row_desc([200, 64, 300])
    assert m.num_row_tiles == 6 and m.cu_m_blocks.tolist() == [0, 2, 3, 6]
    seqlens = [200, 64, 300, 1, 129]
    m = build_row_desc(seqlens)
    for t in range(m.num_row_tiles):
        b, mb = int(m.batch_idx[t]), int(m.m_block[t])
        assert int(m.cu_m_blocks[b]) + mb == t
        assert 0 <= mb < cdiv(seqlens[b], 128)
    for arr in (m.batch_idx, m.m_block, m.cu_m_blocks, m.cu_seqlens_q, m.cu_seqlens_k):
        assert arr.dtype == np.int32


def test_valid_m_tails():
    m = build_row_desc([200])
    assert (m.valid_m(0), m.valid_m(1)) == (128, 72)
    assert (m.q_tile_start(0), m.q_tile_start(1)) == (0, 128)
    m = build_row_desc([1, 256])
    assert m.num_row_tiles == 3
    assert [m.valid_m(t) for t in range(3)] == [1, 128, 128]


def test_q_le_k_precondition():
    m = build_row_desc([200, 64], seqlens_k=[200, 64])
    assert (m.cu_seqlens_q == m.cu_seqlens_k).all()
    m = build_row_desc([200, 64], seqlens_k=[200, 128])
    assert m.k_len(0) == 200 and m.q_len(0) == 200 and m.k_len(2) == 128
    assert m.num_row_tiles == build_row_desc([200, 64]).num_row_tiles
    with pytest.raises(AssertionError):
        build_row_desc([200, 64], seqlens_k=[200, 32])
    with pytest.raises(AssertionError):
        build_row_desc([0, 4])
    with pytest.raises(AssertionError):
        build_row_desc([])


def test_task_space():
    m = build_row_desc([512 * 128])
    assert oproj_task_counts(m.num_row_tiles, 4096, 128, 4) == (32, 8, 4096)
    n_out, n_sg, total = oproj_task_counts(5, 4100, 128, 4)
    assert n_out == 33
    seen = set()
    for slot in range(total):
        rt, nsg, base, valid = decode_oproj_slot(slot, n_sg, 4, 4100, 128)
        assert slot == rt * n_sg + nsg and base == nsg * 4 and 1 <= valid <= 4
        if nsg == n_sg - 1:
            assert valid == 1
        seen.add((rt, nsg))
    assert len(seen) == total == 5 * n_sg


def test_padded_sizes():
    m = build_row_desc([200])
    assert csym_numel(m.num_row_tiles, 4100, 128) == 2 * 128 * 33 * 128
    assert csym_numel(m.num_row_tiles, 4100, 128) > 200 * 4100
    assert oscratch_numel(3, H_local=4, D=128) == 3 * 128 * 4 * 128
    assert csym_numel(4, 4096, 128) == 512 * 4096


def test_ratio_values():
    assert abs(estimate_work_ratio(build_row_desc([2048]), 2048) - 272 / 256) < 1e-12
    meta = build_row_desc([300, 1000, 128, 4096])
    brute = 2 * sum(int(x) + 1 for x in meta.m_block) / (meta.num_row_tiles * cdiv(3072, 128))
    assert estimate_work_ratio(meta, 3072) == brute
    assert (estimate_work_ratio(build_row_desc([16384]), 2048)
            > estimate_work_ratio(build_row_desc([2048]), 2048))


def test_table_rows():
    cfg = choose_launch_config(build_row_desc([4096]), 4096, 1)
    assert isinstance(cfg, LaunchConfig) and cfg.w_ar == 0 and 1 <= cfg.sg <= 32
    bal = choose_launch_config(build_row_desc([4096, 4096]), 4096, 8)
    assert (bal.w_fa, bal.w_oproj, bal.w_ar, bal.sg) == (2, 1, 1, 4)
    fa = choose_launch_config(build_row_desc([16384]), 2048, 8)
    assert (fa.w_fa, fa.w_oproj, fa.w_ar, fa.sg) == (8, 1, 1, 4)
    one = choose_launch_config(build_row_desc([16384]), 2048, 1)
    assert (one.w_fa, one.w_oproj, one.w_ar, one.sg) == (8, 1, 0, 4)
    assert choose_launch_config(build_row_desc([128]), 200, 2).sg == 2


@pytest.mark.parametrize("key", ["a", "b", "c", "d", "e", "f"])
def test_reference_produced_arrays(key):
    sq, sk = GOLD[f"{key}.sq"], GOLD[f"{key}.sk"]
    hidden, tp, rank, H, sg = (int(x) for x in GOLD[f"{key}.args"])
    m = build_row_desc(sq, seqlens_k=sk)
    for f in ("cu_seqlens_q", "cu_seqlens_k", "cu_m_blocks", "batch_idx", "m_block"):
        got, ref = getattr(m, f), GOLD[f"{key}.{f}"]
        assert got.dtype == ref.dtype and got.shape == ref.shape and (got == ref).all(), f
    num_out, nsg, total = oproj_task_counts(m.num_row_tiles, hidden, 128, sg)
    assert [m.num_row_tiles, num_out, nsg, total, csym_numel(m.num_row_tiles, hidden, 128),
            oscratch_numel(m.num_row_tiles, H, 128)] == GOLD[f"{key}.counts"].tolist()
    a = active_counts(m.num_row_tiles, H, nsg, tp, rank)
    assert a.dtype == np.int32 and (a == GOLD[f"{key}.actv"]).all()
    cfg = choose_launch_config(m, hidden, tp)
    assert [cfg.w_fa, cfg.w_oproj, cfg.w_ar, cfg.sg] == GOLD[f"{key}.cfg"].tolist()
    assert estimate_work_ratio(m, hidden) == float(GOLD[f"{key}.ratio"][0])


def test_kv_aware_ratio_is_additional():
    sq = [6800, 2900, 1700, 1100, 600, 300]
    m = build_row_desc(sq, seqlens_k=[4 * s for s in sq])
    assert estimate_work_ratio_kv(build_row_desc(sq), 4096) == estimate_work_ratio(build_row_desc(sq), 4096)
    assert estimate_work_ratio_kv(m, 4096) > 2.0 > estimate_work_ratio(m, 4096)
    assert choose_launch_config_b200(m, 4096, 1).w_fa == 8
    assert choose_launch_config_b200(m, 4096, 8).w_fa == 2      # balanced row with an AllReduce to feed
    assert choose_launch_config(m, 4096, 8).w_fa == 2


def test_claim_order_is_longest_first_with_optional_priming():
    """Host-side order in which attention tasks are claimed (no reference counterpart: the
    reference claims in tile order): a permutation of the row tiles, longest first, stable;
    with priming the given number of shortest tiles comes first."""
    from megaattention_b200.runtime.workspace import claim_order
    meta = build_row_desc([700, 130, 300], seqlens_k=[700, 512, 300])
    nblk = []
    for t in range(meta.num_row_tiles):
        mb = int(meta.m_block[t])
        lq, lk = meta.q_len(t), meta.k_len(t)
        nblk.append(min(-(-lk // 128), -(-((mb + 1) * 128 + lk - lq) // 128)))
    order = claim_order(meta)
    assert sorted(order.tolist()) == list(range(meta.num_row_tiles)) and order.dtype == np.int32
    lens = [nblk[t] for t in order]
    assert lens == sorted(lens, reverse=True)
    primed = claim_order(meta, prime=3)
    assert sorted(primed.tolist()) == list(range(meta.num_row_tiles))
    assert [nblk[t] for t in primed[:3]] == sorted(nblk)[:3]
    rest = [nblk[t] for t in primed[3:]]
    assert rest == sorted(rest, reverse=True)
    assert claim_order(meta, prime=10 ** 6).tolist() == order[::-1].tolist()
    mixed = claim_order(meta, prime=-1)          # longest, shortest, 2nd longest, ...
    assert sorted(mixed.tolist()) == list(range(meta.num_row_tiles))
    assert mixed[0] == order[0] and mixed[1] == order[-1] and mixed[2] == order[1]


def test_b200_launch_choices_for_the_benchmark_shapes():
    """The additional B200 entry points are deterministic functions of the batch: downstream
    work first on 8 ranks and where the AllReduce dominates, interleaved claim order while
    O_proj is a sizeable share of the work, the balanced role row whenever there is an
    AllReduce to feed.  Values as calibrated by metadata/sweep_launch_config.py."""
    from megaattention_b200.metadata.launch_heuristic import (
        fa_prime_tiles_b200, launch_flags_b200)
    from megaattention_b200.workloads import WORKLOADS
    want = {("c2", 1): (0, -1, 2), ("c3", 1): (0, -1, 2), ("c3", 2): (0, -1, 2), ("c3", 4): (0, -1, 2),
            ("c3", 8): (2, -1, 2), ("c4", 8): (2, -1, 2), ("c5", 8): (2, 0, 2),
            ("long16k", 1): (0, 0, 8), ("long32k", 1): (0, 0, 8)}
    for (name, tp), (flags, order, w_fa) in want.items():
        wl = WORKLOADS[name]
        h, _ = wl.heads_local(tp)
        m = build_row_desc(wl.seqlens_q, seqlens_k=wl.seqlens_k)
        got = (launch_flags_b200(m, wl.hidden, tp, h), fa_prime_tiles_b200(m, wl.hidden, tp, h),
               choose_launch_config_b200(m, wl.hidden, tp).w_fa)
        assert got == (flags, order, w_fa), (name, tp, got)
