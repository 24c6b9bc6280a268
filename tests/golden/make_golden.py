"""Regenerate ``tests/golden/chain_*.npz`` from the reference's own oracle module.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports ``mega_attention.reference.fused`` and ``mega_attention.metadata`` from
``<reference>/src`` and stores, per case of ``cases.py``: the attention output ``O``
(fp32), the chained output ``Y_final`` (bf16 bit pattern) and a SHA-256 of the input
bits (to catch generator drift).  It also stores the host-metadata arrays the reference
computes for a few batches (``meta_golden.npz``).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import CASES, make_inputs, digest  # noqa: E402


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from mega_attention.metadata.row_desc import (
        build_row_desc, oproj_task_counts, active_counts, csym_numel, oscratch_numel)
    from mega_attention.metadata.launch_heuristic import (
        estimate_work_ratio, choose_launch_config)
    from mega_attention.reference.fused import full_chain_reference, make_paged_kv

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name, (sq, H, hidden, qpk, sk, seed) in CASES.items():
        Q, K, V, W = make_inputs(name)
        meta = build_row_desc(sq, seqlens_k=sk)
        O, Yp, Yf = full_chain_reference(Q, K, V, W, meta)
        out = dict(y_final_bits=Yf.view(torch.int16).numpy(),
                   input_sha256=np.frombuffer(digest(Q, K, V, W).encode(), dtype=np.uint8))
        if name == "c1":
            out["o_rowsum"] = O.double().sum(dim=2).numpy()
            out["yp_rowsum"] = Yp.double().sum(dim=1).numpy()
        else:
            out["o"] = O.numpy()
        np.savez_compressed(os.path.join(HERE, f"chain_{name}.npz"), **out)
        print(name, tuple(Yf.shape), float(Yf.float().abs().max()))

    # paged-KV packer: page table and checksums of the caches for one batch
    Q, K, V, W = make_inputs("chunk_gqa_q4")
    sk = CASES["chunk_gqa_q4"][4]
    Kc, Vc, table, lens = make_paged_kv(K, V, sk, num_pages=sum((s + 127) // 128 for s in sk) + 3,
                                        shuffle=True, seed=5)
    np.savez_compressed(os.path.join(HERE, "paged_golden.npz"), page_table=table.numpy(),
                        cache_seqlens=lens.numpy(),
                        k_rowsum=Kc.double().sum(dim=(1, 2, 3)).numpy(),
                        v_rowsum=Vc.double().sum(dim=(1, 2, 3)).numpy())

    # host metadata: arrays and scalars for a few batches / shapes
    md = {}
    batches = {
        "a": ([200, 64, 300], None, 4096, 1, 0, 8, 4),
        "b": ([6800, 2900, 1700, 1100, 600, 300], None, 4096, 1, 0, 8, 4),
        "c": ([7500, 4100, 3300, 2600, 2000, 1500, 1000, 600], None, 4096, 8, 3, 8, 4),
        "d": ([6800, 2900, 1700, 1100, 600, 300],
              [27200, 11600, 6800, 4400, 2400, 1200], 4096, 8, 5, 8, 4),
        "e": ([1, 129, 4100], [1, 300, 4100], 4100, 4, 1, 12, 3),
        "f": ([32768], None, 2048, 2, 1, 8, 4),
    }
    for key, (sq, sk, hidden, tp, rank, H, sg) in batches.items():
        m = build_row_desc(sq, seqlens_k=sk)
        for f in ("cu_seqlens_q", "cu_seqlens_k", "cu_m_blocks", "batch_idx", "m_block"):
            md[f"{key}.{f}"] = getattr(m, f)
        num_out, nsg, total = oproj_task_counts(m.num_row_tiles, hidden, 128, sg)
        md[f"{key}.counts"] = np.array([m.num_row_tiles, num_out, nsg, total,
                                        csym_numel(m.num_row_tiles, hidden, 128),
                                        oscratch_numel(m.num_row_tiles, H, 128)], dtype=np.int64)
        md[f"{key}.actv"] = active_counts(m.num_row_tiles, H, nsg, tp, rank)
        cfg = choose_launch_config(m, hidden, tp)
        md[f"{key}.cfg"] = np.array([cfg.w_fa, cfg.w_oproj, cfg.w_ar, cfg.sg], dtype=np.int64)
        md[f"{key}.ratio"] = np.array([estimate_work_ratio(m, hidden)], dtype=np.float64)
        md[f"{key}.args"] = np.array([hidden, tp, rank, H, sg], dtype=np.int64)
        md[f"{key}.sq"] = np.array(sq, dtype=np.int64)
        md[f"{key}.sk"] = np.array(sq if sk is None else sk, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "meta_golden.npz"), **md)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
