"""World-size-2 host-side checks on CPU ranks (gloo): the per-rank slicing of the global
model, the owner arithmetic of the AllReduce slots, and the cross-rank reduction of the
oracle (fp32 all_reduce then one bf16 cast, reference fused.py:207-212) against the
single-rank chain over the whole model."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from megaattention_b200.metadata import active_counts, build_row_desc, oproj_task_counts
from megaattention_b200.workloads import Workload, make_rank_inputs


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


WL = Workload("mini", [150, 70], 4, 2, 320, [1, 2])


def _rank_main(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle.chain_oracle import fa_oracle, oproj_oracle
    torch.set_num_threads(2)
    Q, K, V, W = make_rank_inputs(WL, world, rank)
    yp = oproj_oracle(fa_oracle(Q, K, V, WL.seqlens_q, WL.seqlens_k), W)
    acc = yp.float().clone()
    dist.all_reduce(acc, op=dist.ReduceOp.SUM)
    y = acc.to(torch.bfloat16)
    # every rank must hold the same reduced output
    gathered = [torch.empty_like(y) for _ in range(world)]
    dist.all_gather(gathered, y)
    same = all(torch.equal(gathered[0], g) for g in gathered)
    # slot ownership: each slot has exactly one owner and the counts add up
    meta = build_row_desc(WL.seqlens_q)
    num_out, nsg, total = oproj_task_counts(meta.num_row_tiles, WL.hidden, 128, 2)
    actv = active_counts(meta.num_row_tiles, Q.shape[1], nsg, world, rank)
    owned = torch.tensor([int(actv[5])])
    dist.all_reduce(owned)
    if rank == 0:
        torch.save({"y": y, "same": same, "owned": int(owned), "total": total}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_cpu_ranks_reduce_to_the_single_rank_chain(tmp_path):
    out = str(tmp_path / "r0.pt")
    for attempt in range(5):   # the probed port can be taken before the ranks bind it
        try:
            mp.spawn(_rank_main, args=(2, _free_port(), out), nprocs=2, join=True)
            break
        except Exception:
            if attempt == 4:
                raise
    res = torch.load(out)
    assert res["same"] and res["owned"] == res["total"]
    from oracle.chain_oracle import full_chain_oracle
    Q, K, V, W = make_rank_inputs(WL, 1, 0)
    _, yp, yf = full_chain_oracle(Q, K, V, W, WL.seqlens_q, WL.seqlens_k)
    d = (res["y"].float() - yf.float()).abs()
    ulp = torch.clamp(yf.float().abs() * 2.0 ** -7, min=2e-5)
    assert bool((d <= ulp).all())


def test_rank_slices_tile_the_global_model():
    for tp in (1, 2):
        parts = [make_rank_inputs(WL, tp, r) for r in range(tp)]
        Q = torch.cat([p[0] for p in parts], dim=1)
        W = torch.cat([p[3] for p in parts], dim=0)
        Qg, Kg, Vg, Wg = make_rank_inputs(WL, 1, 0)
        assert torch.equal(Q, Qg) and torch.equal(W, Wg)
        Kc = torch.cat([p[1] for p in parts], dim=1)
        assert torch.equal(Kc, Kg)
