"""Worker of tests/test_fused_multi_gpu.py (one process per GPU, launched by torchrun).

One workspace, built once, runs a sequence of heterogeneous layers back to back with no
host-side reset (the pattern of the reference's tests/fused/test_fused_production.py:45-61,
79-123): full capacity -> one tile, long KV -> short KV, repeats; every layer is checked
against the CPU oracle (sum over ranks of the per-rank partial, one bf16 cast) and for a
clean exit; two over-capacity layers must raise AssertionError and leave the workspace
usable (test_fused_production.py:129-146).  The sequence is repeated for every AllReduce
variant the kernel has, and the run ends with the tensor-parallel benchmark workload at
full size against the oracle.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from megaattention_b200.metadata import build_row_desc
from megaattention_b200.runtime import FusedFaOprojArWorkspace
from oracle.chain_oracle import fa_oracle, oproj_oracle, err_rel, err_beyond_rounding

MAX_RT, H, QPK, HIDDEN, SG = 12, 4, 2, 640, 4
LAYERS = [
    ([1536], None), ([100], None), ([300, 200], None), ([256], [1024]), ([256], None),
    ([128, 128, 128, 128], None), ([700], [700]), ([64, 200, 130], [64, 328, 130]),
    ([1536], None), ([1], None), ([513], [1200]), ([300, 200], None),
]


def rnd(shape, seed, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(torch.bfloat16)


def inputs(layer, rank, sq, sk, h=H, qpk=QPK):
    s = 7000 + layer * 100 + rank * 10 + (0 if (h, qpk) == (H, QPK) else 50000)
    hkv = h // qpk
    return (rnd((sum(sq), h, 128), s), rnd((sum(sk), hkv, 128), s + 1),
            rnd((sum(sk), hkv, 128), s + 2), rnd((h * 128, HIDDEN), s + 3, (h * 128) ** -0.5))


def run_layers(ws, rank, world, dev, tag, layers=None, h=H, qpk=QPK):
    worst = 0.0
    for li, (sq, sk) in enumerate(LAYERS if layers is None else layers):
        sk = sq if sk is None else sk
        meta = build_row_desc(sq, seqlens_k=sk)
        mine = inputs(li, rank, sq, sk, h, qpk)
        ws.set_layer(meta, *[t.to(dev) for t in mine])
        ws.launch()
        ws.check_status()
        acc, parts = None, []
        for r in range(world):
            Q, K, V, W = inputs(li, r, sq, sk, h, qpk)
            yp = oproj_oracle(fa_oracle(Q, K, V, sq, sk), W)
            parts.append(yp)
            acc = yp.clone() if acc is None else acc + yp
        got = ws.output(meta).cpu()
        e_comp = err_beyond_rounding(got, acc, partials=parts)
        e_raw = err_rel(got, acc.to(torch.bfloat16))
        ctrl = ws.ctrl.cpu().tolist()
        tol = 8e-3 if sk != sq else 2e-3
        ok = e_comp <= tol and ctrl == [0] * 8
        print(f"[rank {rank}] {tag} layer {li} {sq}/{sk}: err_comp={e_comp:.3g} err_rel_bf16={e_raw:.3g} "
              f"ctrl={ctrl} {'OK' if ok else 'FAIL'}", flush=True)
        assert ok
        worst = max(worst, e_comp)
        # every rank must hold the same bytes
        mine_sum = got.float().sum().to(dev).double()
        lo, hi = mine_sum.clone(), mine_sum.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert float(lo) == float(hi), "ranks disagree on the reduced output"
    return worst


def run_c3(group, rank, world, dev, flags, p2p):
    """The tensor-parallel benchmark workload at full size (22600 tokens, 64 q / 8 kv heads
    split over the ranks, hidden 4096) against the CPU oracle: every rank computes the fp32
    chain of its own head slice on the CPU, the partials are summed in fp32 across the ranks
    (the reference's allreduce_reference: fused.py:207-212) and the kernel's reduced output
    is compared with that sum on every rank."""
    from megaattention_b200.workloads import WORKLOADS, make_rank_inputs
    from megaattention_b200.metadata import choose_launch_config
    from oracle.chain_oracle import bf16_half_ulp
    wl = WORKLOADS["c3"]
    h, hkv = wl.heads_local(world)
    Q, K, V, W = make_rank_inputs(wl, world, rank)
    meta = build_row_desc(wl.seqlens_q, seqlens_k=wl.seqlens_k)
    cfg = choose_launch_config(meta, wl.hidden, world)
    ws = FusedFaOprojArWorkspace.create(
        group, meta.num_row_tiles, wl.hidden, h, 128, tp_size=world, rank=rank,
        super_group_n_tiles=cfg.sg, q_per_kv=h // hkv, max_num_batch=meta.num_batch,
        max_tot_k=wl.tot_k, device=dev)
    ws.compile(w_fa=cfg.w_fa, w_oproj=cfg.w_oproj, w_ar=cfg.w_ar)
    ws.default_flags, ws.ar_p2p = flags, p2p
    ws.fa_prime_tiles = -1 if flags else 0      # interleaved claim order with "drain first"
    ws.set_layer(meta, Q.to(dev), K.to(dev), V.to(dev), W.to(dev))
    for _ in range(2):                      # the second launch starts from the first one's exit state
        ws.launch()
        ws.check_status()
    assert ws.ctrl.cpu().tolist() == [0] * 8
    torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))
    yp = oproj_oracle(fa_oracle(Q, K, V, wl.seqlens_q, wl.seqlens_k), W)
    acc = yp.to(dev)
    slack = bf16_half_ulp(yp).to(dev)
    dist.all_reduce(acc)
    dist.all_reduce(slack)
    got = ws.output(meta).float()
    e_comp = err_beyond_rounding(got, acc, extra_slack=slack)
    e_raw = err_rel(got, acc)
    ok = e_comp <= 2e-3
    print(f"[rank {rank}] c3 tp{world} flags={flags} p2p={p2p}: err_comp={e_comp:.3g} "
          f"err_rel_fp32={e_raw:.3g} {'OK' if ok else 'FAIL'}", flush=True)
    assert ok
    return e_comp


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device(f"cuda:{int(os.environ['LOCAL_RANK'])}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    import torch.distributed._symmetric_memory as symm_mem
    from megaattention_b200 import _cabi
    group = dist.group.WORLD.group_name
    symm_mem.enable_symm_mem_for_group(group)
    torch.set_num_threads(4)
    ws = FusedFaOprojArWorkspace.create(
        group, MAX_RT, HIDDEN, H, 128, tp_size=world, rank=rank, super_group_n_tiles=SG,
        q_per_kv=QPK, max_tot_k=1536, device=dev)
    ws.compile(w_fa=2, w_oproj=1, w_ar=1, num_ctas=int(os.environ.get("MA_TEST_CTAS", "24")))
    # Every scheduling variant runs the whole layer sequence on the same workspace: the
    # reference's role bias and downstream work first, and with two ranks the reduction
    # through multimem as well as through peer loads.
    variants = [("roles", 0, True), ("drain-first", _cabi.MA_FLAG_DRAIN_FIRST, True)]
    if world == 2:
        variants += [("multimem", 0, False), ("multimem drain-first", _cabi.MA_FLAG_DRAIN_FIRST, False)]
    worst = 0.0
    for tag, flags, p2p in variants:
        ws.default_flags, ws.ar_p2p = flags, p2p
        ws.fa_prime_tiles = {0: 0, 1: -1, 2: 3}[len(tag) % 3]      # every claim order gets a turn
        worst = max(worst, run_layers(ws, rank, world, dev, tag))
    # over-capacity layers: AssertionError before anything is touched, workspace stays usable
    for sq, sk in (([1537], None), ([256], [1537])):
        sk2 = sq if sk is None else sk
        meta = build_row_desc(sq, seqlens_k=sk2)
        try:
            ws.set_layer(meta, *[t.to(dev) for t in inputs(99, rank, sq, sk2)])
            raise SystemExit("over-capacity layer was accepted")
        except AssertionError:
            pass
    sq = [300, 200]
    meta = build_row_desc(sq)
    ws.set_layer(meta, *[t.to(dev) for t in inputs(2, rank, sq, sq)])
    ws.launch(); ws.check_status()
    dist.barrier()
    # Three q heads with a kv head each per rank: attention tasks pair heads that share no
    # K/V stages and the third head runs alone; flags and claim order are left to the
    # workspace's own choice for each batch.
    ws3 = FusedFaOprojArWorkspace.create(
        group, MAX_RT, HIDDEN, 3, 128, tp_size=world, rank=rank, super_group_n_tiles=SG,
        q_per_kv=1, max_tot_k=1536, device=dev)
    ws3.compile(w_fa=2, w_oproj=1, w_ar=1, num_ctas=int(os.environ.get("MA_TEST_CTAS", "24")))
    worst = max(worst, run_layers(ws3, rank, world, dev, "mha h3", layers=LAYERS[:8], h=3, qpk=1))
    dist.barrier()
    if os.environ.get("MA_TEST_C3", "1") == "1":
        for flags in (0, _cabi.MA_FLAG_DRAIN_FIRST):
            worst = max(worst, run_c3(group, rank, world, dev, flags, True))
        dist.barrier()
    print(f"[rank {rank}] ALL OK worst err_comp={worst:.3g}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
