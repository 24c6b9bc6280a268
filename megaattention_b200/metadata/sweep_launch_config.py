#!/usr/bin/env python3
"""Calibration sweep of the launch configuration on the GPU(s) at hand.

    python -m megaattention_b200.metadata.sweep_launch_config                  # one GPU, tp 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m megaattention_b200.metadata.sweep_launch_config --shapes bench        # tp = ranks

Counterpart of the reference's benchmarks/sweep_launch_config.py:25-36 (12 shapes x 7
settings on 8xH200, which calibrated its two-row table, benchmarks/sweep_results.md).
Because role weights, CTA count and launch flags are launch arguments here (the reference
bakes them in at JIT time), one workspace per shape serves every setting.  For every shape
the fused launch is timed (L2 flushed before each launch, CUDA events, max over ranks) for
each (w_fa, w_oproj, w_ar) x launch flags x CTA count, and the table printed at the end
lists the best setting, the time of the reference-compatible default and of the setting
``choose_launch_config_b200`` / ``launch_flags_b200`` pick.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from megaattention_b200 import _cabi  # noqa: E402
from megaattention_b200.metadata import build_row_desc, choose_launch_config  # noqa: E402
from megaattention_b200.metadata.launch_heuristic import (  # noqa: E402
    choose_launch_config_b200, launch_flags_b200, num_ctas_b200, fa_prime_tiles_b200,
    estimate_work_ratio_kv)
from megaattention_b200.workloads import WORKLOADS  # noqa: E402

# (seqlens, H_local, hidden, kv_mult): the reference's twelve shapes ...
REF_SHAPES = [
    ([2048, 2048], 8, 2048, 1), ([1024] * 4, 16, 2048, 1), ([4096, 4096], 8, 4096, 1),
    ([8192], 8, 2048, 1), ([2048] * 8, 8, 2048, 1), ([8192, 8192], 8, 2048, 1),
    ([8192, 8192], 8, 4096, 1), ([8192, 8192], 16, 7168, 1), ([16384], 8, 2048, 1),
    ([16384], 16, 4096, 1), ([16384, 16384], 8, 2048, 1), ([32768], 8, 2048, 1),
]
# ... and the benchmark workloads' per-rank shapes (8 q heads / 1 kv head unless noted)
BENCH_SHAPES = [
    (WORKLOADS["c2"].seqlens_q, 8, 4096, 1), (WORKLOADS["c3"].seqlens_q, 8, 4096, 1),
    (WORKLOADS["c5"].seqlens_q, 8, 4096, 4),
]
WEIGHTS = [(2, 1, 1), (4, 1, 1), (8, 1, 1), (4, 2, 1), (1, 1, 1)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="all", choices=["all", "ref", "bench"])
    ap.add_argument("--iters", type=int, default=3, help="timed launches per setting per pass")
    ap.add_argument("--passes", type=int, default=5)
    ap.add_argument("--json", default=None, help="also write one JSON line per measurement here")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device(f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}")
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD.group_name
        symm_mem.enable_symm_mem_for_group(group)
    from megaattention_b200.runtime import FusedFaOprojArWorkspace

    shapes = {"all": REF_SHAPES + BENCH_SHAPES, "ref": REF_SHAPES, "bench": BENCH_SHAPES}[args.shapes]
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    gate = torch.zeros(1, device=dev)
    stream = torch.cuda.current_stream()
    jf = open(args.json, "w") if (args.json and rank == 0) else None
    flag_sets = [0, _cabi.MA_FLAG_DRAIN_FIRST]
    rows = []
    for seqlens, H, hidden, kvm in shapes:
        sk = [kvm * s for s in seqlens]
        meta = build_row_desc(seqlens, seqlens_k=sk)
        g = torch.Generator(device=dev).manual_seed(1 + rank)
        Q = torch.randn(sum(seqlens), H, 128, device=dev, dtype=torch.bfloat16, generator=g)
        Kt = torch.randn(sum(sk), 1, 128, device=dev, dtype=torch.bfloat16, generator=g)
        V = torch.randn(sum(sk), 1, 128, device=dev, dtype=torch.bfloat16, generator=g)
        Wo = torch.randn(H * 128, hidden, device=dev, dtype=torch.bfloat16, generator=g) * (H * 128 * world) ** -0.5
        ws = FusedFaOprojArWorkspace.create(
            group, meta.num_row_tiles, hidden, H, 128, tp_size=world, rank=rank,
            q_per_kv=H, max_num_batch=meta.num_batch, max_tot_k=sum(sk), device=dev)
        ws.compile()
        ws.set_layer(meta, Q, Kt, V, Wo)
        torch.cuda.synchronize()
        sms = torch.cuda.get_device_properties(dev).multi_processor_count

        def time_setting(w, flags, ctas, order, iters):
            if ws.fa_prime_tiles != order:       # claim order of the attention tasks
                ws.fa_prime_tiles = order
                ws.set_meta(meta)
            ws._args = _cabi.LaunchArgs(w[0], w[1], w[2] if world > 1 else 0, ctas, 0)
            evs = []
            for i in range(1 + iters):
                flush.zero_()
                if world > 1:
                    torch.cuda._sleep(1000000)
                    dist.all_reduce(gate)      # the ranks leave it together: aligned starts
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream); ws.launch(flags=flags); b.record(stream)
                if i >= 1:
                    evs.append((a, b))
            torch.cuda.synchronize()
            ws.check_status()
            ms = sum(a.elapsed_time(b) for a, b in evs) / len(evs)
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

        ref_cfg = choose_launch_config(meta, hidden, world)
        b200 = choose_launch_config_b200(meta, hidden, world)
        b200_flags = launch_flags_b200(meta, hidden, world, H)
        b200_ctas = num_ctas_b200(meta, hidden, world, H, sms)
        b200_order = fa_prime_tiles_b200(meta, hidden, world, H)
        name = f"{','.join(map(str, seqlens)) if len(set(seqlens)) > 1 or len(seqlens) < 3 else f'{seqlens[0]}x{len(seqlens)}'}" \
               f"{'' if kvm == 1 else f' k={kvm}q'} h{H} hid{hidden}"
        settings = []
        for w in WEIGHTS:
            for flags in flag_sets:
                for ctas in (sms, sms - 4, sms - 16):
                    if ctas != sms and (w != WEIGHTS[0] and w != WEIGHTS[1]):
                        continue
                    settings.append((w, flags, ctas, 0))
                # claim orders other than longest-first: long and short row tiles alternating,
                # 24 short row tiles first
                if w == WEIGHTS[0]:
                    settings += [(w, flags, sms, -1), (w, flags, sms, 24)]
        k_ref = ("reference default", (ref_cfg.w_fa, ref_cfg.w_oproj, ref_cfg.w_ar), 0, sms, 0)
        k_b200 = ("b200 choice", (b200.w_fa, b200.w_oproj, b200.w_ar), b200_flags, b200_ctas,
                  b200_order)
        # The clock drifts under sustained load, so every setting is timed once per pass, in
        # the same order, over several passes, and the median over the passes is kept.
        samples = {}
        for _ in range(args.passes):
            for key in settings + [k_ref, k_b200]:
                w, flags, ctas, order = key[-4:]
                samples.setdefault(key, []).append(time_setting(w, flags, ctas, order, args.iters))
        med = {k: sorted(v)[len(v) // 2] for k, v in samples.items()}
        res = {k: med[k] for k in settings}
        t_ref, t_b200 = med[k_ref], med[k_b200]
        if jf:
            for k in settings:
                jf.write(json.dumps({"shape": name, "tp": world, "w": k[0], "flags": k[1],
                                     "ctas": k[2], "order": k[3], "ms": res[k],
                                     "passes": samples[k]}) + "\n")
        best = min(res, key=res.get)
        rows.append((name, estimate_work_ratio_kv(meta, hidden), best, res[best], t_ref, t_b200,
                     (b200.w_fa, b200.w_oproj, b200.w_ar), b200_flags, b200_ctas, b200_order))
        if rank == 0:
            print(f"{name}: best {best} {res[best]:.4f} ms, reference default {t_ref:.4f} ms, "
                  f"b200 choice {t_b200:.4f} ms", flush=True)
        del ws, Q, Kt, V, Wo
        torch.cuda.empty_cache()
    if rank == 0:
        print(f"\n| shape (tp {world}) | r_kv | best (w), flags, CTAs, order | best ms | reference default ms | "
              f"b200 choice | b200 ms | b200 / best |")
        print("|---|---|---|---|---|---|---|---|")
        for name, r, best, tb, tr, t2, w2, f2, c2, o2 in rows:
            print(f"| {name} | {r:.2f} | {best[0]}, {best[1]}, {best[2]}, {best[3]} | {tb:.4f} | {tr:.4f} | "
                  f"{w2}, {f2}, {c2}, {o2} | {t2:.4f} | {t2 / tb:.3f} |")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
