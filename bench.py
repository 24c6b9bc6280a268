#!/usr/bin/env python3
"""Benchmark of the fused FlashAttention -> O_proj -> AllReduce prefill kernel.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU chain on the host cores

A step is one fused launch over one batch of synthetic input (one layer of prefill).
N = 1 runs workload c2 (one GPU, tp = 1); N > 1 runs the tensor-parallel sweep c3 with
tp = N (fixed global model: strong scaling).  The printed line follows the build's bench
contract; the method mirrors the reference's benchmarks/bench_fused_fa_oproj_ar.py:75-131,
158-312 (L2 flushed before every timed launch, device time, max over ranks, the same FLOP
and byte formulas, an unfused FA + cuBLAS + NVLS-AllReduce baseline beside it).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from megaattention_b200.workloads import (  # noqa: E402
    WORKLOADS, make_rank_inputs, fa_flops, oproj_flops, ar_bytes)
from megaattention_b200.metadata import build_row_desc, choose_launch_config  # noqa: E402
from megaattention_b200.metadata.launch_heuristic import launch_flags_b200  # noqa: E402

METRIC = "fused_fa_oproj_ar_prefill_tflops"
UNIT = "TFLOP/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(tflops=float(d["bf16_tflops"]), hbm=float(d["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu), "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx),
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_chain_sample(wl, tp, rank, max_seconds_hint=25.0):
    """Time the CPU oracle on a bounded sample of the workload: whole sequences of rank
    `rank`, longest first, until the estimated cost passes the hint.  Returns
    (tflops, seconds, threads, description)."""
    from oracle.chain_oracle import full_chain_oracle
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    Q, K, V, W = make_rank_inputs(wl, tp, rank)
    h, hkv = wl.heads_local(tp)
    # pick a prefix of sequences (in batch order) worth roughly the hint at ~0.15 TFLOP/s
    budget = max_seconds_hint * 0.15e12
    cq = [0]; ck = [0]
    for a, b in zip(wl.seqlens_q, wl.seqlens_k):
        cq.append(cq[-1] + a); ck.append(ck[-1] + b)
    order = sorted(range(len(wl.seqlens_q)), key=lambda i: wl.seqlens_q[i])
    chosen, cost = [], 0.0
    for i in order:
        c = fa_flops([wl.seqlens_q[i]], h, 128, [wl.seqlens_k[i]]) + \
            oproj_flops(wl.seqlens_q[i], h * 128, wl.hidden)
        if chosen and cost + c > budget:
            continue
        chosen.append(i); cost += c
    chosen.sort()
    sq = [wl.seqlens_q[i] for i in chosen]; sk = [wl.seqlens_k[i] for i in chosen]
    Qs = torch.cat([Q[cq[i]:cq[i + 1]] for i in chosen])
    Ks = torch.cat([K[ck[i]:ck[i + 1]] for i in chosen])
    Vs = torch.cat([V[ck[i]:ck[i + 1]] for i in chosen])
    t0 = time.perf_counter()
    full_chain_oracle(Qs, Ks, Vs, W, sq, sk)
    dt = time.perf_counter() - t0
    desc = (f"{wl.name} rank {rank}/{tp}: sequences {sq} of {wl.seqlens_q} "
            f"({cost / 1e9:.1f} of {(fa_flops(wl.seqlens_q, h, 128, wl.seqlens_k) + oproj_flops(wl.tot_q, h * 128, wl.hidden)) / 1e9:.1f} GFLOP), "
            f"fp32 torch CPU oracle, {threads} threads")
    return cost / dt / 1e12, dt, threads, desc


def run_reference(args, wl, tp):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, descs = [], None
    for i in range(args.warmup + args.steps):
        v, dt, threads, desc = cpu_chain_sample(wl, tp, 0, max_seconds_hint=args.cpu_seconds)
        if i >= args.warmup:
            vals.append((v, dt))
        descs = (threads, desc)
    v = sum(x for x, _ in vals) / len(vals)
    ms = 1e3 * sum(d for _, d in vals) / len(vals)
    h, _ = wl.heads_local(tp)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{wl.name} tp{tp} (bounded CPU sample per step)",
                   "seqlens_q": wl.seqlens_q, "kv_mult": wl.kv_mult, "H_local": h,
                   "hidden": wl.hidden},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": descs[0], "kind": "port",
                         "sample": descs[1]},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None] + list(WORKLOADS))
    ap.add_argument("--tp", type=int, default=None, help="override tensor-parallel size")
    ap.add_argument("--cpu-seconds", type=float, default=20.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-unfused", action="store_true")
    ap.add_argument("--w", type=str, default=None, help="w_fa,w_oproj,w_ar override")
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--stage", default="fused", choices=["fused", "fa", "ar", "oproj"],
                    help="fa / ar: time the attention / AllReduce stage alone (profiling aid)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-p2p", action="store_true",
                    help="tp 2: reduce through multimem instead of peer loads (comparison)")
    ap.add_argument("--per-rank-heads", type=int, default=0,
                    help="experiment: every rank gets this many q heads (1 kv head), c3 sequences")
    ap.add_argument("--flags", type=int, default=None,
                    help="launch flags (2: drain downstream work first, 4: row-tile claim order)")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    tp = args.tp or max(world, 1)
    wl = WORKLOADS[args.workload or ("c2" if tp == 1 else "c3")]
    if args.per_rank_heads:
        from megaattention_b200.workloads import Workload
        wl = Workload(f"{wl.name}-h{args.per_rank_heads}", wl.seqlens_q, args.per_rank_heads * tp, tp,
                      wl.hidden, [tp], kv_mult=wl.kv_mult, per_rank_seed=True)
    if args.impl == "reference":
        if args.steps > 3:
            args.steps = 3
        args.warmup = min(args.warmup, 1)
        return run_reference(args, wl, tp)

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    W = max(args.warmup, 3)
    K = args.steps
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    import torch.distributed as dist
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        import torch.distributed._symmetric_memory as symm_mem
        group = dist.group.WORLD.group_name
        symm_mem.enable_symm_mem_for_group(group)

    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    h, hkv = wl.heads_local(tp)
    Q, Kt, V, Wo = make_rank_inputs(wl, tp, rank)
    Qh, Kh, Vh, Wh = (t.pin_memory() for t in (Q, Kt, V, Wo))
    meta = build_row_desc(wl.seqlens_q, seqlens_k=wl.seqlens_k)
    cfg = choose_launch_config(meta, wl.hidden, tp)
    w = (cfg.w_fa, cfg.w_oproj, cfg.w_ar)
    if args.w:
        w = tuple(int(x) for x in args.w.split(","))
    ws = FusedFaOprojArWorkspace.create(
        group, max_num_row_tiles=meta.num_row_tiles, hidden=wl.hidden, H_local=h, D=128,
        tp_size=tp, rank=rank, super_group_n_tiles=cfg.sg, q_per_kv=h // hkv,
        max_num_batch=meta.num_batch, max_tot_k=wl.tot_k, device=dev)
    ws.compile(w_fa=w[0], w_oproj=w[1], w_ar=w[2], num_ctas=args.ctas or None)
    ws.set_layer(meta, Qh, Kh, Vh, Wh)
    torch.cuda.synchronize()
    ws.ar_p2p = not args.no_p2p
    ws.default_flags = (args.flags if args.flags is not None
                        else launch_flags_b200(meta, wl.hidden, tp, h))

    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)   # 4 x L2
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            flush.zero_(); fn()
        torch.cuda.synchronize(); barrier()
        evs = []
        for _ in range(steps):
            flush.zero_()
            if world > 1:
                torch.cuda._sleep(200000)      # let slower ranks' queues catch up
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream); fn(); b.record(stream)
            evs.append((a, b))
        torch.cuda.synchronize(); barrier()
        ms = sum(a.elapsed_time(b) for a, b in evs) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    stage_fn = {"fused": ws.launch, "fa": ws.launch_fa_only,
                "ar": lambda: ws.launch_ar_only((args.flags or 0) & ~0xF),
                "oproj": ws.launch_oproj_only}[args.stage]
    ms_fused = timed(stage_fn, K, W)
    clocks = sampler.stop() if sampler else None
    ws.check_status()

    flops_rank = fa_flops(wl.seqlens_q, h, 128, wl.seqlens_k) + oproj_flops(wl.tot_q, h * 128, wl.hidden)
    flops_job = flops_rank * tp
    value = flops_job / (ms_fused * 1e-3) / 1e12
    S = ar_bytes(wl.tot_q, wl.hidden)
    bus = S * 2 * (tp - 1) / tp
    peaks = _peaks()
    t_comp = flops_rank / (peaks["tflops"] * 1e12)
    t_ar = bus / 770e9
    roofline = {
        "bound": "tensor" if t_comp >= t_ar else "nvlink",
        "achieved": flops_rank / (ms_fused * 1e-3) / 1e12, "peak": peaks["tflops"],
        "unit": "TFLOP/s", "frac": (flops_rank / (ms_fused * 1e-3) / 1e12) / peaks["tflops"],
        # dram read+write bytes of one launch from an ncu capture (profiles/): c2, tp 1 only
        "traffic": 147.5e6 if (wl.name == "c2" and tp == 1 and args.stage == "fused") else None,
        "traffic_unit": "bytes/launch", "peak_source": peaks["source"],
        "t_compute_ms": t_comp * 1e3, "t_allreduce_ms": t_ar * 1e3,
        "frac_of_slower_leg": max(t_comp, t_ar) * 1e3 / ms_fused,
        "nominal": {"t_compute_ms_2250tf": flops_rank / 2250e12 * 1e3,
                    "t_allreduce_ms_900gbs": bus / 900e9 * 1e3,
                    "frac": max(flops_rank / 2250e12, bus / 900e9) * 1e3 / ms_fused},
    }

    # ---- end-to-end through the public API with host buffers ------------------------
    # Every step copies its inputs from pinned host memory, launches, and reads the whole
    # result back.  On one GPU two workspaces on two streams take turns, so one step's
    # copies overlap the other's (PCIe is full duplex); with tp > 1 the steps stay on one
    # stream: two launches per rank could reach the GPUs in different orders on different
    # ranks and wait on each other.
    lanes = [(ws, torch.cuda.current_stream(dev))]
    if world == 1 and not args.no_e2e:
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):
            ws2 = FusedFaOprojArWorkspace.create(
                group, max_num_row_tiles=meta.num_row_tiles, hidden=wl.hidden, H_local=h, D=128,
                tp_size=tp, rank=rank, super_group_n_tiles=cfg.sg, q_per_kv=h // hkv,
                max_num_batch=meta.num_batch, max_tot_k=wl.tot_k, device=dev)
            ws2.compile(w_fa=w[0], w_oproj=w[1], w_ar=w[2], num_ctas=args.ctas or None)
            ws2.default_flags = ws.default_flags
        side.synchronize()
        lanes.append((ws2, side))
    host_outs = [torch.empty(ws.csym[:meta.num_row_tiles].shape, dtype=torch.bfloat16).pin_memory()
                 for _ in lanes]
    host_out = host_outs[0]
    e2e_i = [0]

    def e2e_step():
        i = e2e_i[0] % len(lanes)
        e2e_i[0] += 1
        w_i, s_i = lanes[i]
        with torch.cuda.stream(s_i):
            w_i.set_layer(meta, Qh, Kh, Vh, Wh)
            w_i.launch()
            host_outs[i].copy_(w_i.csym[:meta.num_row_tiles], non_blocking=True)

    n_e2e = 0 if args.no_e2e else max(3, min(K, 10))
    for _ in range(2 if n_e2e else 0):
        e2e_step()
    torch.cuda.synchronize(); barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    torch.cuda.synchronize(); barrier()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / max(n_e2e, 1) if n_e2e else float("nan")
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    h2d = sum(t.numel() * 2 for t in (Q, Kt, V, Wo)) + 4 * (2 * (meta.num_batch + 1) + 2 * meta.num_row_tiles + 6)
    d2h = host_out.numel() * 2
    e2e = {"value": flops_job / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
           "streams": len(lanes)}
    for w_i, _ in lanes:
        w_i.check_status()

    # ---- unfused baseline on the same box: FA kernel, cuBLAS GEMM, NVLS AllReduce ----
    unfused = None
    if not args.no_unfused:
        ms_fa = timed(ws.launch_fa_only, max(3, K // 2), 3)
        ws.check_status()
        A = ws.Oscr.view(-1, ws.K_local)[:wl.tot_q]
        Wd = Wo.to(dev)
        Y = torch.empty(wl.tot_q, wl.hidden, dtype=torch.bfloat16, device=dev)
        ms_gemm = timed(lambda: torch.matmul(A, Wd, out=Y), max(3, K // 2), 3)
        ms_ar = 0.0
        if world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            Ys = symm_mem.empty(wl.tot_q, wl.hidden, dtype=torch.bfloat16, device=dev)
            symm_mem.rendezvous(Ys, group)
            Ys.zero_()
            ms_ar_nvls = timed(lambda: torch.ops.symm_mem.multimem_all_reduce_(Ys, "sum", group),
                               max(3, K // 2), 3)
            ms_ar_nccl = timed(lambda: dist.all_reduce(Y), max(3, K // 2), 3)
            ms_ar = min(ms_ar_nvls, ms_ar_nccl)
        serial = ms_fa + ms_gemm + ms_ar
        unfused = {"fa_ms": ms_fa, "oproj_cublas_ms": ms_gemm, "allreduce_ms": ms_ar,
                   "allreduce_symm_mem_multimem_ms": ms_ar_nvls if world > 1 else 0.0,
                   "allreduce_nccl_ms": ms_ar_nccl if world > 1 else 0.0,
                   "serial_ms": serial, "ideal_ms": max(ms_fa + ms_gemm, ms_ar),
                   "ratio_serial_over_fused": serial / ms_fused,
                   "fa": "this library's attention stage alone (MA_FLAG_FA_ONLY)"}

    cpu = None
    if rank == 0 and tp == 1 and not args.no_cpu_baseline:
        v, dt, threads, desc = cpu_chain_sample(wl, tp, 0, max_seconds_hint=args.cpu_seconds)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc,
               "seconds": dt}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": tp, "steps": K,
            "warmup": W, "ms_per_step": ms_fused, "higher_is_better": True,
            "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"{wl.name} tp{tp}" + ("" if args.stage == "fused" else " (attention stage only)"), "seqlens_q": wl.seqlens_q,
                       "kv_mult": wl.kv_mult, "H_local": h, "H_kv": hkv, "hidden": wl.hidden,
                       "role_weights": list(w), "sg": cfg.sg, "launch_flags": ws.default_flags,
                       "l2": "512 MiB buffer written before every timed launch"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": K,
            "clocks": clocks, "unfused": unfused,
            "allreduce": {"S_bytes": S, "bus_bytes": bus,
                          "bus_gbs": bus / (ms_fused * 1e-3) / 1e9},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
