#!/usr/bin/env python3
"""Benchmark of the fused FlashAttention -> O_proj -> AllReduce prefill kernel.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU chain on the host cores

A step is one fused launch over one batch of synthetic input (one layer of prefill).
N = 1 runs workload c2 (one GPU, tp = 1); N > 1 runs the tensor-parallel sweep c3 with
tp = N (fixed global model: strong scaling; the N = 1 line carries c3 at tp 1 as
``scaling_anchor``).  The method mirrors the reference's
benchmarks/bench_fused_fa_oproj_ar.py:75-131, 158-312: L2 flushed before every timed
launch, device time, max over ranks, the same FLOP and byte formulas, an unfused
FA + cuBLAS + AllReduce baseline beside it, and the fused output cross-checked against
that baseline's (``parity``).
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
from megaattention_b200.metadata.launch_heuristic import (  # noqa: E402
    launch_flags_b200, fa_prime_tiles_b200)

METRIC = "fused_fa_oproj_ar_prefill_tflops"
UNIT = "TFLOP/s"
NVLINK_GBS_NOMINAL = 900.0      # per direction per GPU
NVLINK_GBS_PEER_COPY = 770.0    # peer copy rate measured on this pool
TENSOR_TFLOPS_NOMINAL = 2250.0  # dense bf16


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


def workload_name(wl, tp):
    return f"{wl.name} tp{tp}"


def cpu_chain_sample(wl, tp, rank, max_seconds_hint=25.0):
    """Time the CPU oracle on a bounded sample of the workload: whole sequences of rank
    `rank`, shortest first, until the estimated cost passes the hint.  Returns
    (tflops, seconds, threads, description, chosen sequence indices, Y_partial fp32)."""
    from oracle.chain_oracle import full_chain_oracle
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    Q, K, V, W = make_rank_inputs(wl, tp, rank)
    h, hkv = wl.heads_local(tp)
    # pick sequences worth roughly the hint at ~0.15 TFLOP/s
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
    _, Yp, _ = full_chain_oracle(Qs, Ks, Vs, W, sq, sk)
    dt = time.perf_counter() - t0
    desc = (f"{wl.name} rank {rank}/{tp}: sequences {sq} of {wl.seqlens_q} "
            f"({cost / 1e9:.1f} of {(fa_flops(wl.seqlens_q, h, 128, wl.seqlens_k) + oproj_flops(wl.tot_q, h * 128, wl.hidden)) / 1e9:.1f} GFLOP), "
            f"fp32 torch CPU oracle, {threads} threads")
    return cost / dt / 1e12, dt, threads, desc, chosen, Yp


def run_reference(args, wl, tp):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, descs = [], None
    for i in range(args.warmup + args.steps):
        v, dt, threads, desc, _, _ = cpu_chain_sample(wl, tp, 0, max_seconds_hint=args.cpu_seconds)
        if i >= args.warmup:
            vals.append((v, dt))
        descs = (threads, desc)
    v = sum(x for x, _ in vals) / len(vals)
    ms = 1e3 * sum(d for _, d in vals) / len(vals)
    h, hkv = wl.heads_local(tp)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(wl, tp), "seqlens_q": wl.seqlens_q,
                   "kv_mult": wl.kv_mult, "H_local": h, "H_kv": hkv, "hidden": wl.hidden},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": descs[0], "kind": "port",
                         "sample": descs[1]},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- error figures (device)
def _half_ulp_bf16(x):
    a = x.float().abs().clamp_min(2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(a)) - 8.0)


def _err_figures(got_bf16, ref_fp32, slack_extra=None):
    """``err_rel`` = max|got - bf16(ref)| / max|ref| (the reference bench's figure,
    benchmarks/bench_fused_fa_oproj_ar.py:259-270) and the same maximum taken beyond the
    rounding any bf16 result carries (half a bf16 ulp of the fp32 value, plus the ranks'
    partials' half-ulps when given)."""
    g = got_bf16.float()
    ref_max = float(ref_fp32.abs().max().clamp_min(1e-30))
    raw = float((g - ref_fp32.to(torch.bfloat16).float()).abs().max()) / ref_max
    slack = _half_ulp_bf16(ref_fp32)
    if slack_extra is not None:
        slack = slack + slack_extra
    beyond = float(((g - ref_fp32).abs() - slack).clamp_min(0).max()) / ref_max
    return raw, beyond, ref_max


def library_attention(dev):
    """The attention leg of the unfused baseline from a library, as in the reference's
    bench (flash_attn_varlen_func, bench_fused_fa_oproj_ar.py:43,247): flash-attn if its
    kernels run on this GPU, else torch's scaled_dot_product_attention per sequence."""
    try:
        from flash_attn import flash_attn_varlen_func
        q = torch.randn(256, 2, 128, device=dev, dtype=torch.bfloat16)
        cu = torch.tensor([0, 256], device=dev, dtype=torch.int32)
        flash_attn_varlen_func(q, q[:, :1].contiguous(), q[:, :1].contiguous(), cu, cu, 256, 256,
                               causal=True)
        torch.cuda.synchronize(dev)

        def run(Q, K, V, cu_q, cu_k, sq, sk):
            return flash_attn_varlen_func(Q, K, V, cu_q, cu_k, max(sq), max(sk), causal=True)
        return "flash_attn %s flash_attn_varlen_func" % __import__("flash_attn").__version__, run
    except Exception:
        import torch.nn.functional as F

        def run(Q, K, V, cu_q, cu_k, sq, sk):
            out = torch.empty_like(Q)
            q0 = k0 = 0
            for lq, lk in zip(sq, sk):
                q = Q[q0:q0 + lq].transpose(0, 1)[None]
                k = K[k0:k0 + lk].transpose(0, 1)[None]
                v = V[k0:k0 + lk].transpose(0, 1)[None]
                if lq == lk:
                    o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                else:        # causal mask aligned bottom-right
                    keep = (torch.arange(lk, device=Q.device)[None, :]
                            <= torch.arange(lq, device=Q.device)[:, None] + (lk - lq))
                    o = F.scaled_dot_product_attention(q, k, v, attn_mask=keep, enable_gqa=True)
                out[q0:q0 + lq] = o[0].transpose(0, 1)
                q0 += lq; k0 += lk
            return out
        return "torch %s scaled_dot_product_attention per sequence" % torch.__version__, run


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
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-anchor", action="store_true")
    # launch configuration (defaults: the reference heuristic's role weights, this library's
    # launch flags); the sweep summarised under profiles/ was made with these
    ap.add_argument("--w", type=str, default=None, help="w_fa,w_oproj,w_ar")
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--flags", type=int, default=None, help="launch flags (MA_FLAG_* bits)")
    ap.add_argument("--prime", type=int, default=None,
                    help="shortest row tiles whose attention is claimed first (workspace.fa_prime_tiles)")
    ap.add_argument("--stage", default="fused", choices=["fused", "fa", "ar", "oproj", "noar"],
                    help="time one stage of the kernel alone (what the profiles/ captures ran)")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    tp = args.tp or max(world, 1)
    wl = WORKLOADS[args.workload or ("c2" if tp == 1 else "c3")]
    if args.impl == "reference":
        if args.steps > 3:
            args.steps = 3
        args.warmup = min(args.warmup, 1)
        return run_reference(args, wl, tp)

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    assert not (args.stage == "ar" and tp == 1), "--stage ar needs more than one GPU"
    assert not (args.stage == "oproj" and tp > 1), "--stage oproj is single-GPU"
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

    from megaattention_b200 import _cabi
    from megaattention_b200.runtime import FusedFaOprojArWorkspace
    h, hkv = wl.heads_local(tp)
    Q, Kt, V, Wo = make_rank_inputs(wl, tp, rank)
    Qh, Kh, Vh, Wh = (t.pin_memory() for t in (Q, Kt, V, Wo))
    meta = build_row_desc(wl.seqlens_q, seqlens_k=wl.seqlens_k)
    cfg = choose_launch_config(meta, wl.hidden, tp)
    w = (cfg.w_fa, cfg.w_oproj, cfg.w_ar)
    if args.w:
        w = tuple(int(x) for x in args.w.split(","))
    flags = args.flags if args.flags is not None else launch_flags_b200(meta, wl.hidden, tp, h)
    prime = args.prime if args.prime is not None else fa_prime_tiles_b200(meta, wl.hidden, tp, h)

    def make_ws():
        x = FusedFaOprojArWorkspace.create(
            group, max_num_row_tiles=meta.num_row_tiles, hidden=wl.hidden, H_local=h, D=128,
            tp_size=tp, rank=rank, super_group_n_tiles=cfg.sg, q_per_kv=h // hkv,
            max_num_batch=meta.num_batch, max_tot_k=wl.tot_k, device=dev)
        x.compile(w_fa=w[0], w_oproj=w[1], w_ar=w[2], num_ctas=args.ctas or None)
        x.default_flags = flags
        x.fa_prime_tiles = prime
        return x

    ws = make_ws()
    ws.set_layer(meta, Qh, Kh, Vh, Wh)
    torch.cuda.synchronize()

    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)   # 4 x L2
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()

    gate = torch.zeros(1, device=dev)

    def align():
        """Start the ranks' next launch together: a short device-side sleep absorbs the host's
        enqueue jitter, then a tiny all-reduce, which ends on all ranks at the same moment, is
        the last thing on the stream before the timed launch.  Without it a rank whose host
        was late starts late, and the other ranks' launches (which wait for its partial sums)
        are charged for the delay."""
        if world > 1:
            torch.cuda._sleep(1000000)
            dist.all_reduce(gate)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            flush.zero_(); align(); fn()
        torch.cuda.synchronize(); barrier()
        evs = []
        for _ in range(steps):
            flush.zero_()
            align()
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
                "ar": lambda: ws.launch_ar_only(flags & ~0xFF),
                "noar": lambda: ws.launch(flags=(flags | _cabi.MA_FLAG_NO_AR)),
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
    # Roofline: the slower of the compute leg (FLOPs at the bf16 tensor peak) and the
    # AllReduce leg (bus bytes at 900 GB/s per direction).  Which leg is slower is decided
    # at nominal peaks, as the target is stated; the figure reported against the measured
    # tensor peak is kept next to it.
    t_comp_nom = flops_rank / (TENSOR_TFLOPS_NOMINAL * 1e12)
    t_comp_meas = flops_rank / (peaks["tflops"] * 1e12)
    t_ar_nom = bus / (NVLINK_GBS_NOMINAL * 1e9)
    tensor_achieved = flops_rank / (ms_fused * 1e-3) / 1e12
    if t_ar_nom > t_comp_nom:
        roofline = {"bound": "nvlink", "achieved": bus / (ms_fused * 1e-3) / 1e9,
                    "peak": NVLINK_GBS_NOMINAL, "unit": "GB/s",
                    "frac": t_ar_nom * 1e3 / ms_fused, "peak_source": "nominal per direction"}
    else:
        roofline = {"bound": "tensor", "achieved": tensor_achieved, "peak": peaks["tflops"],
                    "unit": "TFLOP/s", "frac": tensor_achieved / peaks["tflops"],
                    "peak_source": peaks["source"]}
    roofline.update({
        # dram read+write bytes of one launch from an ncu capture (profiles/): c2, tp 1 only
        "traffic": 141.9e6 if (wl.name == "c2" and tp == 1 and args.stage == "fused") else None,
        "traffic_unit": "bytes/launch",
        "tensor_tflops": tensor_achieved, "tensor_frac_of_measured": tensor_achieved / peaks["tflops"],
        "tensor_frac_of_nominal": tensor_achieved / TENSOR_TFLOPS_NOMINAL,
        "t_compute_ms_nominal": t_comp_nom * 1e3, "t_compute_ms_measured_peak": t_comp_meas * 1e3,
        "t_allreduce_ms_900gbs": t_ar_nom * 1e3,
        "frac_of_slower_leg_nominal": max(t_comp_nom, t_ar_nom) * 1e3 / ms_fused,
        "frac_of_slower_leg_measured": max(t_comp_meas, bus / (NVLINK_GBS_PEER_COPY * 1e9)) * 1e3 / ms_fused,
    })

    # ---- strong-scaling anchor: the tensor-parallel workload on one GPU ---------------
    anchor = None
    if tp == 1 and args.workload is None and args.stage == "fused" and not args.no_anchor:
        wa = WORKLOADS["c3"]
        ha, hkva = wa.heads_local(1)
        Qa, Ka, Va, Wa = make_rank_inputs(wa, 1, 0)
        ma = build_row_desc(wa.seqlens_q, seqlens_k=wa.seqlens_k)
        ca = choose_launch_config(ma, wa.hidden, 1)
        wsa = FusedFaOprojArWorkspace.create(
            None, ma.num_row_tiles, wa.hidden, ha, 128, super_group_n_tiles=ca.sg,
            q_per_kv=ha // hkva, max_num_batch=ma.num_batch, max_tot_k=wa.tot_k, device=dev)
        wsa.compile(w_fa=ca.w_fa, w_oproj=ca.w_oproj, w_ar=0)
        wsa.set_layer(ma, Qa, Ka, Va, Wa)
        ms_a = timed(wsa.launch, max(3, min(K, 10)), 3)
        wsa.check_status()
        fl_a = fa_flops(wa.seqlens_q, ha, 128, wa.seqlens_k) + oproj_flops(wa.tot_q, ha * 128, wa.hidden)
        anchor = {"workload": workload_name(wa, 1), "ms": ms_a, "tflops": fl_a / (ms_a * 1e-3) / 1e12,
                  "frac_of_measured_peak": fl_a / (ms_a * 1e-3) / 1e12 / peaks["tflops"]}
        del wsa, Qa, Ka, Va, Wa

    # ---- end-to-end through the public API with host buffers ------------------------
    # Every step copies its inputs from pinned host memory, launches, and reads the result
    # back: the whole output on one GPU, this rank's 1/tp share of the rows (the output is
    # replicated) with tp > 1.  Two workspaces on two streams take turns, so one step's
    # copies overlap the other's (PCIe is full duplex); each launch waits for the previous
    # one, so the ranks run their launches in the same order.
    lanes = [(ws, torch.cuda.current_stream(dev))]
    if not args.no_e2e:
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):
            ws2 = make_ws()
        side.synchronize()
        lanes.append((ws2, side))
    R = meta.num_row_tiles
    r_lo, r_hi = (rank * R) // tp, ((rank + 1) * R) // tp
    host_outs = [torch.empty(ws.csym[r_lo:r_hi].shape, dtype=torch.bfloat16).pin_memory()
                 for _ in lanes]
    e2e_i = [0]
    last_kernel = [None]

    def e2e_step():
        i = e2e_i[0] % len(lanes)
        e2e_i[0] += 1
        w_i, s_i = lanes[i]
        with torch.cuda.stream(s_i):
            w_i.set_layer(meta, Qh, Kh, Vh, Wh)
            if last_kernel[0] is not None:
                s_i.wait_event(last_kernel[0])
            w_i.launch()
            ev = torch.cuda.Event()
            ev.record(s_i)
            last_kernel[0] = ev
            host_outs[i].copy_(w_i.csym[r_lo:r_hi], non_blocking=True)

    n_e2e = 0 if args.no_e2e else max(4, min(K, 10))
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
    h2d = sum(t.numel() * 2 for t in (Q, Kt, V, Wo)) + 4 * (2 * (meta.num_batch + 1) + 3 * R + 6)
    d2h = host_outs[0].numel() * 2
    e2e = {"value": flops_job / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
           "streams": len(lanes), "bytes": "per rank"}
    for w_i, _ in lanes:
        w_i.check_status()
    lanes = lanes[:1]

    # ---- unfused baseline on the same box: attention, cuBLAS GEMM, AllReduce ---------
    unfused = None
    parity = None
    cu_q = torch.tensor(meta.cu_seqlens_q, dtype=torch.int32, device=dev)
    cu_k = torch.tensor(meta.cu_seqlens_k, dtype=torch.int32, device=dev)
    if not args.no_unfused and args.stage == "fused":
        nrep = max(3, K // 2)
        ms_fa_own = timed(ws.launch_fa_only, nrep, 3)
        ws.check_status()
        lib_name, lib_fa = library_attention(dev)
        Qd, Kd, Vd = ws.Q[:wl.tot_q], ws.K[:wl.tot_k], ws.V[:wl.tot_k]
        ms_fa_lib = timed(lambda: lib_fa(Qd, Kd, Vd, cu_q, cu_k, wl.seqlens_q, wl.seqlens_k), nrep, 3)
        A = torch.empty(wl.tot_q, ws.K_local, dtype=torch.bfloat16, device=dev).normal_()
        Wd = Wo.to(dev)
        Y = torch.empty(wl.tot_q, wl.hidden, dtype=torch.bfloat16, device=dev)
        ms_gemm = timed(lambda: torch.matmul(A, Wd, out=Y), nrep, 3)
        ms_ar = ms_ar_nvls = ms_ar_nccl = 0.0
        if world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            Ys = symm_mem.empty(wl.tot_q, wl.hidden, dtype=torch.bfloat16, device=dev)
            symm_mem.rendezvous(Ys, group)
            Ys.zero_()
            ms_ar_nvls = timed(lambda: torch.ops.symm_mem.multimem_all_reduce_(Ys, "sum", group),
                               nrep, 3)
            ms_ar_nccl = timed(lambda: dist.all_reduce(Y), nrep, 3)
            ms_ar = min(ms_ar_nvls, ms_ar_nccl)
        ms_fa = min(ms_fa_own, ms_fa_lib)
        serial = ms_fa + ms_gemm + ms_ar
        unfused = {"fa_ms": ms_fa, "fa_library_ms": ms_fa_lib, "fa_library": lib_name,
                   "fa_own_stage_ms": ms_fa_own, "oproj_cublas_ms": ms_gemm, "allreduce_ms": ms_ar,
                   "allreduce_symm_mem_multimem_ms": ms_ar_nvls, "allreduce_nccl_ms": ms_ar_nccl,
                   "serial_ms": serial, "serial_with_library_fa_ms": ms_fa_lib + ms_gemm + ms_ar,
                   "ideal_ms": max(ms_fa + ms_gemm, ms_ar),
                   "ratio_serial_over_fused": serial / ms_fused,
                   "ratio_serial_library_fa_over_fused": (ms_fa_lib + ms_gemm + ms_ar) / ms_fused,
                   "note": "serial_ms takes the faster attention leg (library kernel or this "
                           "library's attention stage alone) and the faster AllReduce"}

        # ---- parity: the fused output against the unfused chain on the same inputs ----
        # attention from the library kernel (an implementation that shares nothing with the
        # fused kernel), O_proj as an fp32 matmul, AllReduce as an fp32 sum over the ranks;
        # compared over the valid region of every tile.
        ws.launch(); ws.check_status()
        fused = ws.output(meta)
        O_lib = lib_fa(Qd, Kd, Vd, cu_q, cu_k, wl.seqlens_q, wl.seqlens_k)
        ref = O_lib.reshape(wl.tot_q, -1).float() @ Wd.float()
        slack = None
        if world > 1:
            slack = _half_ulp_bf16(ref)
            dist.all_reduce(ref); dist.all_reduce(slack)
        raw, beyond, ref_max = _err_figures(fused, ref, slack)
        parity = {"err_rel_vs_unfused": raw, "err_beyond_bf16_rounding": beyond, "ref_max": ref_max,
                  "tol": 8e-3 if wl.kv_mult > 1 else 2e-3, "unfused_attention": lib_name,
                  "note": "err_rel as in the reference bench (max abs / ref max, both bf16); "
                          "tol applies beyond the half-ulp a bf16 value carries"}
        if world > 1:
            t = torch.tensor([raw, beyond], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            parity["err_rel_vs_unfused"], parity["err_beyond_bf16_rounding"] = (float(x) for x in t)
        parity["ok"] = bool(parity["err_beyond_bf16_rounding"] <= parity["tol"])

    cpu = None
    if rank == 0 and tp == 1 and not args.no_cpu_baseline:
        v, dt, threads, desc, chosen, Yp = cpu_chain_sample(wl, tp, 0, max_seconds_hint=args.cpu_seconds)
        cpu = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc,
               "seconds": dt}
        if parity is not None:
            fused = ws.output(meta)
            cq = [0]
            for a in wl.seqlens_q:
                cq.append(cq[-1] + a)
            rows = torch.cat([fused[cq[i]:cq[i + 1]] for i in chosen])
            raw, beyond, _ = _err_figures(rows, Yp.to(dev))
            parity["err_rel_vs_cpu_oracle"] = raw
            parity["err_beyond_bf16_rounding_vs_cpu_oracle"] = beyond
            parity["cpu_oracle_rows"] = int(rows.shape[0])
            parity["ok"] = bool(parity["ok"] and beyond <= parity["tol"])

    if rank == 0:
        stage_note = {"fused": "", "fa": " (attention stage only)", "ar": " (AllReduce stage only)",
                      "oproj": " (O_proj stage only)", "noar": " (no AllReduce)"}[args.stage]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": tp, "steps": K,
            "warmup": W, "ms_per_step": ms_fused, "higher_is_better": True,
            "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(wl, tp) + stage_note, "seqlens_q": wl.seqlens_q,
                       "kv_mult": wl.kv_mult, "H_local": h, "H_kv": hkv, "hidden": wl.hidden,
                       "role_weights": list(w), "sg": cfg.sg, "launch_flags": flags,
                       "fa_prime_tiles": prime,
                       "l2": "512 MiB buffer written before every timed launch"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": K,
            "clocks": clocks, "unfused": unfused, "parity": parity, "scaling_anchor": anchor,
            "allreduce": {"S_bytes": S, "bus_bytes": bus,
                          "bus_gbs": bus / (ms_fused * 1e-3) / 1e9},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
