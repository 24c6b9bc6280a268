// One persistent kernel: causal varlen GQA FlashAttention -> O_proj GEMM -> AllReduce.
//
// Work identity is a 128-row tile.  A CTA repeatedly asks the in-kernel scheduler for a
// task (protocol of the reference's FusedFaOprojAr kernel,
// src/mega_attention/kernels/sm90/fused_fa_oproj_ar.py:148-398):
//   FA task    (row_tile, q head[s])  : S = Q K^T and O += P V as tcgen05 MMAs with fp32
//                                       accumulators in TMEM, online softmax by one thread
//                                       per row, result to O_scratch (bf16)
//   O_proj task (row_tile, n super-group): C[128, <=512] = O_scratch tile @ W_o columns,
//                                       one TMEM accumulator of up to 512 columns so the
//                                       A tile streams once per super-group
//   AR task    (owned slot)           : multimem.ld_reduce / multimem.st over the NVLS
//                                       multicast view of the symmetric output
//
// Warp roles (12 warps): warp 0 = scheduler + TMA producer, warp 1 = MMA issuer (and TMEM
// allocator), warps 2-3 = extra AllReduce lanes, warps 4-7 / 8-11 = two compute
// warpgroups (softmax + epilogues).  When q heads come in pairs that share a kv head, an
// FA task is two q heads of one row tile: both tiles use the same K/V stages and the two
// compute warpgroups alternate, so the tensor pipe runs one tile's MMAs under the other
// tile's softmax.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kparams.h"
#include "ptx.cuh"

namespace ma {

namespace {

constexpr uint32_t kTile = 32768;          // 128 x 128 bf16
constexpr uint32_t kPanel = 16384;         // 128 rows x 64 bf16 (one 128-byte-swizzle panel)
constexpr uint32_t kSmQ = 0;               // two Q tiles
constexpr uint32_t kSmKV = 2 * kTile;      // ring of four K/V tiles
constexpr uint32_t kOpStage = 16384 + 65536;   // O_proj stage: A 128x64 + W 64x512
constexpr uint32_t kWPanel = 8192;         // 64 k-rows x 64 n bf16
constexpr uint32_t kTmemS = 0;             // S0 at 0, S1 at 128 (P aliases the first 64 cols)
constexpr uint32_t kTmemO = 256;           // O0 at 256, O1 at 384
constexpr uint32_t kIdescQK = make_idesc_bf16(128, 128, 0, 0);
constexpr uint32_t kIdescPV = make_idesc_bf16(128, 128, 0, 1);
constexpr float kRescaleThreshold = 8.0f;  // in log2 units

struct Bars {
  uint64_t q_full[2];
  uint64_t kv_full[4];
  uint64_t kv_empty[4];
  uint64_t s_full[2];
  uint64_t p_full[2];
  uint64_t o_done[2];
  uint64_t op_full[2];
  uint64_t op_empty[2];
  uint64_t op_done;
};

struct Env {
  const KParams* p;
  volatile int* abort_flag;
};

__device__ __noinline__ void report(const Env& e, uint32_t code, uint32_t site, uint32_t aux) {
  if (atomicCAS(e.p->status, 0u, code) == 0u) {
    e.p->status[1] = site;
    e.p->status[2] = blockIdx.x;
    e.p->status[3] = aux;
  }
  __threadfence();
  *e.abort_flag = 1;
}

// Bounded mbarrier wait.  Returns false once the wait limit passed or the CTA aborted.
__device__ __forceinline__ bool wait_bar(const Env& e, uint32_t bar, uint32_t parity,
                                         uint32_t site) {
  if (*e.abort_flag) return false;
#pragma unroll 1
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 31u) == 0) {
      if (*e.abort_flag) return false;
      if (globaltimer_ns() - t0 > e.p->wait_limit_ns) {
        report(e, ST_TIMEOUT_MBAR, site, parity);
        return false;
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------- scheduler (thread 0)
__device__ __forceinline__ bool try_fa(const KParams& p, int num_fa, int* arg) {
  const uint32_t step = p.pair ? 2u : 1u;
  if (static_cast<int>(ld_relaxed_gpu(p.ctrl + C_FA_COUNTER)) < num_fa) {
    const uint32_t id = atom_add_relaxed_gpu(p.ctrl + C_FA_COUNTER, step);
    if (static_cast<int>(id) < num_fa) { *arg = static_cast<int>(id); return true; }
  }
  return false;
}

__device__ __forceinline__ bool try_pop_oproj(const KParams& p, int* arg) {
  const uint32_t head = ld_relaxed_gpu(p.ctrl + C_OP_CONSUME);
  const uint32_t tail = ld_acquire_gpu(p.ctrl + C_OP_PUBLISH);
  if (head < tail && atom_cas_relaxed_gpu(p.ctrl + C_OP_CONSUME, head, head + 1) == head) {
    *arg = static_cast<int>(ld_relaxed_gpu(p.oproj_queue + head));
    return true;
  }
  return false;
}

__device__ __forceinline__ bool try_claim_ar(const KParams& p, int owner_words, int local_owned,
                                             int* arg) {
  if (owner_words <= 0) return false;
  const uint32_t start = ld_relaxed_gpu(p.ctrl + C_AR_CURSOR);
  for (int i = 0; i < owner_words; ++i) {
    const uint32_t w = (start + i) % static_cast<uint32_t>(owner_words);
    uint64_t* wp = reinterpret_cast<uint64_t*>(p.ready_bits) + w;
    const uint64_t word = ld_acquire_sys_u64(wp);
    if (word == 0) continue;
    const uint64_t lowest = word & (0ull - word);
    const int bit = __ffsll(static_cast<long long>(lowest)) - 1;
    const uint64_t old = atom_and_acqrel_sys_u64(wp, ~lowest);
    if ((old & lowest) == 0) continue;          // another CTA cleared it first
    const int owner_idx = static_cast<int>(w) * 64 + bit;
    if (owner_idx >= local_owned) continue;     // stray tail bit: cleared, not counted
    atom_exch_relaxed_gpu(p.ctrl + C_AR_CURSOR, w);
    *arg = owner_idx * p.tp + p.rank;
    return true;
  }
  return false;
}

__device__ __noinline__ void schedule_pick(const Env& e, int role, int num_fa, int total_op,
                                           int owner_words, int local_owned, int* mode,
                                           int* arg) {
  const KParams& p = *e.p;
  *mode = MODE_IDLE;
  *arg = -1;
  if (ld_relaxed_gpu(p.status) != 0u) {       // some CTA (or rank) gave up: leave
    *e.abort_flag = 1;
    *mode = MODE_DONE;
    return;
  }
  const bool fa_only = (p.flags & 1u) != 0;
  const int fa_d = static_cast<int>(ld_acquire_gpu(p.ctrl + C_FA_DONE));
  bool done = fa_d >= num_fa;
  if (!fa_only) {
    const int op_d = static_cast<int>(ld_acquire_gpu(p.ctrl + C_OP_DONE));
    const int ar_d = static_cast<int>(ld_acquire_gpu(p.ctrl + C_AR_DONE));
    done = done && op_d >= total_op && ar_d >= local_owned;
  }
  if (done) { *mode = MODE_DONE; return; }
  // probe order by role: 0: FA,OPROJ,AR  1: OPROJ,AR,FA  2: AR,FA,OPROJ
  for (int i = 0; i < 3; ++i) {
    const int src = (role == 0) ? (MODE_FA + i) : (role == 1) ? (MODE_OPROJ + i) : (MODE_AR + i);
    const int m = (src > MODE_AR) ? src - 3 : src;
    bool ok = false;
    if (m == MODE_FA) ok = try_fa(p, num_fa, arg);
    else if (fa_only) ok = false;
    else if (m == MODE_OPROJ) ok = try_pop_oproj(p, arg);
    else if (p.tp > 1) ok = try_claim_ar(p, owner_words, local_owned, arg);
    if (ok) { *mode = m; return; }
  }
}

// Reserve, fill and publish (in reservation order) the O_proj slots of one row tile.
__device__ __noinline__ void publish_oproj(const Env& e, int row_tile) {
  const KParams& p = *e.p;
  const uint32_t n = static_cast<uint32_t>(p.nsg);
  const uint32_t start = atom_add_relaxed_gpu(p.ctrl + C_OP_RESERVE, n);
  for (uint32_t i = 0; i < n; ++i) p.oproj_queue[start + i] = row_tile * n + i;
  fence_acq_rel_gpu();
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (ld_acquire_gpu(p.ctrl + C_OP_PUBLISH) != start) {
    if ((++it & 63u) == 0) {
      if (ld_relaxed_gpu(p.status) != 0u) { *e.abort_flag = 1; return; }
      if (globaltimer_ns() - t0 > p.wait_limit_ns) {
        report(e, ST_TIMEOUT_PUBLISH, start, row_tile);
        return;
      }
    }
  }
  atom_add_release_gpu(p.ctrl + C_OP_PUBLISH, n);
}

__device__ __forceinline__ void finish_ar_slot(const KParams& p, int slot) {
  const int owner_idx = slot / p.tp;
  const uint64_t bit = 1ull << (owner_idx & 63);
  const uint64_t old = atom_or_acqrel_gpu_u64(
      reinterpret_cast<uint64_t*>(p.ar_done_bits) + (owner_idx >> 6), bit);
  if ((old & bit) == 0) atom_add_release_gpu(p.ctrl + C_AR_DONE, 1u);
}

// After an O_proj task: tell the slot's owner rank that this rank's partial is in place.
__device__ __noinline__ void publish_ar_ready(const KParams& p, int slot) {
  if (p.tp == 1) {
    // one rank: the partial is the result; account the (identity) AllReduce right here
    fence_acq_rel_gpu();
    finish_ar_slot(p, slot);
  } else {
    fence_acq_rel_sys();
    const int owner_rank = slot % p.tp;
    const int owner_idx = slot / p.tp;
    uint32_t* rc = reinterpret_cast<uint32_t*>(p.peer_rc[owner_rank]) + owner_idx;
    const uint32_t old = atom_add_acqrel_sys(rc, 1u);
    if (old + 1u == static_cast<uint32_t>(p.tp)) {
      uint64_t* rb = reinterpret_cast<uint64_t*>(p.peer_rb[owner_rank]) + (owner_idx >> 6);
      atom_or_release_sys_u64(rb, 1ull << (owner_idx & 63));
    }
  }
  atom_add_release_gpu(p.ctrl + C_OP_DONE, 1u);
}

// ---------------------------------------------------------------- grid / rank barriers
// Grid barrier on one sync word: CTA 0 adds 0x80000000-(G-1), the others add 1, so one
// episode flips only the top bit and the word never needs zeroing
// (fused_fa_oproj_ar.py:74-96).  The spin is bounded.
__device__ __noinline__ void grid_sync(const Env& e, int idx) {
  __syncthreads();
  if (threadIdx.x == 0 && !*e.abort_flag) {
    const KParams& p = *e.p;
    const uint32_t delta = (blockIdx.x == 0) ? (0x80000000u - (gridDim.x - 1)) : 1u;
    const uint32_t old = atom_add_release_gpu(p.sync_ctrl + idx, delta);
    const uint64_t t0 = globaltimer_ns();
    uint32_t it = 0;
    while (((ld_acquire_gpu(p.sync_ctrl + idx) ^ old) & 0x80000000u) == 0) {
      if ((++it & 63u) == 0) {
        if (ld_relaxed_gpu(p.status) != 0u) { *e.abort_flag = 1; break; }
        if (globaltimer_ns() - t0 > p.wait_limit_ns) { report(e, ST_TIMEOUT_GRID, idx, old); break; }
      }
    }
  }
  __syncthreads();
}

// Cross-rank barrier at kernel exit: two signal slots (phase) counted up to tp and back
// down to 0 (sign), selected by a rank-local counter, so it is reusable without any reset
// (fused_fa_oproj_ar.py:99-143).  CTA 0 only.
__device__ __noinline__ void rank_barrier(const Env& e) {
  const KParams& p = *e.p;
  __syncthreads();
  if (blockIdx.x == 0 && !*e.abort_flag) {
    const uint32_t st = ld_relaxed_gpu(p.sync_ctrl + S_NVL_COUNTER);
    const int phase = st & 1u;
    const int down = (st >> 1) & 1u;
    if (static_cast<int>(threadIdx.x) < p.tp) {
      int* peer = reinterpret_cast<int*>(p.peer_nvl[threadIdx.x]) + phase;
      atom_add_release_sys_s32(peer, down ? -1 : 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      atom_add_relaxed_gpu(p.sync_ctrl + S_NVL_COUNTER, 1u);
      const int target = down ? 0 : p.tp;
      const uint64_t t0 = globaltimer_ns();
      uint32_t it = 0;
      while (ld_acquire_sys_s32(p.nvl_signal + phase) != target) {
        if ((++it & 63u) == 0 && globaltimer_ns() - t0 > p.wait_limit_ns) {
          report(e, ST_TIMEOUT_NVL, phase, target);
          break;
        }
      }
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------- FA: MMA helpers
__device__ __forceinline__ void issue_qk(uint32_t tmem_s, uint32_t sm_q, uint32_t sm_k) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t off = (kk >> 2) * kPanel + (kk & 3) * 32;
    mma_ss(tmem_s, make_smem_desc(sm_q + off, 16, 1024), make_smem_desc(sm_k + off, 16, 1024),
           kIdescQK, kk > 0);
  }
}
// O (+)= P V : P is bf16 in TMEM (8 columns per 16 kv), V tile is [kv][d] in two d panels.
__device__ __forceinline__ void issue_pv(uint32_t tmem_o, uint32_t tmem_p, uint32_t sm_v,
                                         bool acc) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    mma_ts(tmem_o, tmem_p + kk * 8, make_smem_desc(sm_v + kk * 2048, kPanel, 1024), kIdescPV,
           (acc || kk > 0) ? 1u : 0u);
  }
}

}  // namespace

struct TaskFA { int ft, head0, nt, kv_head, q_row0, valid_m, k_start, k_len, offset, nblk, mb; };
struct TaskOP { int ft, base_out, vnt, valid_m, slot; };

__global__ void __launch_bounds__(kThreads, 1)
fused_prefill_kernel(const __grid_constant__ CUtensorMap tmQ,
                     const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmO,
                     const __grid_constant__ CUtensorMap tmW,
                     const __grid_constant__ KParams p) {
  extern __shared__ uint8_t dyn_smem[];
  __shared__ __align__(8) Bars bars;
  __shared__ uint32_t s_tmem;
  __shared__ int s_mode, s_abort;
  __shared__ int s_task[12];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t smem0 = (smem_u32(dyn_smem) + 1023u) & ~1023u;
  Env env{&p, &s_abort};

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.q_full[i]), 1);
      mbar_init(smem_u32(&bars.s_full[i]), 1);
      mbar_init(smem_u32(&bars.p_full[i]), 128);
      mbar_init(smem_u32(&bars.o_done[i]), 1);
      mbar_init(smem_u32(&bars.op_full[i]), 1);
      mbar_init(smem_u32(&bars.op_empty[i]), 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&bars.kv_full[i]), 1);
      mbar_init(smem_u32(&bars.kv_empty[i]), 1);
    }
    mbar_init(smem_u32(&bars.op_done), 1);
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO); tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  const int num_fa = p.actv[0];
  const int total_op = p.actv[1];
  const int owner_words = p.actv[4];
  const int local_owned = p.actv[5];
  int role = 0;
  {
    const int wsum = p.w_fa + p.w_oproj + p.w_ar;
    const int r = static_cast<int>(blockIdx.x) % wsum;
    role = (r < p.w_fa) ? 0 : (r < p.w_fa + p.w_oproj) ? 1 : 2;
  }

  // mbarrier phase bookkeeping; every role advances its own copies in lockstep
  uint32_t kvc = 0;                 // K/V ring uses (producer and MMA issuer)
  uint32_t opc = 0;                 // O_proj stage uses (producer and MMA issuer)
  uint32_t q_par[2] = {0, 0};       // MMA issuer
  uint32_t p_par[2] = {0, 0};       // MMA issuer
  uint32_t s_par = 0, o_par = 0;    // compute warpgroup (its own tile)
  uint32_t d_par = 0;               // compute warpgroups: op_done

  const int wg = (warp >= 4) ? ((warp - 4) >> 2) : -1;       // compute warpgroup 0 / 1
  const int row = (warp & 3) * 32 + lane;                    // TMEM lane == tile row
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;

  while (true) {
    if (tid == 0) {
      int mode, arg;
      schedule_pick(env, role, num_fa, total_op, owner_words, local_owned, &mode, &arg);
      if (mode == MODE_FA) {
        const int nt = p.pair ? 2 : 1;
        const int ft = arg / p.H, head0 = arg % p.H;
        const int b = p.fa_b[ft], mb = p.fa_mb[ft];
        const int q0 = p.cu_q[b], q_len = p.cu_q[b + 1] - q0;
        const int k0 = p.cu_k[b], k_len = p.cu_k[b + 1] - k0;
        const int offset = k_len - q_len;
        int nblk = (k_len + 127) >> 7;
        const int nb2 = ((mb + 1) * 128 + offset + 127) >> 7;
        if (nb2 < nblk) nblk = nb2;
        s_task[0] = ft; s_task[1] = head0; s_task[2] = nt; s_task[3] = head0 / p.q_per_kv;
        s_task[4] = q0 + mb * 128;
        s_task[5] = min(128, q_len - mb * 128);
        s_task[6] = k0; s_task[7] = k_len; s_task[8] = offset; s_task[9] = nblk; s_task[10] = mb;
      } else if (mode == MODE_OPROJ || mode == MODE_AR) {
        const int ft = arg / p.nsg, g = arg % p.nsg;
        const int base_out = g * p.sg;
        const int b = p.fa_b[ft], mb = p.fa_mb[ft];
        const int q_len = p.cu_q[b + 1] - p.cu_q[b];
        s_task[0] = ft; s_task[1] = base_out; s_task[2] = min(p.sg, p.num_out - base_out);
        s_task[3] = min(128, q_len - mb * 128); s_task[4] = arg;
      } else if (mode == MODE_IDLE) {
        __nanosleep(200);
      }
      s_mode = mode;
    }
    __syncthreads();
    const int mode = s_mode;
    if (mode == MODE_DONE) break;

    if (mode == MODE_FA) {
      // ====================================================================== FA
      const int ft = s_task[0], head0 = s_task[1], nt = s_task[2], kv_head = s_task[3];
      const int q_row0 = s_task[4], valid_m = s_task[5], k_start = s_task[6];
      const int k_len = s_task[7], offset = s_task[8], nblk = s_task[9], mb = s_task[10];

      if (warp == 0) {
        if (lane == 0) {
          for (int i = 0; i < nt; ++i) {
            const uint32_t bar = smem_u32(&bars.q_full[i]);
            const uint32_t dst = smem0 + kSmQ + i * kTile;
            mbar_expect_tx(bar, kTile);
            tma_load_3d(dst, &tmQ, bar, 0, head0 + i, q_row0);
            tma_load_3d(dst + kPanel, &tmQ, bar, 64, head0 + i, q_row0);
          }
          for (int jj = 0; jj < nblk; ++jj) {
            const int kv_row = k_start + (nblk - 1 - jj) * 128;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
              const uint32_t slot = kvc & 3u;
              wait_bar(env, smem_u32(&bars.kv_empty[slot]), ((kvc >> 2) & 1u) ^ 1u, 0x10 + slot);
              const uint32_t bar = smem_u32(&bars.kv_full[slot]);
              const uint32_t dst = smem0 + kSmKV + slot * kTile;
              const CUtensorMap* tm = which ? &tmV : &tmK;
              mbar_expect_tx(bar, kTile);
              tma_load_3d(dst, tm, bar, 0, kv_head, kv_row);
              tma_load_3d(dst + kPanel, tm, bar, 64, kv_head, kv_row);
              ++kvc;
            }
          }
        }
        __syncwarp();
      } else if (warp == 1) {
        if (lane == 0) {
          for (int i = 0; i < nt; ++i) {
            wait_bar(env, smem_u32(&bars.q_full[i]), q_par[i], 0x20 + i);
            q_par[i] ^= 1u;
          }
          uint32_t slot_k = kvc & 3u;
          wait_bar(env, smem_u32(&bars.kv_full[slot_k]), (kvc >> 2) & 1u, 0x30 + slot_k);
          ++kvc;
          tc_fence_after();
          for (int i = 0; i < nt; ++i) {
            issue_qk(tmem + kTmemS + i * 128, smem0 + kSmQ + i * kTile,
                     smem0 + kSmKV + slot_k * kTile);
            tc_commit(smem_u32(&bars.s_full[i]));
          }
          tc_commit(smem_u32(&bars.kv_empty[slot_k]));
          for (int jj = 0; jj < nblk; ++jj) {
            const uint32_t slot_v = kvc & 3u;
            wait_bar(env, smem_u32(&bars.kv_full[slot_v]), (kvc >> 2) & 1u, 0x40 + slot_v);
            ++kvc;
            const bool has_next = (jj + 1 < nblk);
            if (has_next) {
              slot_k = kvc & 3u;
              wait_bar(env, smem_u32(&bars.kv_full[slot_k]), (kvc >> 2) & 1u, 0x50 + slot_k);
              ++kvc;
            }
            for (int i = 0; i < nt; ++i) {
              wait_bar(env, smem_u32(&bars.p_full[i]), p_par[i], 0x60 + i);
              p_par[i] ^= 1u;
              tc_fence_after();
              issue_pv(tmem + kTmemO + i * 128, tmem + kTmemS + i * 128,
                       smem0 + kSmKV + slot_v * kTile, jj > 0);
              if (!has_next) {
                tc_commit(smem_u32(&bars.o_done[i]));
              } else {
                issue_qk(tmem + kTmemS + i * 128, smem0 + kSmQ + i * kTile,
                         smem0 + kSmKV + slot_k * kTile);
                tc_commit(smem_u32(&bars.s_full[i]));
              }
            }
            tc_commit(smem_u32(&bars.kv_empty[slot_v]));
            if (has_next) tc_commit(smem_u32(&bars.kv_empty[slot_k]));
          }
        }
        __syncwarp();
      } else if (wg >= 0 && wg < nt) {
        // ------------------------------------------------ softmax + epilogue of tile `wg`
        const uint32_t t_s = tmem + kTmemS + wg * 128 + lane_base;
        const uint32_t t_o = tmem + kTmemO + wg * 128 + lane_base;
        const uint32_t bar_s = smem_u32(&bars.s_full[wg]);
        const uint32_t bar_p = smem_u32(&bars.p_full[wg]);
        const float sl2 = p.scale_log2;
        // last kv position this row may see (bottom-right causal, clipped to k_len)
        const int lim_abs = min(mb * 128 + row + offset, k_len - 1);
        float m_ref = -INFINITY;      // max the exponent is taken against (raw score units)
        float l_run = 0.f;            // running row sum of exp2
        for (int jj = 0; jj < nblk; ++jj) {
          const int j = nblk - 1 - jj;
          wait_bar(env, bar_s, s_par, 0x70 + wg);
          s_par ^= 1u;
          tc_fence_after();
          uint32_t s[4][32];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, s[c]);
          tc_wait_ld();
          const bool need_mask = ((j + 1) * 128 - 1 > mb * 128 + offset) || ((j + 1) * 128 > k_len);
          float m_blk = -INFINITY;
          if (need_mask) {
            const int lim = lim_abs - j * 128;    // columns > lim are masked
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int k = 0; k < 32; ++k) {
                float v = __uint_as_float(s[c][k]);
                v = (c * 32 + k <= lim) ? v : -INFINITY;
                s[c][k] = __float_as_uint(v);
                m_blk = fmaxf(m_blk, v);
              }
          } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int k = 0; k < 32; ++k) m_blk = fmaxf(m_blk, __uint_as_float(s[c][k]));
          }
          // lazy rescale: move the reference max only when it would grow by > 2^8
          const bool grow = (m_blk > -INFINITY) &&
                            ((m_ref == -INFINITY) || ((m_blk - m_ref) * sl2 > kRescaleThreshold));
          float o_scale = 1.f;
          if (grow) {
            o_scale = (m_ref == -INFINITY) ? 0.f : ex2((m_ref - m_blk) * sl2);
            m_ref = m_blk;
            l_run *= o_scale;
          }
          if (jj > 0 && __any_sync(0xffffffffu, grow)) {
            // the PV MMA of the previous block completed before this block's S was
            // committed (in-order tensor pipe), so O is quiescent here
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(t_o + c * 32, o);
              tc_wait_ld();
#pragma unroll
              for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * o_scale);
              tmem_st32(t_o + c * 32, o);
            }
          }
          const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * sl2;
          float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const float e0 = ex2(fmaf(__uint_as_float(s[c][2 * k]), sl2, neg_m));
              const float e1 = ex2(fmaf(__uint_as_float(s[c][2 * k + 1]), sl2, neg_m));
              sum0 += e0; sum1 += e1;
              pk[k] = pack_bf16x2(e0, e1);
            }
            // 16 packed columns per 32 scores; reuse the 32-wide store as two halves
            if ((c & 1) == 0) {
#pragma unroll
              for (int k = 0; k < 16; ++k) s[c][k] = pk[k];
            } else {
#pragma unroll
              for (int k = 0; k < 16; ++k) s[c - 1][16 + k] = pk[k];
            }
          }
          l_run += sum0 + sum1;
          tmem_st32(t_s, s[0]);
          tmem_st32(t_s + 32, s[2]);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar_p);
        }
        // epilogue: O / l -> bf16 -> O_scratch[ft, row, head, :]; tail rows are zeros
        wait_bar(env, smem_u32(&bars.o_done[wg]), o_par, 0x80 + wg);
        o_par ^= 1u;
        tc_fence_after();
        const float inv = (row < valid_m && l_run > 0.f) ? (1.f / l_run) : 0.f;
        uint16_t* dst = p.o_scratch +
            (static_cast<size_t>(ft * 128 + row) * p.H + (head0 + wg)) * 128;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(t_o + c * 32, o);
          tc_wait_ld();
          uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[8 * q + 0]) * inv, __uint_as_float(o[8 * q + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv);
            d4[q] = v;
          }
        }
        tc_fence_before();
        __threadfence();
        fence_proxy_async_global();   // O_scratch is read back by TMA (async proxy)
      }
      __syncthreads();
      if (tid == 0 && !s_abort) {
        fence_acq_rel_gpu();
        const uint32_t old = atom_add_acqrel_gpu(p.head_ready + ft, static_cast<uint32_t>(nt));
        if (!(p.flags & 1u) && static_cast<int>(old) + nt == p.H) publish_oproj(env, ft);
        atom_add_release_gpu(p.ctrl + C_FA_DONE, static_cast<uint32_t>(nt));
      }
    } else if (mode == MODE_OPROJ) {
      // ====================================================================== O_proj
      const int ft = s_task[0], base_out = s_task[1], vnt = s_task[2], valid_m = s_task[3];
      const int slot = s_task[4];
      const int nkc = p.K_local >> 6;
      if (warp == 0) {
        if (lane == 0) {
          fence_proxy_async_global();
          for (int kc = 0; kc < nkc; ++kc) {
            const uint32_t st = opc & 1u;
            wait_bar(env, smem_u32(&bars.op_empty[st]), ((opc >> 1) & 1u) ^ 1u, 0x90 + st);
            const uint32_t bar = smem_u32(&bars.op_full[st]);
            const uint32_t a_dst = smem0 + st * kOpStage;
            mbar_expect_tx(bar, kPanel + static_cast<uint32_t>(vnt) * 2u * kWPanel);
            tma_load_2d(a_dst, &tmO, bar, kc * 64, ft * 128);
            for (int pn = 0; pn < vnt * 2; ++pn)
              tma_load_2d(a_dst + kPanel + pn * kWPanel, &tmW, bar, base_out * 128 + pn * 64,
                          kc * 64);
            ++opc;
          }
        }
        __syncwarp();
      } else if (warp == 1) {
        if (lane == 0) {
          for (int kc = 0; kc < nkc; ++kc) {
            const uint32_t st = opc & 1u;
            wait_bar(env, smem_u32(&bars.op_full[st]), (opc >> 1) & 1u, 0xA0 + st);
            ++opc;
            tc_fence_after();
            const uint32_t a_sm = smem0 + st * kOpStage;
            const uint32_t w_sm = a_sm + kPanel;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t adesc = make_smem_desc(a_sm + kk * 32, 16, 1024);
              for (int ng = 0; ng * 2 < vnt; ++ng) {
                const int ncols = min(256, vnt * 128 - ng * 256);
                const uint64_t bdesc =
                    make_smem_desc(w_sm + ng * 4 * kWPanel + kk * 2048, kWPanel, 1024);
                mma_ss(tmem + ng * 256, adesc, bdesc, make_idesc_bf16(128, ncols, 0, 1),
                       (kc > 0 || kk > 0) ? 1u : 0u);
              }
            }
            tc_commit(smem_u32(&bars.op_empty[st]));
          }
          tc_commit(smem_u32(&bars.op_done));
        }
        __syncwarp();
      } else if (wg >= 0) {
        wait_bar(env, smem_u32(&bars.op_done), d_par, 0xB0);
        d_par ^= 1u;
        tc_fence_after();
        for (int oo = 0; oo < 2; ++oo) {
          const int o_t = wg * 2 + oo;                  // column tile inside the super-group
          if (o_t >= vnt) break;
          const int out_n = base_out + o_t;
          uint16_t* dst = p.csym +
              ((static_cast<size_t>(ft * 128 + row) * p.num_out + out_n) * 128);
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_base + o_t * 128 + c * 32, r);
            tc_wait_ld();
            const int col0 = out_n * 128 + c * 32;
            if (row < valid_m) {
              if (col0 + 32 <= p.hidden) {
                uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 v;
                  v.x = pack_bf16x2(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
                  v.y = pack_bf16x2(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                  v.z = pack_bf16x2(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
                  v.w = pack_bf16x2(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                  d4[q] = v;
                }
              } else {
#pragma unroll
                for (int k = 0; k < 32; ++k)
                  if (col0 + k < p.hidden)
                    dst[c * 32 + k] =
                        static_cast<uint16_t>(pack_bf16x2(__uint_as_float(r[k]), 0.f) & 0xFFFFu);
              }
            }
          }
        }
        tc_fence_before();
        if (p.tp > 1) __threadfence_system(); else __threadfence();
      }
      __syncthreads();
      if (tid == 0 && !s_abort) publish_ar_ready(p, slot);
    } else if (mode == MODE_AR) {
      // ====================================================================== AllReduce
      const int ft = s_task[0], base_out = s_task[1], vnt = s_task[2], slot = s_task[4];
      const int total = vnt * 2048;                    // 16-byte chunks in the slot
      for (int c0 = tid; c0 < total; c0 += kThreads * 4) {
        uint4 v[4];
        unsigned long long a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * kThreads;
          const int o_t = c >> 11, m = (c >> 4) & 127, nc = c & 15;
          const size_t elem =
              ((static_cast<size_t>(ft * 128 + m) * p.num_out + base_out + o_t) * 128) + nc * 8;
          a[u] = p.csym_mc + elem * 2;
          if (c < total) v[u] = multimem_ld_reduce_bf16x8(a[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c0 + u * kThreads < total) multimem_st_b128(a[u], v[u]);
      }
      __threadfence_system();
      __syncthreads();
      if (tid == 0) finish_ar_slot(p, slot);
    } else {
      __syncthreads();
    }
  }

  // ------------------------------------------------------------------ exit protocol
  // quiesce -> every CTA clears the per-launch control state at full capacity -> all
  // cleared -> (tp > 1) one cross-rank barrier, which also opens the next launch
  if (!s_abort) {
    grid_sync(env, S_GS_QUIESCE);
    if (!s_abort) {
      const int stride = gridDim.x * kThreads;
      const int g0 = blockIdx.x * kThreads + tid;
      for (int i = g0; i < p.max_row_tiles; i += stride) p.head_ready[i] = 0u;
      for (int i = g0; i < p.max_owner_slots; i += stride) p.ready_count[i] = 0u;
      for (int i = g0; i < p.max_owner_words; i += stride) { p.ready_bits[i] = 0ull; p.ar_done_bits[i] = 0ull; }
      if (blockIdx.x == 0 && tid < 8) p.ctrl[tid] = 0u;
      __threadfence();
      grid_sync(env, S_GS_CLEANDONE);
      if (p.tp > 1 && !(p.flags & 1u)) rank_barrier(env);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------- host launcher
cudaError_t launch_fused_prefill(const CUtensorMap* maps, const KParams& kp, int num_ctas,
                                 cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    err = cudaFuncSetAttribute(fused_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSmemDynamic);
    if (err != cudaSuccess) return err;
    attr_set[dev] = true;
  }
  fused_prefill_kernel<<<num_ctas, kThreads, kSmemDynamic, stream>>>(maps[0], maps[1], maps[2],
                                                                     maps[3], maps[4], kp);
  return cudaGetLastError();
}

cudaError_t fused_prefill_attributes(cudaFuncAttributes* out) {
  return cudaFuncGetAttributes(out, fused_prefill_kernel);
}

}  // namespace ma
