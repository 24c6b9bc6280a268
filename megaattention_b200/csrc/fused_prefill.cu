// One persistent kernel: causal varlen GQA FlashAttention -> O_proj GEMM -> AllReduce.
//
// Work identity is a 128-row tile.  A CTA repeatedly asks the in-kernel scheduler for a
// task (protocol of the reference's FusedFaOprojAr kernel,
// src/mega_attention/kernels/sm90/fused_fa_oproj_ar.py:148-398):
//   FA task    (row_tile, q head[s])  : S = Q K^T and O += P V as tcgen05 MMAs with fp32
//                                       accumulators in TMEM, online softmax by one thread
//                                       per row, result to O_scratch (bf16) by TMA store
//   O_proj task (row_tile, n super-group): C[128, <=512] = O_scratch tile @ W_o columns in
//                                       two passes of 256 columns, each into one of two
//                                       ping-pong TMEM accumulators, so a pass's epilogue
//                                       runs under the next pass's MMAs (the A tile
//                                       streams once per pass)
//   AR task    (owned slot)           : multimem.ld_reduce / multimem.st over the NVLS
//                                       multicast view of the symmetric output (or plain
//                                       peer loads / stores with two ranks)
//
// Warp roles (12 warps, 384 threads):
//   warp 0 (lane 0)  TMA producer: Q tiles, the K/V ring, O_proj stages
//   warp 1 (lane 0)  MMA issuer of attention tile 0 and of every O_proj task; warp 1 also
//                    allocates and frees TMEM
//   warp 2 (lane 0)  scheduler: claims tasks, fills one of two descriptor slots, publishes
//                    completions (runs one task ahead of the workers)
//   warp 3 (lane 0)  MMA issuer of attention tile 1
//   warps 4-7, 8-11  two compute warpgroups: online softmax (one thread per row), both
//                    epilogues, AllReduce slots
// An FA task is two q heads of one row tile whenever the rank has two: the two compute
// warpgroups alternate, so the tensor pipe runs one tile's MMAs under the other tile's
// softmax.  With an even number of q heads per kv head the two heads share a kv head and
// every K/V stage of the ring; otherwise (MHA included) each head gets K/V stages of its
// own in the same ring (K of both heads, then V of both heads, per key block), and the
// head an odd count leaves over runs alone.
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
constexpr uint32_t kSmKV = 2 * kTile;      // ring of five K/V tiles
constexpr int kKvSlots = 5;
constexpr uint32_t kSmOpStaging = 4 * (16384 + 32768);   // O_proj output staging, 2 x 16 KB
constexpr uint32_t kOpStage = 16384 + 32768;   // O_proj stage: A 128x64 + W 64x256 (4 stages)
constexpr uint32_t kWPanel = 8192;         // 64 k-rows x 64 n bf16
constexpr uint32_t kTmemS = 0;             // S0 at 0, S1 at 128 (P aliases the first 64 cols)
constexpr uint32_t kTmemO = 256;           // O0 at 256, O1 at 384
constexpr uint32_t kIdescQK = make_idesc_bf16(128, 128, 0, 0);
constexpr uint32_t kIdescPV = make_idesc_bf16(128, 128, 0, 1);
constexpr float kRescaleThreshold = 8.0f;  // in log2 units

struct Bars {
  uint64_t task_full[2];    // scheduler -> roles: descriptor k is valid        (count 1)
  uint64_t task_empty[2];   // roles -> scheduler: task in slot k is finished   (count 11)
  uint64_t loads_done[2];   // producer: every load of the task in slot k is issued (count 1)
  uint64_t q_full[2];       // TMA: Q tile i landed
  uint64_t q_empty[2];      // MMA: last Q K^T of tile i done + epilogue: staging released (count 2)
  uint64_t kv_full[kKvSlots];
  uint64_t kv_empty[kKvSlots];   // shared K/V stages: both MMA issuers release a slot (count 2);
                                 // separate stages: the one issuer that reads it (count 1)
  uint64_t s_full[2];       // MMA: S_i ready
  uint64_t p_full[2];       // softmax warps: P_i written (count 4, one arrival per warp)
  uint64_t o_done[2];       // MMA: last P V of the task for tile i completed
  uint64_t o_free[2];       // epilogue warps: O_i read out (count 4)
  uint64_t op_full[4];
  uint64_t op_empty[4];
  uint64_t acc_full[2];     // MMA: O_proj accumulator half h complete
  uint64_t acc_free[2];     // epilogue warps: half h read out (count 8)
  uint64_t drain[2];        // abort path only: an issuer's outstanding MMAs have retired
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
  if (mbar_try_wait(bar, parity)) return true;
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
  if (p.sep) {
    // two heads per task, the last head of an odd count alone: the counter numbers tasks,
    // (H + 1) / 2 per row tile; arg stays position * H + first head
    const int hp = (p.H + 1) >> 1;
    const int n_tasks = (num_fa / p.H) * hp;
    if (static_cast<int>(ld_relaxed_gpu(p.ctrl + C_FA_COUNTER)) < n_tasks) {
      const int id = static_cast<int>(atom_add_relaxed_gpu(p.ctrl + C_FA_COUNTER, 1u));
      if (id < n_tasks) { *arg = (id / hp) * p.H + 2 * (id % hp); return true; }
    }
    return false;
  }
  const uint32_t step = p.pair ? 2u : 1u;
  if (static_cast<int>(ld_relaxed_gpu(p.ctrl + C_FA_COUNTER)) < num_fa) {
    const uint32_t id = atom_add_relaxed_gpu(p.ctrl + C_FA_COUNTER, step);
    if (static_cast<int>(id) < num_fa) { *arg = static_cast<int>(id); return true; }
  }
  return false;
}

// Pop from the published O_proj ready queue.  The reference pops with a CAS on the consume
// index (fused_fa_oproj_ar.py:168-189); with one CTA per SM all polling, a CAS admits one
// winner per L2 round trip and the queue drains at ~2 tasks/us.  Here a CTA takes a ticket
// with one atomicAdd (every attempt succeeds) after seeing head < tail.  A ticket that lost
// the race to a not-yet-published entry stays pending in this CTA (at most one) and is
// served as soon as the publish index passes it; meanwhile the CTA keeps taking other work.
__device__ __forceinline__ bool try_pop_oproj(const KParams& p, int total_op, int* pending,
                                              int* arg) {
  if (*pending < 0) {
    const uint32_t head = ld_relaxed_gpu(p.ctrl + C_OP_CONSUME);
    const uint32_t tail = ld_acquire_gpu(p.ctrl + C_OP_PUBLISH);
    if (head >= tail) return false;
    const uint32_t t = atom_add_relaxed_gpu(p.ctrl + C_OP_CONSUME, 1u);
    if (static_cast<int>(t) >= total_op) return false;    // past the end: nothing there
    *pending = static_cast<int>(t);
    if (t >= tail && static_cast<uint32_t>(*pending) >= ld_acquire_gpu(p.ctrl + C_OP_PUBLISH))
      return false;
  } else if (static_cast<uint32_t>(*pending) >= ld_acquire_gpu(p.ctrl + C_OP_PUBLISH)) {
    return false;
  }
  *arg = static_cast<int>(ld_relaxed_gpu(p.oproj_queue + *pending));
  *pending = -1;
  return true;
}

// Claim one ready AllReduce slot of this (owner) rank.
//
// The reference has the last of the tp arriving ranks set a bit in the owner's ready
// bitset, found by its atomic add returning tp-1, and owners claim by clearing the lowest
// set bit (fused_fa_oproj_ar.py:192-239, 294-317).  On NVSwitch that costs every O_proj
// task a blocking remote round trip (tens of microseconds once the links carry the
// AllReduce itself) and makes all polling CTAs fight for one bit.  Here arrivals are
// fire-and-forget adds on the owner's ready counts and the owner finds ready slots by
// reading the counts: they are packed as one byte per slot (tp <= 8 arrivals; bit 7 marks
// a slot as claimed), so sixteen slots come with one 16-byte load and a scan of all the
// slots a rank owns is a handful of loads - cheap enough that every CTA looks at every
// slot each time it asks for work, and no ready slot waits to be discovered.  A CTA starts
// its scan at a place of its own so that CTAs polling at the same moment do not all go for
// the same slot; the claim is an atomic OR of the slot's flag, won by whoever sees the
// flag clear in the value that comes back.  The reference's ready bitset has no role here
// (the plan descriptor still has the field so that the workspace keeps the reference's
// buffer list; it may be 0).
__device__ __noinline__ int try_claim_ar(const KParams& p, int local_owned, uint32_t poll_no) {
  if (local_owned <= 0) return -1;
  const uint32_t tp = static_cast<uint32_t>(p.tp);
  const uint32_t n_words = (static_cast<uint32_t>(local_owned) + 3u) >> 2;   // 4 slots per word
  const uint32_t n_vec = (n_words + 3u) >> 2;                                // 16 slots per load
  const uint32_t cap_words = static_cast<uint32_t>(p.max_owner_slots);       // buffer length
  const uint32_t start = (blockIdx.x * 5u + poll_no) % n_vec;
  for (uint32_t v0 = 0; v0 < n_vec; v0 += 8) {
    uint4 w[8];
    uint32_t vi[8];
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {
      uint32_t v = start + v0 + u;
      if (v >= n_vec) v -= n_vec;
      vi[u] = v;
      w[u] = make_uint4(0u, 0u, 0u, 0u);
      if (v0 + u < n_vec) {
        // (gpu-scope loads: a hint only - the atomic below is the synchronising access)
        const uint32_t* src = p.ready_count + v * 4;
        if (v * 4 + 4 <= cap_words) {
          w[u] = ld_relaxed_gpu_b128(src);
        } else {                     // last, partial vector of a short buffer
          if (v * 4 + 0 < cap_words) w[u].x = ld_relaxed_gpu(src + 0);
          if (v * 4 + 1 < cap_words) w[u].y = ld_relaxed_gpu(src + 1);
          if (v * 4 + 2 < cap_words) w[u].z = ld_relaxed_gpu(src + 2);
        }
      }
    }
#pragma unroll
    for (uint32_t u = 0; u < 8; ++u) {
      const uint32_t ws[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
#pragma unroll
      for (uint32_t k = 0; k < 4; ++k) {
        // bytes equal to tp (a claimed slot reads tp | 0x80, an unfinished one < tp)
        const uint32_t x = ws[k] ^ (tp * 0x01010101u);
        uint32_t hit = (x - 0x01010101u) & ~x & 0x80808080u;
        while (hit) {
          const uint32_t b = (__ffs(hit) - 1) >> 3;            // byte number 0..3
          hit &= ~(0xFFu << (b * 8));
          if (((ws[k] >> (b * 8)) & 0xFFu) != tp) continue;      // borrow artefact
          const uint32_t idx = (vi[u] * 4 + k) * 4 + b;
          if (idx >= static_cast<uint32_t>(local_owned)) continue;
          const uint32_t old = atom_or_relaxed_sys(p.ready_count + vi[u] * 4 + k, 0x80u << (b * 8));
          if (((old >> (b * 8)) & 0xFFu) == tp) {
            fence_acq_rel_sys();      // the tp arrivals (release) happen before what follows
            return static_cast<int>(idx * tp + p.rank);
          }
        }
      }
    }
  }
  return -1;
}

__device__ __noinline__ void schedule_pick(const Env& e, int role, int num_fa, int total_op,
                                           int local_owned, uint32_t poll_no, bool busy,
                                           int* pending, int* mode, int* arg) {
  const KParams& p = *e.p;
  *mode = MODE_IDLE;
  *arg = -1;
  if (ld_relaxed_gpu(p.status) != 0u) {       // some CTA (or rank) gave up: leave
    *e.abort_flag = 1;
    *mode = MODE_DONE;
    return;
  }
  if (p.flags & 8u) {
    // AllReduce-only launch: every owned slot is taken as ready (the caller made sure all
    // ranks' partials are in place); slots are handed out by a counter
    if (static_cast<int>(ld_acquire_gpu(p.ctrl + C_AR_DONE)) >= local_owned) { *mode = MODE_DONE; return; }
    if (static_cast<int>(ld_relaxed_gpu(p.ctrl + C_AR_CURSOR)) < local_owned) {
      const int idx = static_cast<int>(atom_add_relaxed_gpu(p.ctrl + C_AR_CURSOR, 1u));
      if (idx < local_owned) { *mode = MODE_AR; *arg = idx * p.tp + p.rank; }
    }
    return;
  }
  if (p.flags & 32u) {
    // O_proj-only launch (single rank): O_scratch is taken as complete, slots are handed
    // out in order by the consume counter
    if (static_cast<int>(ld_acquire_gpu(p.ctrl + C_OP_DONE)) >= total_op) { *mode = MODE_DONE; return; }
    if (static_cast<int>(ld_relaxed_gpu(p.ctrl + C_OP_CONSUME)) < total_op) {
      const int t = static_cast<int>(atom_add_relaxed_gpu(p.ctrl + C_OP_CONSUME, 1u));
      if (t < total_op) { *mode = MODE_OPROJ; *arg = t; }
    }
    return;
  }
  const bool fa_only = (p.flags & 1u) != 0;
  const int fa_d = static_cast<int>(ld_acquire_gpu(p.ctrl + C_FA_DONE));
  bool done = fa_d >= num_fa;
  if (!fa_only) {
    const int op_d = static_cast<int>(ld_acquire_gpu(p.ctrl + C_OP_DONE));
    const int ar_d = static_cast<int>(ld_acquire_gpu(p.ctrl + C_AR_DONE));
    done = done && op_d >= total_op && ((p.flags & 16u) || ar_d >= local_owned);
  }
  if (done) { *mode = MODE_DONE; return; }
  // probe order by role: 0: FA,OPROJ,AR  1: OPROJ,AR,FA  2: AR,FA,OPROJ (the reference's
  // three orders).  With the "drain first" launch flag downstream work goes first so that
  // AllReduce traffic starts early and keeps flowing: roles 0/1 become 3: OPROJ,FA,AR and
  // role 2 becomes 4: AR,OPROJ,FA.
  for (int i = 0; i < 3; ++i) {
    int m;
    if (role == 3) m = (i == 0) ? MODE_OPROJ : (i == 1) ? MODE_FA : MODE_AR;
    else if (role == 4) m = MODE_AR - i;
    else {
      const int src = (role == 0) ? (MODE_FA + i) : (role == 1) ? (MODE_OPROJ + i) : (MODE_AR + i);
      m = (src > MODE_AR) ? src - 3 : src;
    }
    bool ok = false;
    if (m == MODE_FA) ok = try_fa(p, num_fa, arg);
    else if (fa_only) ok = false;
    else if (m == MODE_OPROJ) ok = try_pop_oproj(p, total_op, pending, arg);
    else if (p.tp > 1 && !(p.flags & 16u) &&
             !(busy && static_cast<int>(ld_relaxed_gpu(p.ctrl + C_OP_CONSUME)) >= total_op))
    {
      // (once every O_proj task has been handed out only reductions are left and CTAs go
      // idle: a CTA that still has a task running leaves ready slots to them instead of
      // queueing one behind its own)
      const int q = try_claim_ar(p, local_owned, poll_no);
      if (q >= 0) { *arg = q; ok = true; }
    }
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
  if (p.flags & 16u) {
    // partial sums only (measurement aid): no AllReduce, no cross-rank traffic
  } else if (p.tp == 1) {
    // one rank: the partial is the result; account the (identity) AllReduce right here
    fence_acq_rel_gpu();
    finish_ar_slot(p, slot);
  } else {
    const int owner_rank = slot % p.tp;
    const int owner_idx = slot / p.tp;
    red_add_release_sys(reinterpret_cast<uint32_t*>(p.peer_rc[owner_rank]) + (owner_idx >> 2),
                        1u << ((owner_idx & 3) * 8));      // one byte per slot
  }
  atom_add_release_gpu(p.ctrl + C_OP_DONE, 1u);
}

// ---------------------------------------------------------------- rank barrier
// Cross-rank barrier at kernel exit: two signal slots (phase) counted up to tp and back
// down to 0 (sign), selected by a rank-local counter, so it is reusable without any reset
// (fused_fa_oproj_ar.py:99-143).  Run by one CTA (the last one to finish).
__device__ __noinline__ void rank_barrier(const Env& e) {
  const KParams& p = *e.p;
  __syncthreads();
  if (!*e.abort_flag) {
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
constexpr uint64_t kDescK = smem_desc_template(16, 1024);          // K-major, 128-B swizzle
constexpr uint64_t kDescVmn = smem_desc_template(kPanel, 1024);    // V tile [kv][d], MN-major
constexpr uint64_t kDescWmn = smem_desc_template(kWPanel, 1024);   // W slab [k][n], MN-major

// S = Q K^T over d = 128: 8 k-steps; both tiles are two 64-wide swizzled panels.
__device__ __forceinline__ void issue_qk(uint32_t tmem_s, uint32_t sm_q, uint32_t sm_k) {
  const uint32_t q16 = sm_q >> 4, k16 = sm_k >> 4;
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t off16 = ((kk >> 2) * kPanel + (kk & 3) * 32) >> 4;
    mma_ss(tmem_s, smem_desc_at(kDescK, q16 + off16), smem_desc_at(kDescK, k16 + off16),
           kIdescQK, kk > 0);
  }
}
// O (+)= P V : P is bf16 in TMEM (8 columns per 16 kv), V tile is [kv][d] in two d panels.
__device__ __forceinline__ void issue_pv(uint32_t tmem_o, uint32_t tmem_p, uint32_t sm_v,
                                         bool acc) {
  const uint32_t v16 = sm_v >> 4;
#pragma unroll
  for (int kk = 0; kk < 8; ++kk)
    mma_ts(tmem_o, tmem_p + kk * 8, smem_desc_at(kDescVmn, v16 + kk * 128), kIdescPV,
           (acc || kk > 0) ? 1u : 0u);
}

// Convert 32 fp32 values (columns col0..col0+31 of this thread's row, col0 in {0, 32}) to
// bf16 and put them into a [128 rows][64 columns] staging panel laid out as TMA expects
// for a 128-byte-swizzled box: 16-byte chunk c of row r lives at chunk c ^ (r & 7).
__device__ __forceinline__ void stage_row32(uint32_t panel, int row, int col0,
                                            const uint32_t (&v)[32], float scale) {
  const uint32_t rbase = panel + static_cast<uint32_t>(row) * 128u;
  const uint32_t sw = static_cast<uint32_t>(row & 7);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t c = static_cast<uint32_t>((col0 >> 3) + q);
    st_shared_v4(rbase + ((c ^ sw) << 4),
                 pack_bf16x2(__uint_as_float(v[8 * q + 0]) * scale, __uint_as_float(v[8 * q + 1]) * scale),
                 pack_bf16x2(__uint_as_float(v[8 * q + 2]) * scale, __uint_as_float(v[8 * q + 3]) * scale),
                 pack_bf16x2(__uint_as_float(v[8 * q + 4]) * scale, __uint_as_float(v[8 * q + 5]) * scale),
                 pack_bf16x2(__uint_as_float(v[8 * q + 6]) * scale, __uint_as_float(v[8 * q + 7]) * scale));
  }
}

// ---------------------------------------------------------------- AllReduce of one slot
// One AllReduce slot: 128 rows x (vnt x 128) bf16 columns, reduced in the switch and
// written back to every rank.  `nthr` threads cooperate; each keeps U 16-byte reductions in
// flight before its first store (NVLink round trips are microseconds).
template <int U>
__device__ __forceinline__ void ar_batch(const KParams& p, int ft, int base_out, int c0, int nthr) {
  auto chunk_addr = [&](int c) -> unsigned long long {
    const int o_t = c >> 11, m = (c >> 4) & 127, nc = c & 15;
    const size_t elem =
        ((static_cast<size_t>(ft * 128 + m) * p.num_out + base_out + o_t) * 128) + nc * 8;
    return p.csym_mc + elem * 2;
  };
  uint4 v[U];
#pragma unroll
  for (int u = 0; u < U; ++u) v[u] = multimem_ld_reduce_bf16x8(chunk_addr(c0 + u * nthr));
#pragma unroll
  for (int u = 0; u < U; ++u) multimem_st_b128(chunk_addr(c0 + u * nthr), v[u]);
}

// The same batch with plain peer loads and stores, two ranks only: the owner reads its own
// and the peer's partial, adds in fp32, rounds once and writes both copies.  With two GPUs
// the multicast path is several times slower than the NVLink copy rate; this one is not.
template <int U>
__device__ __forceinline__ void ar_batch_p2p(const KParams& p, int ft, int base_out, int c0, int nthr) {
  auto chunk_off = [&](int c) -> unsigned long long {
    const int o_t = c >> 11, m = (c >> 4) & 127, nc = c & 15;
    const size_t elem =
        ((static_cast<size_t>(ft * 128 + m) * p.num_out + base_out + o_t) * 128) + nc * 8;
    return elem * 2;
  };
  const unsigned long long mine = p.peer_csym[p.rank], peer = p.peer_csym[p.rank ^ 1];
  uint4 a[U], b[U];
#pragma unroll
  for (int u = 0; u < U; ++u) b[u] = ld_relaxed_sys_b128(peer + chunk_off(c0 + u * nthr));
#pragma unroll
  for (int u = 0; u < U; ++u)      // this GPU's own partial: gpu scope is enough
    a[u] = ld_relaxed_gpu_b128(reinterpret_cast<const void*>(mine + chunk_off(c0 + u * nthr)));
#pragma unroll
  for (int u = 0; u < U; ++u) {
    uint4 r;
    r.x = add_bf16x2_via_f32(a[u].x, b[u].x); r.y = add_bf16x2_via_f32(a[u].y, b[u].y);
    r.z = add_bf16x2_via_f32(a[u].z, b[u].z); r.w = add_bf16x2_via_f32(a[u].w, b[u].w);
    const unsigned long long off = chunk_off(c0 + u * nthr);
    st_relaxed_sys_b128(peer + off, r);
    st_relaxed_sys_b128(mine + off, r);
  }
}

// One AllReduce slot: 128 rows x (vnt x 128) bf16 columns, reduced in the switch and
// written back to every rank.  `nthr` (256) threads cooperate; each keeps 16 16-byte
// reductions in flight before its first store (NVLink round trips are microseconds).  A
// slot is vnt x 2048 chunks: whole batches of nthr x 16, then one of nthr x 8 if vnt is odd.
__device__ __forceinline__ void ar_slot(const KParams& p, int ft, int base_out, int vnt, int t,
                                        int nthr) {
  const int total = vnt * 2048;
  int c0 = t;
  if (p.flags & 64u) {      // MA_FLAG_AR_P2P (host side admits it at tp == 2 only)
    for (; c0 + nthr * 7 < total; c0 += nthr * 8) ar_batch_p2p<8>(p, ft, base_out, c0, nthr);
    return;
  }
  for (; c0 + nthr * 15 < total; c0 += nthr * 16) ar_batch<16>(p, ft, base_out, c0, nthr);
  if (c0 + nthr * 7 < total) ar_batch<8>(p, ft, base_out, c0, nthr);
}

}  // namespace

// Task descriptor words written by the scheduler (shared memory, two slots).
enum : int { T_MODE = 0, T_FT = 1,
             TF_HEAD0 = 2, TF_NT = 3, TF_KVH = 4, TF_QROW0 = 5, TF_VALID = 6, TF_KSTART = 7,
             TF_KLEN = 8, TF_OFFSET = 9, TF_NBLK = 10, TF_MB = 11,
             TO_BASE = 2, TO_VNT = 3, TO_VALID = 4, TO_SLOT = 5, T_WORDS = 12 };

__device__ __forceinline__ bool is_tile_mode(int m) { return m == MODE_FA || m == MODE_OPROJ; }

__global__ void __launch_bounds__(kThreads, 1)
fused_prefill_kernel(const __grid_constant__ CUtensorMap tmQ,
                     const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV,
                     const __grid_constant__ CUtensorMap tmO,
                     const __grid_constant__ CUtensorMap tmW,
                     const __grid_constant__ CUtensorMap tmC,
                     const __grid_constant__ KParams p) {
  extern __shared__ uint8_t dyn_smem[];
  // The words that threads spin on (the abort flag is read in every wait loop, the issuers'
  // lock is hammered with atomics) get 128-byte lines of their own, away from the mbarriers:
  // where the compiler put them next to the barrier block by default depended on the
  // block's size, and one such placement cost the attention stage 2.5 % (0.1597 vs 0.1560 ms).
  __shared__ __align__(128) Bars bars;
  __shared__ uint32_t s_tmem;
  __shared__ __align__(128) int s_abort_line[32];
  __shared__ __align__(128) int s_desc[2][T_WORDS];
  __shared__ __align__(128) int s_pipe_line[32];
  int& s_abort = s_abort_line[0];
  int& s_pipe_turn = s_pipe_line[0];   // serialises the two issuers' MMA batches (scheduling only)

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t smem0 = (smem_u32(dyn_smem) + 1023u) & ~1023u;
  Env env{&p, &s_abort};

  if (tid == 0) {
    s_abort = 0;
    s_pipe_turn = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars.task_full[i]), 1);
      mbar_init(smem_u32(&bars.task_empty[i]), 11);
      mbar_init(smem_u32(&bars.loads_done[i]), 1);
      mbar_init(smem_u32(&bars.q_full[i]), 1);
      mbar_init(smem_u32(&bars.q_empty[i]), 2);
      mbar_init(smem_u32(&bars.s_full[i]), 1);
      mbar_init(smem_u32(&bars.p_full[i]), 4);
      mbar_init(smem_u32(&bars.o_done[i]), 1);
      mbar_init(smem_u32(&bars.o_free[i]), 4);
      mbar_init(smem_u32(&bars.acc_full[i]), 1);
      mbar_init(smem_u32(&bars.acc_free[i]), 8);
    }
    for (int i = 0; i < kKvSlots; ++i) {
      mbar_init(smem_u32(&bars.kv_full[i]), 1);
      mbar_init(smem_u32(&bars.kv_empty[i]), p.sep ? 1 : 2);   // issuers that consume a slot
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&bars.op_full[i]), 1);
      mbar_init(smem_u32(&bars.op_empty[i]), 1);
    }
    mbar_init(smem_u32(&bars.drain[0]), 1);
    mbar_init(smem_u32(&bars.drain[1]), 1);
    fence_mbar_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO); tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem;

  // Every role walks the two descriptor slots in turn.  A role arrives on task_empty[k]
  // when its part of the task in slot k is finished; the scheduler publishes the task's
  // completion and refills the slot once all eleven arrivals are in (producer, two MMA
  // issuers, eight compute warps), so the scheduler runs
  // one task ahead of the workers.  Attention tiles and O_proj tiles overlay the same
  // shared memory and TMEM: a role that goes from one kind to the other first waits for
  // the previous task to finish completely (same-kind neighbours overlap freely).
  int slot_k = 0;
  uint32_t tf_par[2] = {0, 0};
  uint32_t n_arrived[2] = {0, 0};
  int prev_mode = MODE_IDLE, prev_k = 0;

#define MA_NEXT_TASK(desc_ptr, mode_var)                                                   \
  if (!wait_bar(env, smem_u32(&bars.task_full[slot_k]), tf_par[slot_k], 0x100 + warp)) break; \
  tf_par[slot_k] ^= 1u;                                                                    \
  const int* desc_ptr = s_desc[slot_k];                                                    \
  const int mode_var = desc_ptr[T_MODE];                                                   \
  if (mode_var == MODE_DONE) break;
#define MA_DRAIN_IF_SWITCH(mode_var)                                                       \
  if (is_tile_mode(mode_var) && is_tile_mode(prev_mode) && mode_var != prev_mode)          \
    wait_bar(env, smem_u32(&bars.task_empty[prev_k]), (n_arrived[prev_k] - 1u) & 1u, 0x110 + warp);
#define MA_TASK_DONE(mode_var)                                                             \
  mbar_arrive(smem_u32(&bars.task_empty[slot_k]));                                         \
  ++n_arrived[slot_k];                                                                     \
  prev_mode = mode_var; prev_k = slot_k; slot_k ^= 1;

  if (warp < 4) {
    reg_dec<80>();
    if (warp == 2 && lane == 0) {
      // ==================================================================== scheduler
      const int num_fa = p.actv[0];
      const int total_op = p.actv[1];
      const int local_owned = p.actv[5];
      int role;
      {
        const int wsum = p.w_fa + p.w_oproj + p.w_ar;
        const int r = static_cast<int>(blockIdx.x) % wsum;
        role = (r < p.w_fa) ? 0 : (r < p.w_fa + p.w_oproj) ? 1 : 2;
        if (p.flags & 2u) role = (role == 2) ? 4 : 3;
      }
      int k = 0;
      bool occupied[2] = {false, false};
      uint32_t te_par[2] = {0, 0}, ld_par[2] = {0, 0};
      bool ld_pending[2] = {false, false}, ld_skip[2] = {false, false};
      int pending_ticket = -1;
      uint32_t poll_no = 0;
      int occ_mode[2] = {0, 0}, occ_a[2] = {0, 0}, occ_b[2] = {0, 0};
#ifdef MA_AUDIT
      int occ_h[2] = {0, 0};
#endif
      auto publish = [&](int kk) {
        if (s_abort) return;
#ifdef MA_AUDIT
        if (p.audit) {      // exactly-once audit (audit build only): one count per finished unit
          if (occ_mode[kk] == MODE_FA) {
            for (int i = 0; i < occ_b[kk]; ++i) atomicAdd(p.audit + occ_a[kk] * p.H + occ_h[kk] + i, 1u);
          } else if (occ_mode[kk] == MODE_OPROJ) {
            atomicAdd(p.audit + p.audit_op_base + occ_a[kk], 1u);
          } else if (occ_mode[kk] == MODE_AR) {
            atomicAdd(p.audit + p.audit_ar_base + occ_a[kk] / p.tp, 1u);
          }
        }
#endif
        if (occ_mode[kk] == MODE_FA) {
          fence_acq_rel_gpu();
          const uint32_t old = atom_add_acqrel_gpu(p.head_ready + occ_a[kk],
                                                   static_cast<uint32_t>(occ_b[kk]));
          if (!(p.flags & 1u) && static_cast<int>(old) + occ_b[kk] == p.H)
            publish_oproj(env, occ_a[kk]);
          atom_add_release_gpu(p.ctrl + C_FA_DONE, static_cast<uint32_t>(occ_b[kk]));
        } else if (occ_mode[kk] == MODE_OPROJ) {
          publish_ar_ready(p, occ_a[kk]);
        } else if (occ_mode[kk] == MODE_AR) {
          fence_acq_rel_sys();
          finish_ar_slot(p, occ_a[kk]);
        }
      };
      while (true) {
        if (occupied[k]) {
          wait_bar(env, smem_u32(&bars.task_empty[k]), te_par[k], 0x120 + k);
          te_par[k] ^= 1u;
          occupied[k] = false;
          publish(k);
        }
        // A long attention task must not sit claimed behind another one: take the next
        // task only once the producer has issued the running task's last load (a few
        // blocks before its end), which keeps the claim order close to greedy.
        if (ld_pending[k ^ 1]) {
          wait_bar(env, smem_u32(&bars.loads_done[k ^ 1]), ld_par[k ^ 1], 0x128 + k);
          ld_par[k ^ 1] ^= 1u;
          ld_pending[k ^ 1] = false;
        } else if (ld_skip[k ^ 1]) {
          ld_par[k ^ 1] ^= 1u;        // that task's loads_done phase is never waited for
          ld_skip[k ^ 1] = false;
        }
        int mode, arg;
        uint64_t idle_t0 = 0;
        while (true) {
          schedule_pick(env, role, num_fa, total_op, local_owned, poll_no++, occupied[k ^ 1],
                        &pending_ticket, &mode, &arg);
          if (mode != MODE_IDLE) break;
          // nothing to do and not finished: bounded like every other wait (a rank that
          // never shows up, or counts that can never be reached, must not hang the GPU)
          if ((poll_no & 15u) == 0) {
            const uint64_t now = globaltimer_ns();
            if (idle_t0 == 0) idle_t0 = now;
            else if (now - idle_t0 > p.wait_limit_ns) {
              report(env, ST_TIMEOUT_IDLE, poll_no, static_cast<uint32_t>(pending_ticket));
              mode = MODE_DONE;
              break;
            }
          }
          const int o = k ^ 1;
          if (occupied[o] && mbar_try_wait(smem_u32(&bars.task_empty[o]), te_par[o])) {
            te_par[o] ^= 1u;
            occupied[o] = false;
            publish(o);
          } else {
            __nanosleep(100);
          }
        }
        int* d = s_desc[k];
        if (mode == MODE_FA) {
          const int pos = arg / p.H, head0 = arg % p.H;
          const int nt = p.pair ? 2 : (p.sep ? min(2, p.H - head0) : 1);
          const int ft = (p.fa_order && !(p.flags & 4u)) ? p.fa_order[pos] : pos;
          const int b = p.fa_b[ft], mb = p.fa_mb[ft];
          const int q0 = p.cu_q[b], q_len = p.cu_q[b + 1] - q0;
          // contiguous KV: rows [k0, k0 + k_len) of K/V; paged KV: k0 is the sequence's row
          // in the page table and the length comes from cache_seqlens
          const int k0 = p.page_table ? b * p.pps : p.cu_k[b];
          const int k_len = p.page_table ? p.cache_seqlens[b] : p.cu_k[b + 1] - k0;
          const int offset = k_len - q_len;
          int nblk = (k_len + 127) >> 7;
          const int nb2 = ((mb + 1) * 128 + offset + 127) >> 7;
          if (nb2 < nblk) nblk = nb2;
          d[T_FT] = ft; d[TF_HEAD0] = head0; d[TF_NT] = nt; d[TF_KVH] = head0 / p.q_per_kv;
          d[TF_QROW0] = q0 + mb * 128; d[TF_VALID] = min(128, q_len - mb * 128);
          d[TF_KSTART] = k0; d[TF_KLEN] = k_len; d[TF_OFFSET] = offset; d[TF_NBLK] = nblk;
          d[TF_MB] = mb;
          occ_a[k] = ft; occ_b[k] = nt;
#ifdef MA_AUDIT
          occ_h[k] = head0;
#endif
        } else if (mode == MODE_OPROJ || mode == MODE_AR) {
          const int ft = arg / p.nsg, g = arg % p.nsg;
          const int base_out = g * p.sg;
          const int b = p.fa_b[ft], mb = p.fa_mb[ft];
          const int q_len = p.cu_q[b + 1] - p.cu_q[b];
          d[T_FT] = ft; d[TO_BASE] = base_out; d[TO_VNT] = min(p.sg, p.num_out - base_out);
          d[TO_VALID] = min(128, q_len - mb * 128); d[TO_SLOT] = arg;
          occ_a[k] = arg;
        }
        d[T_MODE] = mode;
        occ_mode[k] = mode;
        mbar_arrive(smem_u32(&bars.task_full[k]));
        if (mode == MODE_DONE) break;
        occupied[k] = true;
        // claim-ahead is only held back behind long attention tasks; short tasks (O_proj,
        // AllReduce, a few key blocks) want their successor posted before they end
        ld_pending[k] = (mode == MODE_FA && d[TF_NBLK] > 6);
        ld_skip[k] = !ld_pending[k];
        k ^= 1;
      }
    } else if (warp == 0 && lane == 0) {
      // ==================================================================== TMA producer
      uint32_t kv_slot = 0, kv_ph = 0, opc = 0, q_uses[2] = {0, 0};
      while (true) {
        MA_NEXT_TASK(d, mode)
        MA_DRAIN_IF_SWITCH(mode)
        if (mode == MODE_FA) {
          const int nt = d[TF_NT], nblk = d[TF_NBLK];
          // a wait that gave up (abort) ends the task's loads: nothing is written into a
          // buffer that was not waited for
          bool ok = true;
          for (int i = 0; i < nt && ok; ++i) {
            ok = wait_bar(env, smem_u32(&bars.q_empty[i]), (q_uses[i] & 1u) ^ 1u, 0x18 + i);
            if (!ok) break;
            ++q_uses[i];
            const uint32_t bar = smem_u32(&bars.q_full[i]);
            mbar_expect_tx(bar, kTile);
            tma_load_4d(smem0 + kSmQ + i * kTile, &tmQ, bar, 0, d[TF_QROW0], 0, d[TF_HEAD0] + i);
          }
          // shared stages: one K and one V tile per key block; separate stages (p.sep): the
          // K tiles of the task's heads, then their V tiles
          const int nld = p.sep ? nt : 1;
          const int kvh0 = p.sep ? d[TF_HEAD0] / p.q_per_kv : d[TF_KVH];
          const int kvh1 = p.sep ? (d[TF_HEAD0] + 1) / p.q_per_kv : kvh0;
          const int k_base = d[TF_KSTART];
          for (int jj = 0; jj < nblk && ok; ++jj) {
            const int blk = nblk - 1 - jj;
            // key block -> first row of its 128-row tile (paged: one page is one block)
            const int kv_row = p.page_table ? p.page_table[k_base + blk] * 128 : k_base + blk * 128;
            for (int ld = 0; ld < 2 * nld; ++ld) {
              const int which = ld >= nld, i = which ? ld - nld : ld;
              if (!(ok = wait_bar(env, smem_u32(&bars.kv_empty[kv_slot]), kv_ph ^ 1u, 0x10 + kv_slot)))
                break;
              const uint32_t bar = smem_u32(&bars.kv_full[kv_slot]);
              mbar_expect_tx(bar, kTile);
              tma_load_4d(smem0 + kSmKV + kv_slot * kTile, which ? &tmV : &tmK, bar, 0, kv_row, 0,
                          i ? kvh1 : kvh0);
              if (++kv_slot == kKvSlots) { kv_slot = 0; kv_ph ^= 1u; }
            }
          }
        } else if (mode == MODE_OPROJ) {
          const int ft = d[T_FT], base_out = d[TO_BASE], vnt = d[TO_VNT];
          const int nkc = p.K_local >> 6;
          fence_proxy_async_global();   // O_scratch was written by other CTAs' TMA stores
          bool ok = true;
          for (int h = 0; h * 2 < vnt && ok; ++h) {
            for (int kc = 0; kc < nkc; ++kc) {
              const uint32_t st = opc & 3u;
              ok = wait_bar(env, smem_u32(&bars.op_empty[st]), ((opc >> 2) & 1u) ^ 1u, 0x90 + st);
              if (!ok) break;
              const uint32_t bar = smem_u32(&bars.op_full[st]);
              const uint32_t a_dst = smem0 + st * kOpStage;
              // A chunk 128 x 64 and a W slab of 64 k x 256 n (4 panels; panels past the
              // padded width are filled with zeros)
              mbar_expect_tx(bar, kPanel + 4u * kWPanel);
              tma_load_2d(a_dst, &tmO, bar, kc * 64, ft * 128);
              tma_load_3d(a_dst + kPanel, &tmW, bar, 0, kc * 64, (base_out + 2 * h) * 2);
              ++opc;
            }
          }
        }
        mbar_arrive(smem_u32(&bars.loads_done[slot_k]));
        MA_TASK_DONE(mode)
      }
    } else if ((warp == 1 || warp == 3) && lane == 0) {
      // ============================================= MMA issuers: warp 1 -> attention tile 0
      // and every O_proj task, warp 3 -> attention tile 1.  Both follow the K/V ring so a
      // slot is released only when both tiles are done with it.
      const int mi = (warp == 1) ? 0 : 1;
      uint32_t kv_slot = 0, kv_ph = 0, opc = 0;
      uint32_t q_par = 0, p_par = 0, o_uses = 0, acc_uses[2] = {0, 0};
      const uint32_t t_s = tmem + kTmemS + mi * 128, t_o = tmem + kTmemO + mi * 128;
      const uint32_t sm_q = smem0 + kSmQ + mi * kTile;
      // One tile's batch (P V, then the next Q K^T) is issued as a unit: when both tiles
      // become ready together the second waits for the first, which staggers the two
      // softmax warpgroups so that one tile's MMAs run under the other tile's softmax.
      // The lock only shapes the schedule; giving up on it is harmless.
      auto pipe_lock = [&]() {
        for (int it = 0; it < (1 << 16); ++it)
          if (atomicCAS(&s_pipe_turn, 0, 1) == 0) return;
      };
      auto pipe_unlock = [&]() { atomicExch(&s_pipe_turn, 0); };
      while (true) {
        MA_NEXT_TASK(d, mode)
        MA_DRAIN_IF_SWITCH(mode)
        if (mode == MODE_FA) {
          const int nblk = d[TF_NBLK], nt = d[TF_NT];
          const bool act = mi < nt;
          // Shared K/V stages: both issuers follow every slot of the ring.  Separate stages
          // (p.sep): a key block is nt K slots then nt V slots, issuer mi uses the mi-th of
          // each group and leaves the others alone (an idle issuer only keeps count).
          const bool sep = p.sep != 0;
          const bool walk = act || !sep;
          auto my_slot = [&](uint32_t& slot, uint32_t& ph) {
            uint32_t s = kv_slot + (sep ? static_cast<uint32_t>(mi) : 0u), h = kv_ph;
            if (s >= static_cast<uint32_t>(kKvSlots)) { s -= kKvSlots; h ^= 1u; }
            slot = s; ph = h;
            kv_slot += sep ? static_cast<uint32_t>(nt) : 1u;
            if (kv_slot >= static_cast<uint32_t>(kKvSlots)) { kv_slot -= kKvSlots; kv_ph ^= 1u; }
          };
          if (act) {
            wait_bar(env, smem_u32(&bars.q_full[mi]), q_par, 0x20 + mi);
            q_par ^= 1u;
          }
          uint32_t slot_kk, ph_kk;
          my_slot(slot_kk, ph_kk);
          if (walk) wait_bar(env, smem_u32(&bars.kv_full[slot_kk]), ph_kk, 0x30 + slot_kk);
          if (act) {
            tc_fence_after();
            pipe_lock();
            issue_qk(t_s, sm_q, smem0 + kSmKV + slot_kk * kTile);
            tc_commit(smem_u32(&bars.s_full[mi]));
            pipe_unlock();
            if (nblk == 1) tc_commit(smem_u32(&bars.q_empty[mi]));
          }
          if (walk) tc_commit(smem_u32(&bars.kv_empty[slot_kk]));
          for (int jj = 0; jj < nblk; ++jj) {
            uint32_t slot_v, ph_v;
            my_slot(slot_v, ph_v);
            if (walk) wait_bar(env, smem_u32(&bars.kv_full[slot_v]), ph_v, 0x40 + slot_v);
            if (act) {
              if (jj == 0) {   // the previous task's epilogue must have read O out
                wait_bar(env, smem_u32(&bars.o_free[mi]), (o_uses & 1u) ^ 1u, 0x68 + mi);
                ++o_uses;
              }
              wait_bar(env, smem_u32(&bars.p_full[mi]), p_par, 0x60 + mi);
              p_par ^= 1u;
              tc_fence_after();
            }
            const bool has_next = (jj + 1 < nblk);
            if (has_next) {          // K of the next block: prefetched long ago
              my_slot(slot_kk, ph_kk);
              if (walk) wait_bar(env, smem_u32(&bars.kv_full[slot_kk]), ph_kk, 0x50 + slot_kk);
            }
            if (act) {
              pipe_lock();
              issue_pv(t_o, t_s, smem0 + kSmKV + slot_v * kTile, jj > 0);
              tc_commit(smem_u32(&bars.kv_empty[slot_v]));
              if (has_next) {
                issue_qk(t_s, sm_q, smem0 + kSmKV + slot_kk * kTile);
                tc_commit(smem_u32(&bars.s_full[mi]));
                pipe_unlock();
                tc_commit(smem_u32(&bars.kv_empty[slot_kk]));
                if (jj + 2 == nblk) tc_commit(smem_u32(&bars.q_empty[mi]));
              } else {
                tc_commit(smem_u32(&bars.o_done[mi]));
                pipe_unlock();
              }
            } else if (walk) {
              tc_commit(smem_u32(&bars.kv_empty[slot_v]));
              if (has_next) tc_commit(smem_u32(&bars.kv_empty[slot_kk]));
            }
          }
        } else if (mode == MODE_OPROJ && mi == 0) {
          const int vnt = d[TO_VNT];
          const int nkc = p.K_local >> 6;
          for (int h = 0; h * 2 < vnt; ++h) {
            const int ncols = min(2, vnt - 2 * h) * 128;
            const uint32_t idesc = make_idesc_bf16(128, ncols, 0, 1);
            wait_bar(env, smem_u32(&bars.acc_free[h]), (acc_uses[h] & 1u) ^ 1u, 0xA8 + h);
            ++acc_uses[h];
            for (int kc = 0; kc < nkc; ++kc) {
              const uint32_t st = opc & 3u;
              wait_bar(env, smem_u32(&bars.op_full[st]), (opc >> 2) & 1u, 0xA0 + st);
              ++opc;
              tc_fence_after();
              const uint32_t a16 = (smem0 + st * kOpStage) >> 4;
              const uint32_t w16 = a16 + (kPanel >> 4);
#pragma unroll
              for (int kk = 0; kk < 4; ++kk)
                mma_ss(tmem + h * 256, smem_desc_at(kDescK, a16 + kk * 2),
                       smem_desc_at(kDescWmn, w16 + kk * 128), idesc,
                       (kc > 0 || kk > 0) ? 1u : 0u);
              tc_commit(smem_u32(&bars.op_empty[st]));
            }
            tc_commit(smem_u32(&bars.acc_full[h]));
          }
        }
        MA_TASK_DONE(mode)
      }
    }
    __syncwarp();
  } else {
    // ====================================================================== compute warps
    reg_inc<208>();
    const int wg = (warp - 4) >> 2;                            // compute warpgroup 0 / 1
    const int row = (warp & 3) * 32 + lane;                    // TMEM lane == tile row
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint32_t s_par = 0, o_par = 0, acc_par[2] = {0, 0};
    while (true) {
      MA_NEXT_TASK(d, mode)
      if (mode == MODE_FA && wg < d[TF_NT]) {
        // -------------------------------------------- softmax + epilogue of tile `wg`
        const int ft = d[T_FT], head = d[TF_HEAD0] + wg, valid_m = d[TF_VALID];
        const int k_len = d[TF_KLEN], offset = d[TF_OFFSET], nblk = d[TF_NBLK], mb = d[TF_MB];
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
          if (need_mask) {
            const int lim = lim_abs - j * 128;    // columns > lim are masked
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
              for (int kx = 0; kx < 32; ++kx)
                if (c * 32 + kx > lim) s[c][kx] = 0xff800000u;   // -inf
          }
          // Fast path (every block after the first that needs no mask): the exponentials do
          // not wait for this block's row maximum.  They are taken against the reference
          // maximum as it stands while the block maximum is computed alongside; only if
          // some row of the warp turns out to need a new reference (growth beyond 2^8,
          // rare after the first block) the scores are read again from TMEM, where P has
          // not been stored over them yet, and the block goes down the ordinary path.
          // Scale-and-subtract and the row sums work on packed pairs (fma / add on two
          // floats per instruction): the loop is short of issue slots, not of pipes.
          bool done = false;
          if (jj > 0 && !need_mask) {
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * sl2;
            const uint64_t sl2x2 = pack_f32x2(sl2, sl2), negm2 = pack_f32x2(neg_m, neg_m);
            uint64_t sum2[2] = {pack_f32x2(0.f, 0.f), pack_f32x2(0.f, 0.f)};
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pk[16];
#pragma unroll
              for (int kx = 0; kx < 16; ++kx) {
                const float x0 = __uint_as_float(s[c][2 * kx]), x1 = __uint_as_float(s[c][2 * kx + 1]);
                mx[kx & 3] = fmax3(mx[kx & 3], x0, x1);
                const uint64_t a2 = fma_f32x2(pack_f32x2(x0, x1), sl2x2, negm2);
                float a0, a1;
                unpack_f32x2(a2, a0, a1);
                const float e0 = ex2(a0), e1 = ex2(a1);
                sum2[kx & 1] = add_f32x2(sum2[kx & 1], pack_f32x2(e0, e1));
                pk[kx] = pack_bf16x2(e0, e1);
              }
              if ((c & 1) == 0) {
#pragma unroll
                for (int kx = 0; kx < 16; ++kx) s[c][kx] = pk[kx];
              } else {
#pragma unroll
                for (int kx = 0; kx < 16; ++kx) s[c - 1][16 + kx] = pk[kx];
              }
            }
            float s0, s1, s2, s3;
            unpack_f32x2(sum2[0], s0, s1);
            unpack_f32x2(sum2[1], s2, s3);
            const float l_blk = (s0 + s1) + (s2 + s3);
            const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            const bool grow = (m_blk > -INFINITY) &&
                              ((m_ref == -INFINITY) || ((m_blk - m_ref) * sl2 > kRescaleThreshold));
            if (!__any_sync(0xffffffffu, grow)) {
              tmem_st32(t_s, s[0]);
              tmem_st32(t_s + 32, s[2]);
              l_run += l_blk;
              done = true;
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c) tmem_ld32(t_s + c * 32, s[c]);
              tc_wait_ld();
            }
          }
          if (!done) {
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int kx = 0; kx < 32; kx += 2)
#pragma unroll
              for (int c = 0; c < 4; ++c)
                mx[c] = fmax3(mx[c], __uint_as_float(s[c][kx]), __uint_as_float(s[c][kx + 1]));
            const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
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
              // the P V MMA of the previous block completed before this block's S was
              // committed (in-order tensor pipe), so O is quiescent here
#pragma unroll 1
              for (int c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld32(t_o + c * 32, o);
                tc_wait_ld();
#pragma unroll
                for (int kx = 0; kx < 32; ++kx)
                  o[kx] = __float_as_uint(__uint_as_float(o[kx]) * o_scale);
                tmem_st32(t_o + c * 32, o);
              }
            }
            const float neg_m = (m_ref == -INFINITY) ? 0.f : -m_ref * sl2;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t pk[16];
#pragma unroll
              for (int kx = 0; kx < 16; ++kx) {
                const float e0 = ex2(fmaf(__uint_as_float(s[c][2 * kx]), sl2, neg_m));
                const float e1 = ex2(fmaf(__uint_as_float(s[c][2 * kx + 1]), sl2, neg_m));
                sum[(kx & 1) * 2] += e0; sum[(kx & 1) * 2 + 1] += e1;
                pk[kx] = pack_bf16x2(e0, e1);
              }
              // 16 packed columns per 32 scores: two chunks fill one 32-column store
              if ((c & 1) == 0) {
#pragma unroll
                for (int kx = 0; kx < 16; ++kx) s[c][kx] = pk[kx];
              } else {
#pragma unroll
                for (int kx = 0; kx < 16; ++kx) s[c - 1][16 + kx] = pk[kx];
                tmem_st32(t_s + (c >> 1) * 32, s[c - 1]);
              }
            }
            l_run += (sum[0] + sum[1]) + (sum[2] + sum[3]);
          }
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_p);   // 4 arrivals, not 128 serialised ones
        }
        // epilogue: O / l -> bf16 -> O_scratch[ft, row, head, :]; tail rows are zeros
        wait_bar(env, smem_u32(&bars.o_done[wg]), o_par, 0x80 + wg);
        o_par ^= 1u;
        tc_fence_after();
        const float inv = (row < valid_m && l_run > 0.f) ? (1.f / l_run) : 0.f;
        // O / l -> bf16 -> this tile's Q buffer (free: every Q K^T of the task is done),
        // then two TMA stores of 128 rows x 64 columns into O_scratch[ft, :, head, :].
        const uint32_t stg = smem0 + kSmQ + wg * kTile;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t o[2][32];
          tmem_ld32(t_o + hh * 64, o[0]);
          tmem_ld32(t_o + hh * 64 + 32, o[1]);
          tc_wait_ld();
          if (hh == 1) {            // all of O is in registers: the next task may overwrite it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.o_free[wg]));
          }
          stage_row32(stg + hh * kPanel, row, 0, o[0], inv);
          stage_row32(stg + hh * kPanel, row, 32, o[1], inv);
        }
        fence_proxy_async_smem();
        named_bar_sync(1 + wg, 128);
        if ((warp & 3) == 0 && lane == 0) {
          tma_store_2d(&tmO, stg, head * 128, ft * 128);
          tma_store_2d(&tmO, stg + kPanel, head * 128 + 64, ft * 128);
          tma_store_commit();
          tma_store_wait_read();
          mbar_arrive(smem_u32(&bars.q_empty[wg]));     // the producer may refill this Q buffer
          tma_store_wait_all();
          fence_proxy_async_all();     // O_scratch is read back by TMA loads of other CTAs
          __threadfence();
        }
      } else if (mode == MODE_OPROJ) {
        const int ft = d[T_FT], base_out = d[TO_BASE], vnt = d[TO_VNT], valid_m = d[TO_VALID];
        const bool leader = ((warp & 3) == 0 && lane == 0);
        const uint32_t stg = smem0 + kSmOpStaging + wg * kPanel;   // [128 rows][64 cols] bf16
        for (int h = 0; h * 2 < vnt; ++h) {
          wait_bar(env, smem_u32(&bars.acc_full[h]), acc_par[h], 0xB0 + h);
          acc_par[h] ^= 1u;
          tc_fence_after();
          const int o_t = 2 * h + wg;                   // column tile inside the super-group
          if (o_t < vnt) {
            const int out_n = base_out + o_t;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              uint32_t r[2][32];
              tmem_ld32(tmem + lane_base + h * 256 + wg * 128 + hh * 64, r[0]);
              tmem_ld32(tmem + lane_base + h * 256 + wg * 128 + hh * 64 + 32, r[1]);
              tc_wait_ld();
              if (hh == 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars.acc_free[h]));
              }
              if (valid_m == 128) {
                // full row tile: stage 64 columns, one TMA store (clipped at `hidden`)
                if (leader) tma_store_wait_read();
                named_bar_sync(1 + wg, 128);
                stage_row32(stg, row, 0, r[0], 1.f);
                stage_row32(stg, row, 32, r[1], 1.f);
                fence_proxy_async_smem();
                named_bar_sync(1 + wg, 128);
                if (leader) {
                  tma_store_2d(&tmC, stg, out_n * 128 + hh * 64, ft * 128);
                  tma_store_commit();
                }
              } else if (row < valid_m) {
                // last tile of a sequence: rows past valid_m must stay untouched
                uint16_t* dst = p.csym + ((static_cast<size_t>(ft * 128 + row) * p.num_out + out_n) * 128);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                  const int col0 = out_n * 128 + hh * 64 + c * 32;
                  if (col0 + 32 <= p.hidden) {
                    uint4* d4 = reinterpret_cast<uint4*>(dst + hh * 64 + c * 32);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                      uint4 v;
                      v.x = pack_bf16x2(__uint_as_float(r[c][8 * q + 0]), __uint_as_float(r[c][8 * q + 1]));
                      v.y = pack_bf16x2(__uint_as_float(r[c][8 * q + 2]), __uint_as_float(r[c][8 * q + 3]));
                      v.z = pack_bf16x2(__uint_as_float(r[c][8 * q + 4]), __uint_as_float(r[c][8 * q + 5]));
                      v.w = pack_bf16x2(__uint_as_float(r[c][8 * q + 6]), __uint_as_float(r[c][8 * q + 7]));
                      d4[q] = v;
                    }
                  } else {
#pragma unroll
                    for (int kx = 0; kx < 32; ++kx)
                      if (col0 + kx < p.hidden)
                        dst[hh * 64 + c * 32 + kx] = static_cast<uint16_t>(
                            pack_bf16x2(__uint_as_float(r[c][kx]), 0.f) & 0xFFFFu);
                  }
                }
              }
            }
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.acc_free[h]));
          }
        }
        // Ordering towards other CTAs / ranks: the leader waits for its TMA stores, rows
        // written directly get a gpu-scope fence; the one system-scope fence per task is
        // the scheduler's, after it has seen every warp arrive.  (A system fence by each of
        // the 256 threads costs tens of microseconds per task while NVLink is busy.)
        if (leader) {
          tma_store_wait_all();
          fence_proxy_async_all();
        }
        if (valid_m != 128) __threadfence();
      } else if (mode == MODE_AR) {
        ar_slot(p, d[T_FT], d[TO_BASE], d[TO_VNT], tid - 128, 256);
        if (lane == 0) __threadfence_system();   // one per warp; the scheduler fences again
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.task_empty[slot_k]));
      ++n_arrived[slot_k];
      prev_mode = mode; prev_k = slot_k; slot_k ^= 1;
    }
  }
#undef MA_NEXT_TASK
#undef MA_DRAIN_IF_SWITCH
#undef MA_TASK_DONE

  // ------------------------------------------------------------------ exit protocol
  // The reference ends with grid barrier -> every CTA clears the per-launch control state
  // -> grid barrier -> cross-rank barrier (fused_fa_oproj_ar.py:1154-1177).  Here each CTA
  // only counts itself out; the last one to do so (every other CTA has stopped touching
  // the control words by then) clears the state at full capacity, resets the counter and,
  // with tp > 1, runs the cross-rank barrier that also opens the next launch.  No CTA
  // waits for another one.
  __syncthreads();
  if (!s_abort) {
    __shared__ int s_last;
    if (tid == 0) {
      fence_acq_rel_gpu();
      s_last = (atom_add_acqrel_gpu(p.sync_ctrl + S_GS_QUIESCE, 1u) == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
      for (int i = tid; i < p.max_row_tiles; i += kThreads) p.head_ready[i] = 0u;
      for (int i = tid; i < p.max_owner_slots; i += kThreads) p.ready_count[i] = 0u;
      for (int i = tid; i < p.max_owner_words; i += kThreads) p.ar_done_bits[i] = 0ull;
      if (tid < 8) p.ctrl[tid] = 0u;
      if (tid == 8) p.sync_ctrl[S_GS_QUIESCE] = 0u;
      __threadfence_system();
      if (p.tp > 1 && !(p.flags & (1u | 16u))) rank_barrier(env);
    }
  }

  if (s_abort) {
    // A wait ran out (here or in another CTA) and the roles left their loops wherever they
    // were: MMAs, TMA loads and TMA stores of this CTA may still be in flight, and none of
    // them may outlive the CTA's shared memory and TMEM.  Each issuer waits (bounded) for
    // its own MMAs, the store leaders for their bulk stores, and everybody gives loads
    // already issued 100 us to land (nothing issues new ones any more).
    if ((warp == 1 || warp == 3) && lane == 0) {
      const uint32_t bar = smem_u32(&bars.drain[warp == 1 ? 0 : 1]);
      tc_commit(bar);
      for (int it = 0; it < (1 << 20); ++it)
        if (mbar_try_wait(bar, 0)) break;
    }
    if ((warp == 4 || warp == 8) && lane == 0) tma_store_wait_all();
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 100000ull) {}
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
                                                                     maps[3], maps[4], maps[5], kp);
  return cudaGetLastError();
}

cudaError_t fused_prefill_attributes(cudaFuncAttributes* out) {
  return cudaFuncGetAttributes(out, fused_prefill_kernel);
}

}  // namespace ma
