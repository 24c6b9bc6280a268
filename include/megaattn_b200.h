/*
 * C ABI of the B200 (sm_100a) fused prefill path:
 *   causal varlen GQA FlashAttention -> row-parallel O_proj GEMM -> tensor-parallel
 *   AllReduce, one persistent kernel, one 128-row tile as the unit of work.
 *
 * The reference project exposes this path only as Python objects; each entry point
 * below names the reference interface it stands in for (path:line inside the reference
 * tree).  Plain pointers and sizes only: device addresses travel as uint64_t, the
 * stream as an opaque pointer (a cudaStream_t).  Every function returns 0 on success or
 * a negative ma_error code; nothing throws and nothing exits the process.
 *
 * The library never allocates or frees the caller's buffers.  A plan borrows every
 * device pointer it is given; they must stay valid until ma_plan_destroy.
 */
#ifndef MEGAATTN_B200_H_
#define MEGAATTN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MA_MAX_TP 8
#define MA_NUM_CTRL 8     /* src/mega_attention/kernels/sm90/fused_fa_oproj_ar.py:47-55 */
#define MA_NUM_SYNC 3     /* fused_fa_oproj_ar.py:64-67 */
#define MA_NUM_ACTV 6     /* src/mega_attention/metadata/row_desc.py:156-174 */
#define MA_NUM_STATUS 8   /* device status block (no reference counterpart) */

typedef enum ma_error {
  MA_OK = 0,
  MA_ERR_INVALID = -1,        /* bad argument / unsupported shape                      */
  MA_ERR_CUDA = -2,           /* a CUDA runtime or driver call failed                  */
  MA_ERR_NOT_SM100 = -3,      /* device is not compute capability 10.x                 */
  MA_ERR_DEVICE_TIMEOUT = -4, /* a bounded device-side wait gave up (see ma_status)    */
  MA_ERR_CAPACITY = -5        /* request exceeds a stated maximum                      */
} ma_error;

/* ma_launch_args.flags */
#define MA_FLAG_FA_ONLY 1u    /* run the attention stage only (fills O_scratch)         */
#define MA_FLAG_DRAIN_FIRST 2u /* downstream work first: attention- and O_proj-role CTAs probe
                                  O_proj, attention, AllReduce; AllReduce-role CTAs probe
                                  AllReduce, O_proj, attention (no reference counterpart; for
                                  NVLink-bound launches, so that AllReduce traffic starts early) */
#define MA_FLAG_AR_ONLY 8u    /* AllReduce stage only: every owned slot of C_sym is reduced;
                                 all ranks' partials must already be in place             */
#define MA_FLAG_NO_AR 16u     /* stop after O_proj: C_sym holds this rank's partial (measurement aid) */
#define MA_FLAG_OPROJ_ONLY 32u /* O_proj stage only (single rank): O_scratch must be complete */
#define MA_FLAG_AR_P2P 64u     /* tp_size == 2 only: the slot owner reduces with plain peer loads and
                                  stores through peer_csym instead of multimem (with two GPUs the
                                  multicast path runs far below the NVLink copy rate).  Same sum:
                                  fp32, rounded once.  No reference counterpart. */
#define MA_FLAG_TILE_ORDER 4u /* claim attention tasks in row-tile order, ignoring fa_order */
/* ma_launch refuses (MA_ERR_INVALID): more than one of FA_ONLY / AR_ONLY / NO_AR / OPROJ_ONLY;
 * AR_ONLY on one rank or without a multicast address; OPROJ_ONLY with tp_size > 1; AR_P2P unless
 * tp_size == 2 with both peer_csym set; unknown bits. */

typedef struct ma_devinfo {
  int32_t cc_major, cc_minor, num_sms, max_smem_optin;
  int32_t kernel_threads, kernel_smem_bytes, kernel_regs, max_ctas; /* of the fused kernel */
} ma_devinfo;

/*
 * Everything FusedFaOprojArWorkspace.create() + compile() fix for the lifetime of a
 * workspace (src/mega_attention/runtime/workspace.py:46-150, :174-194).  Buffer shapes
 * and dtypes are the reference's (workspace.py:116-139):
 *   Q [max_tot_q, H_local, D] bf16      K, V [max_tot_k, H_kv, D] bf16
 *   W_o [K_local, hidden_pad] bf16 (columns >= hidden zero)
 *   o_scratch [max_row_tiles, 128, H_local, D] bf16
 *   csym [max_row_tiles, 128, num_out, 128] bf16 (symmetric across ranks when tp > 1)
 *   ctrl u32[8]  sync_ctrl u32[3]  actv i32[6]  head_ready u32[max_row_tiles]
 *   oproj_queue u32[max_total_oproj]  ready_count u32[max_owner_slots] (symmetric)
 *   ready_bits u64[max_owner_words] (symmetric; the reference's ready bitset, kept in the
 *   descriptor for its buffer list but not read by this kernel: may be 0)
 *   ar_done_bits u64[max_owner_words]
 *   nvl_signal i32[2] (symmetric)  cu_q, cu_k i32[max_batch+1]  fa_b, fa_mb, fa_order i32[max_row_tiles]
 *   status u32[8]
 * All control buffers must be zero when the plan is first launched.
 */
typedef struct ma_plan_desc {
  int32_t device;
  int32_t tp_size, rank;
  int32_t H_local, H_kv, D, hidden;   /* H_local % H_kv == 0; any group size H_local / H_kv:
                                         an attention task takes two q heads of a row tile,
                                         sharing the K/V stages when the group size is even,
                                         with stages of their own otherwise (MHA included) */
  int32_t super_group_n_tiles;
  int32_t max_row_tiles, max_batch, max_tot_q, max_tot_k;
  float softmax_scale;            /* <= 0: D^-0.5                                       */
  uint32_t wait_limit_ms;         /* bound of every device-side wait; 0: default 2000   */
  uint64_t Q, K, V, W_o, o_scratch, csym;
  uint64_t ctrl, sync_ctrl, actv, head_ready, oproj_queue;
  uint64_t ready_count, ready_bits, ar_done_bits, nvl_signal;
  uint64_t cu_q, cu_k, fa_b, fa_mb, status;
  uint64_t csym_multicast;                      /* NVLS multicast address of csym; 0 if tp==1 */
  uint64_t peer_ready_count[MA_MAX_TP];         /* per-rank addresses of the symmetric buffers */
  uint64_t peer_ready_bits[MA_MAX_TP];
  uint64_t peer_nvl_signal[MA_MAX_TP];
  /* Paged KV (src/mega_attention/runtime/workspace.py:67-74, 130-137, 213-222 of the
   * reference; page size 128 = one key block): when page_table is non-zero, K and V are
   * caches [max_pages, 128, H_kv, D], key block j of sequence b lives in page
   * page_table[b * max_pages_per_seq + j], and the KV length of sequence b is
   * cache_seqlens[b] (cu_k is ignored).  max_tot_k must be max_pages * 128. */
  uint64_t page_table;      /* i32[max_batch, max_pages_per_seq], or 0: contiguous KV   */
  uint64_t cache_seqlens;   /* i32[max_batch]                                            */
  int32_t max_pages_per_seq;
  int32_t reserved0;
  uint64_t fa_order;   /* i32[max_row_tiles]: row tiles in the order attention tasks are
                          claimed; 0 = natural order.  Any permutation of the active row
                          tiles is valid: the order only shapes the schedule.  The Python
                          workspace writes longest-first (one GPU, small AllReduce share),
                          or long and short tiles alternating so that row tiles complete,
                          and their AllReduce slots become ready, from the start of the
                          launch (runtime/workspace.py, claim_order).
                          No reference counterpart: the reference claims in tile order. */
  uint64_t peer_csym[MA_MAX_TP];   /* per-rank addresses of C_sym (symmetric); needed for
                                      MA_FLAG_AR_P2P, may be 0 otherwise.  No reference
                                      counterpart: the reference reduces through multimem only. */
  uint64_t audit;   /* optional (0 = off; read by the audit build of the library only, see
                       megaattention_b200/build.py): u32[max_row_tiles*H_local +
                       max_total_oproj + max_owner_slots], zeroed by the caller.  The kernel
                       adds 1 for every
                       attention (row tile, head), every O_proj slot and every owned AllReduce
                       slot it finished: after a launch all active entries must read 1
                       (exactly-once check; the reference has none, its status notes ask for
                       one: docs/status/STATUS.md:42-53). */
} ma_plan_desc;

/* Role weights etc.: the arguments of FusedFaOprojArWorkspace.compile()
 * (workspace.py:174-175) that the reference bakes at JIT time and this library takes per
 * launch. */
typedef struct ma_launch_args {
  int32_t w_fa, w_oproj, w_ar;
  int32_t num_ctas;               /* <= 0: one per SM                                    */
  uint32_t flags;
} ma_launch_args;

typedef struct ma_status {
  uint32_t code;                  /* 0 = clean; else which wait gave up                  */
  uint32_t site, cta, aux;
} ma_status;

typedef struct ma_plan ma_plan;

/* Device / kernel facts (no reference counterpart; the reference hard-codes 132 CTAs,
 * benchmarks/bench_fused_fa_oproj_ar.py:217). */
int ma_query_device(int device, ma_devinfo* out);

/* Stands in for FusedFaOprojArWorkspace.compile() -> cute.compile(...)
 * (workspace.py:174-194): encodes the TMA descriptors over the capacity-shaped buffers. */
int ma_plan_create(const ma_plan_desc* desc, ma_plan** out);

/* Stands in for FusedFaOprojArWorkspace.launch() (workspace.py:237-240).  Asynchronous on
 * `stream`; one launch in flight per plan.  With tp > 1 every rank must launch the same
 * layer: the kernel ends with a cross-rank barrier. */
int ma_launch(ma_plan* plan, const ma_launch_args* args, void* stream);

/* Point the plan at caller-owned inputs instead of the workspace's capacity buffers: the
 * TMA descriptors of Q, K, V and W_o are re-encoded over the given tensors, nothing is
 * copied.  The reference copies Q/K/V/W_o into the workspace on every layer
 * (workspace.py:210-231); this is the in-place alternative.  Q [tot_q, H_local, D],
 * K/V [tot_k, H_kv, D] (or the caches [tot_k/128, 128, H_kv, D] of a paged plan), W_o
 * [K_local, w_width] with hidden <= w_width and w_width % 64 == 0 (columns past the width
 * are read as zeros).  All 16-byte aligned, bf16, contiguous; they must stay valid until the
 * launch that uses them has finished.  Host-side only; takes effect at the next ma_launch. */
int ma_plan_set_inputs(ma_plan* plan, uint64_t Q, uint64_t K, uint64_t V, uint64_t W_o,
                       int64_t tot_q, int64_t tot_k, int64_t w_width);

/* Reads the device status block (synchronises `stream` first).  No reference
 * counterpart: the reference's device waits are unbounded. */
int ma_read_status(ma_plan* plan, void* stream, ma_status* out);

void ma_plan_destroy(ma_plan* plan);

/*
 * One-call fused prefill for callers that must not allocate device memory.
 * (No counterpart in the reference, whose workspace allocates everything with torch.)
 *
 * Who needs it: code that runs where cudaMalloc is off limits - inside a serving engine
 * that sized its memory pool at start-up, where one more allocation breaks the pool's
 * accounting or fails outright because the pool already holds every free byte; on a
 * latency-critical path where an allocation's implicit device synchronisation is not
 * acceptable; or in a plug-in that is handed buffers but is forbidden to create any.
 * Such a caller owns its inputs and its output but cannot give the kernel a workspace.
 *
 * The attention-output scratch, the scheduler's control words, the O_proj ready queue and
 * the tile descriptors live in ONE fixed array inside the library
 * (MA_NOALLOC_SCRATCH_BYTES of device memory per GPU that loads the library, held until
 * the process exits).  The call itself allocates nothing: it computes the tile
 * descriptors on the host, copies them and zeroes the control words with stream-ordered
 * copies into that array, encodes TMA descriptors on the host and launches the same
 * kernel as ma_launch (single rank, AllReduce = identity).
 *
 * Limits (MA_ERR_CAPACITY beyond them): num_batch <= MA_NOALLOC_MAX_BATCH,
 * row tiles R = sum ceil(q_len/128) <= MA_NOALLOC_MAX_ROW_TILES,
 * R * num_super_groups <= MA_NOALLOC_MAX_SLOTS, and
 * R * 128 * H_local * 128 * 2 bytes <= MA_NOALLOC_OSCRATCH_BYTES.
 * Shapes: head_dim 128; hidden % 64 == 0; W_o is [H_local*128, hidden] row-major with no
 * padding; `out` is the tile-padded layout [R, 128, ceil(hidden/128), 128] bf16, of which
 * only rows < valid_m and columns < hidden are written.
 *
 * The first call on a device looks up the array's device address; make that first call
 * before any stream capture.  A call on a stream that is being captured is refused with
 * MA_ERR_INVALID (it copies descriptors from a host buffer that the next call reuses).
 * Every call uses the same array: it keeps the previous
 * call's contents (what has to start from zero is cleared by the call), and two calls
 * that overlap on the GPU - different streams, or different host threads - race on it.
 * The device must be current.  The call returns once the work is queued on `stream`;
 * if `status_out` is not NULL it instead waits for the stream and fills it, returning
 * MA_ERR_DEVICE_TIMEOUT when a device-side wait gave up.  `status_out` is the only way to
 * learn of such a timeout: the status words sit in the array and no other call reads them.
 */
#define MA_NOALLOC_OSCRATCH_BYTES (16u << 20)
#define MA_NOALLOC_CONTROL_BYTES (64u << 10)
#define MA_NOALLOC_SCRATCH_BYTES (MA_NOALLOC_OSCRATCH_BYTES + MA_NOALLOC_CONTROL_BYTES)
#define MA_NOALLOC_MAX_BATCH 512
#define MA_NOALLOC_MAX_ROW_TILES 512
#define MA_NOALLOC_MAX_SLOTS 4096

typedef struct ma_noalloc_args {
  int32_t H_local, H_kv, hidden, super_group_n_tiles;
  int32_t num_batch;
  int32_t w_fa, w_oproj, num_ctas;      /* role weights; num_ctas <= 0: one per SM        */
  float softmax_scale;                  /* <= 0: 128^-0.5                                 */
  uint32_t wait_limit_ms;               /* 0: 2000                                        */
  const int32_t* seqlens_q;             /* host, [num_batch]                              */
  const int32_t* seqlens_k;             /* host, [num_batch]; NULL: same as seqlens_q     */
  uint64_t Q, K, V, W_o;                /* device, bf16                                   */
  uint64_t out;                         /* device, bf16, tile-padded layout               */
  ma_status* status_out;                /* host, may be NULL                              */
} ma_noalloc_args;

int ma_fused_prefill_noalloc(const ma_noalloc_args* args, void* stream);

/*
 * Consumer of the fused launch's output: residual add + RMSNorm, read straight from the
 * tile-padded csym buffer.  The reference lists this op as the next one after its fused
 * kernel (README.md:41-44 of the reference, "residual / RMSNorm consumer") and has no code
 * or interface for it, so the entry point mirrors nothing; the arithmetic is
 *   h   = bf16( float(y) + float(residual) )            (the residual stream, rounded once)
 *   out = bf16( float(h) * rsqrt(mean(float(h)^2) + eps) * float(weight) )
 * per token row over `hidden` columns.  Token row i of sequence b is row (i % 128) of row
 * tile (first tile of b) + i / 128 in csym; cu_q / fa_b / fa_mb are the plan's device arrays
 * of the launch that produced csym.  All pointers are device addresses, 16-byte aligned;
 * hidden % 8 == 0, hidden <= 16384 (MA_ERR_CAPACITY beyond); row_pitch = csym's row pitch in
 * elements (num_out * 128).  residual_out may be residual_in (in place).  Asynchronous on
 * `stream`; no allocation, no synchronisation.
 */
typedef struct ma_rmsnorm_args {
  uint64_t csym;           /* bf16 [num_row_tiles, 128, row_pitch]                     */
  uint64_t residual_in;    /* bf16 [tot_q, hidden]                                     */
  uint64_t weight;         /* bf16 [hidden]                                            */
  uint64_t residual_out;   /* bf16 [tot_q, hidden]                                     */
  uint64_t normed_out;     /* bf16 [tot_q, hidden]                                     */
  uint64_t cu_q, fa_b, fa_mb;   /* i32 device arrays, as in ma_plan_desc               */
  int32_t num_row_tiles, hidden, row_pitch;
  float eps;
} ma_rmsnorm_args;

int ma_residual_rmsnorm(const ma_rmsnorm_args* args, void* stream);

/*
 * Producer-side op: rotary position embedding, in place, on the packed varlen Q
 * [tot_q, H_local, 128] and on the new rows of K [tot_k, H_kv, 128] (contiguous layout),
 * before the fused launch reads them.  The reference lists the "QKV-proj / RoPE producer"
 * as a step it has not built (README.md:41-44 of the reference): no interface to mirror.
 * Rotate-half convention with the 64 frequencies inv_freq[d] (fp32, e.g. theta^(-d/64)),
 * fp32 angles and products, one rounding.  Query row i of sequence b has position (k_len_b - q_len_b) + i; the K rows
 * rotated are the last q_len_b rows of sequence b (with a cached prefix, the prefix was
 * rotated when it was written).  token_batch[i] is the sequence of packed query row i.
 * Device addresses; q and k 16-byte aligned; asynchronous on `stream`.
 */
typedef struct ma_rope_args {
  uint64_t q, k;                    /* bf16, rotated in place                           */
  uint64_t cu_q, cu_k;              /* i32 [num_batch + 1]                              */
  uint64_t token_batch;             /* i32 [tot_q]                                      */
  uint64_t inv_freq;                /* f32 [64]                                         */
  int32_t tot_q, H_local, H_kv;
  int32_t reserved0;
} ma_rope_args;

int ma_rope_qk(const ma_rope_args* args, void* stream);

const char* ma_strerror(int code);

#ifdef __cplusplus
}
#endif
#endif /* MEGAATTN_B200_H_ */
