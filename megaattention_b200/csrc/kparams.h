// Kernel parameter block shared by the host launcher and the device code.
#pragma once
#include <stdint.h>

namespace ma {

// Control-word indices: same numbering as the reference kernel
// (src/mega_attention/kernels/sm90/fused_fa_oproj_ar.py:47-67), which host code reads.
enum : int {
  C_FA_COUNTER = 0, C_FA_DONE = 1, C_OP_RESERVE = 2, C_OP_PUBLISH = 3,
  C_OP_CONSUME = 4, C_OP_DONE = 5, C_AR_DONE = 6, C_AR_CURSOR = 7
};
enum : int { S_GS_QUIESCE = 0, S_GS_CLEANDONE = 1, S_NVL_COUNTER = 2 };
enum : int { MODE_IDLE = 0, MODE_FA = 1, MODE_OPROJ = 2, MODE_AR = 3, MODE_DONE = 4 };

// status[0] codes
enum : uint32_t {
  ST_OK = 0, ST_TIMEOUT_MBAR = 1, ST_TIMEOUT_PUBLISH = 2, ST_TIMEOUT_GRID = 3,
  ST_TIMEOUT_NVL = 4, ST_BAD_DESC = 5, ST_TIMEOUT_IDLE = 6
};

constexpr int kMaxTp = 8;

struct KParams {
  int H, Hkv, q_per_kv, K_local, hidden, num_out, sg, nsg;
  int tp, rank;
  int w_fa, w_oproj, w_ar;
  uint32_t flags;
  float scale_log2;
  int pair;                       // 1: an FA task is two q heads sharing a kv head (q_per_kv even)
  int sep;                        // 1: an FA task is two q heads, each with K/V stages of its own
                                  //    (q_per_kv odd, MHA included; the last head of an odd count alone)
  int max_row_tiles, max_owner_slots, max_owner_words;
  unsigned long long wait_limit_ns;

  uint16_t* o_scratch;            // bf16 bits
  uint16_t* csym;
  uint32_t* ctrl;
  uint32_t* sync_ctrl;
  const int* actv;
  uint32_t* head_ready;
  uint32_t* oproj_queue;
  uint32_t* ready_count;
  unsigned long long* ar_done_bits;
  int* nvl_signal;
  const int* cu_q;
  const int* cu_k;
  const int* fa_b;
  const int* fa_mb;
  const int* fa_order;            // row tiles in claim order (longest first), or null
  const int* page_table;          // paged KV: [batch][pps] page of each 128-key block, or null
  const int* cache_seqlens;       // paged KV: KV length per sequence
  int pps;                        // page-table row pitch
  uint32_t* status;
  uint32_t* audit;                // optional execution counters (null: off): one per attention
                                  // (row tile, head), per O_proj slot, per owned AllReduce slot
  int audit_op_base, audit_ar_base;

  unsigned long long csym_mc;
  unsigned long long peer_rc[kMaxTp];
  unsigned long long peer_nvl[kMaxTp];
  unsigned long long peer_csym[kMaxTp];   // every rank's C_sym (peer-load AllReduce, tp 2)
};

constexpr int kThreads = 384;
constexpr int kSmemDynamic = 65536 + 5 * 32768 + 1024;   // Q x2, K/V ring x5, align slack

}  // namespace ma
