// C ABI (include/megaattn_b200.h): plan creation (TMA descriptor encoding), launch,
// status read-back.  Host code only; the kernel lives in fused_prefill.cu.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <new>

#include "../../include/megaattn_b200.h"
#include "kparams.h"

namespace ma {
cudaError_t launch_fused_prefill(const CUtensorMap* maps, const KParams& kp, int num_ctas,
                                 cudaStream_t stream);
cudaError_t fused_prefill_attributes(cudaFuncAttributes* out);
int encode_path_maps(CUtensorMap* maps, uint64_t Q, uint64_t K, uint64_t V, uint64_t oscr,
                     uint64_t W, uint64_t H, uint64_t Hkv, uint64_t tot_q, uint64_t tot_k,
                     uint64_t row_tiles, uint64_t w_width, uint64_t csym, uint64_t hidden,
                     uint64_t csym_pitch);
}  // namespace ma

struct ma_plan {
  ma::KParams kp;
  CUtensorMap maps[6];   // Q, K, V, O_scratch (2-D), W_o, C_sym (store)
  int device;
  int num_sms;
  ma_plan_desc desc;     // as given at creation (shapes for re-encoding)
};

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encoder() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
          cudaSuccess || qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

// bf16 tensor, innermost dimension contiguous, 128-byte swizzle, zero fill out of bounds
int encode(CUtensorMap* out, uint64_t base, int rank, const uint64_t* dims,
           const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn enc = get_encoder();
  if (!enc) return MA_ERR_CUDA;
  if (base == 0 || (base & 15u)) return MA_ERR_INVALID;
  cuuint64_t d[4], s[3];
  cuuint32_t b[4], e[4] = {1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) {
    if (strides_bytes[i] & 15u) return MA_ERR_INVALID;
    s[i] = strides_bytes[i];
  }
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank),
                   reinterpret_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MA_OK : MA_ERR_CUDA;
}

int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace

// The five TMA descriptors of the path.  A 128 x 128 tile of Q, K or V is fetched by ONE
// instruction as two 64-wide swizzled panels: the tensor is described as
// {64 d, tokens, 2 d-halves, heads} so the box {64, 128, 2, 1} lands panel after panel.
// W_o [K_local, width] is described as {64 n, K_local, width/64 panels}: the box
// {64, 64, 4} is a 64-k slab of 256 output columns, panel after panel.
int ma::encode_path_maps(CUtensorMap* maps, uint64_t Q, uint64_t K, uint64_t V, uint64_t oscr,
                         uint64_t W, uint64_t H, uint64_t Hkv, uint64_t tot_q, uint64_t tot_k,
                         uint64_t row_tiles, uint64_t w_width, uint64_t csym, uint64_t hidden,
                         uint64_t csym_pitch) {
  if (w_width % 64) return MA_ERR_INVALID;
  const uint64_t KL = H * 128;
  int rc;
  {
    const uint64_t dims[4] = {64, tot_q, 2, H};
    const uint64_t str[3] = {H * 256, 128, 256};
    const uint32_t box[4] = {64, 128, 2, 1};
    rc = encode(&maps[0], Q, 4, dims, str, box);
  }
  if (rc == MA_OK) {
    const uint64_t dims[4] = {64, tot_k, 2, Hkv};
    const uint64_t str[3] = {Hkv * 256, 128, 256};
    const uint32_t box[4] = {64, 128, 2, 1};
    rc = encode(&maps[1], K, 4, dims, str, box);
    if (rc == MA_OK) rc = encode(&maps[2], V, 4, dims, str, box);
  }
  if (rc == MA_OK) {
    const uint64_t dims[2] = {KL, row_tiles * 128};
    const uint64_t str[1] = {KL * 2};
    const uint32_t box[2] = {64, 128};
    rc = encode(&maps[3], oscr, 2, dims, str, box);
  }
  if (rc == MA_OK) {
    const uint64_t dims[3] = {64, KL, w_width / 64};
    const uint64_t str[2] = {w_width * 2, 128};
    const uint32_t box[3] = {64, 64, 4};
    rc = encode(&maps[4], W, 3, dims, str, box);
  }
  if (rc == MA_OK) {
    // output tiles are stored through TMA: [rows, hidden] with the padded row pitch, so a
    // store is clipped at `hidden` and padding columns are never written
    const uint64_t dims[2] = {hidden, row_tiles * 128};
    const uint64_t str[1] = {csym_pitch * 2};
    const uint32_t box[2] = {64, 128};
    rc = encode(&maps[5], csym, 2, dims, str, box);
  }
  return rc;
}

extern "C" {

const char* ma_strerror(int code) {
  switch (code) {
    case MA_OK: return "ok";
    case MA_ERR_INVALID: return "invalid argument or unsupported shape";
    case MA_ERR_CUDA: return "CUDA call failed";
    case MA_ERR_NOT_SM100: return "device is not compute capability 10.x";
    case MA_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case MA_ERR_CAPACITY: return "request exceeds a stated maximum";
    default: return "unknown error";
  }
}

int ma_query_device(int device, ma_devinfo* out) {
  if (!out) return MA_ERR_INVALID;
  memset(out, 0, sizeof(*out));
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess)
    return MA_ERR_CUDA;
  out->cc_major = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, device); out->cc_minor = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device); out->num_sms = v;
  cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  out->max_smem_optin = v;
  out->kernel_threads = ma::kThreads;
  out->kernel_smem_bytes = ma::kSmemDynamic;
  out->max_ctas = out->num_sms;   // 1 CTA per SM: the kernel takes > half of shared memory
  if (out->cc_major != 10) return MA_ERR_NOT_SM100;
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(device);
  cudaFuncAttributes fa;
  cudaError_t e = ma::fused_prefill_attributes(&fa);
  cudaSetDevice(cur);
  if (e != cudaSuccess) return MA_ERR_CUDA;
  out->kernel_regs = fa.numRegs;
  return MA_OK;
}

int ma_plan_create(const ma_plan_desc* d, ma_plan** out) {
  if (!d || !out) return MA_ERR_INVALID;
  *out = nullptr;
  if (d->D != 128) return MA_ERR_INVALID;                      // head_dim 128 only
  if (d->tp_size < 1 || d->tp_size > MA_MAX_TP || d->rank < 0 || d->rank >= d->tp_size)
    return MA_ERR_INVALID;
  if (d->H_local < 1 || d->H_kv < 1 || d->H_local % d->H_kv) return MA_ERR_INVALID;
  if (d->super_group_n_tiles < 1 || d->super_group_n_tiles > 4) return MA_ERR_INVALID;
  if (d->hidden < 1 || d->max_row_tiles < 1 || d->max_batch < 1) return MA_ERR_INVALID;
  if (d->max_tot_q < 1 || d->max_tot_k < 1) return MA_ERR_INVALID;
  const uint64_t need[] = {d->Q, d->K, d->V, d->W_o, d->o_scratch, d->csym, d->ctrl, d->sync_ctrl,
                           d->actv, d->head_ready, d->oproj_queue, d->ready_count,
                           d->ar_done_bits, d->nvl_signal, d->cu_q, d->cu_k, d->fa_b, d->fa_mb,
                           d->status};
  for (uint64_t a : need) if (a == 0) return MA_ERR_INVALID;
  if (d->page_table && (!d->cache_seqlens || d->max_pages_per_seq < 1 || d->max_tot_k % 128))
    return MA_ERR_INVALID;
  if (d->tp_size > 1) {
    if (d->csym_multicast == 0) return MA_ERR_INVALID;
    for (int r = 0; r < d->tp_size; ++r)
      if (!d->peer_ready_count[r] || !d->peer_nvl_signal[r])
        return MA_ERR_INVALID;
  }

  int cc = 0, sms = 0;
  if (cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, d->device) != cudaSuccess)
    return MA_ERR_CUDA;
  if (cc != 10) return MA_ERR_NOT_SM100;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->device);

  ma_plan* pl = new (std::nothrow) ma_plan;
  if (!pl) return MA_ERR_CUDA;
  memset(pl, 0, sizeof(*pl));
  pl->device = d->device;
  pl->num_sms = sms;
  pl->desc = *d;

  ma::KParams& k = pl->kp;
  k.H = d->H_local; k.Hkv = d->H_kv; k.q_per_kv = d->H_local / d->H_kv;
  k.K_local = d->H_local * 128; k.hidden = d->hidden;
  k.num_out = cdiv(d->hidden, 128);
  k.sg = d->super_group_n_tiles;
  k.nsg = cdiv(k.num_out, k.sg);
  k.tp = d->tp_size; k.rank = d->rank;
  const float scale = d->softmax_scale > 0.f ? d->softmax_scale : 0.08838834764831845f;
  k.scale_log2 = scale * 1.4426950408889634f;
  k.pair = (k.q_per_kv % 2 == 0) ? 1 : 0;
  k.sep = (!k.pair && k.H >= 2) ? 1 : 0;
  k.max_row_tiles = d->max_row_tiles;
  const long long max_total = static_cast<long long>(d->max_row_tiles) * k.nsg;
  k.max_owner_slots = static_cast<int>((max_total + d->tp_size - 1) / d->tp_size);
  k.max_owner_words = cdiv(k.max_owner_slots, 64);
  k.wait_limit_ns = 1000000ull * (d->wait_limit_ms ? d->wait_limit_ms : 2000u);
  k.o_scratch = reinterpret_cast<uint16_t*>(d->o_scratch);
  k.csym = reinterpret_cast<uint16_t*>(d->csym);
  k.ctrl = reinterpret_cast<uint32_t*>(d->ctrl);
  k.sync_ctrl = reinterpret_cast<uint32_t*>(d->sync_ctrl);
  k.actv = reinterpret_cast<const int*>(d->actv);
  k.head_ready = reinterpret_cast<uint32_t*>(d->head_ready);
  k.oproj_queue = reinterpret_cast<uint32_t*>(d->oproj_queue);
  k.ready_count = reinterpret_cast<uint32_t*>(d->ready_count);
  k.ar_done_bits = reinterpret_cast<unsigned long long*>(d->ar_done_bits);
  k.nvl_signal = reinterpret_cast<int*>(d->nvl_signal);
  k.cu_q = reinterpret_cast<const int*>(d->cu_q);
  k.cu_k = reinterpret_cast<const int*>(d->cu_k);
  k.fa_b = reinterpret_cast<const int*>(d->fa_b);
  k.fa_mb = reinterpret_cast<const int*>(d->fa_mb);
  k.fa_order = reinterpret_cast<const int*>(d->fa_order);
  k.page_table = reinterpret_cast<const int*>(d->page_table);
  k.cache_seqlens = reinterpret_cast<const int*>(d->cache_seqlens);
  k.pps = d->max_pages_per_seq;
  k.status = reinterpret_cast<uint32_t*>(d->status);
#ifdef MA_AUDIT
  k.audit = reinterpret_cast<uint32_t*>(d->audit);
#else
  if (d->audit) { delete pl; return MA_ERR_INVALID; }     // counters need the audit build
#endif
  k.audit_op_base = d->max_row_tiles * d->H_local;
  k.audit_ar_base = k.audit_op_base + static_cast<int>(max_total);
  k.csym_mc = d->csym_multicast;
  for (int r = 0; r < MA_MAX_TP; ++r) {
    k.peer_rc[r] = d->peer_ready_count[r];
    k.peer_nvl[r] = d->peer_nvl_signal[r];
    k.peer_csym[r] = d->peer_csym[r];
  }

  const uint64_t H = d->H_local, Hkv = d->H_kv;
  const uint64_t hidden_pad = static_cast<uint64_t>(k.num_out) * 128;
  int rc = ma::encode_path_maps(pl->maps, d->Q, d->K, d->V, d->o_scratch, d->W_o, H, Hkv,
                                static_cast<uint64_t>(d->max_tot_q),
                                static_cast<uint64_t>(d->max_tot_k),
                                static_cast<uint64_t>(d->max_row_tiles), hidden_pad, d->csym,
                                static_cast<uint64_t>(d->hidden), hidden_pad);
  if (rc != MA_OK) { delete pl; return rc; }
  *out = pl;
  return MA_OK;
}

int ma_launch(ma_plan* pl, const ma_launch_args* a, void* stream) {
  if (!pl || !a) return MA_ERR_INVALID;
  ma::KParams kp = pl->kp;
  kp.w_fa = a->w_fa; kp.w_oproj = a->w_oproj;
  kp.w_ar = (kp.tp > 1) ? a->w_ar : 0;          // one rank: no AllReduce role
  kp.flags = a->flags;
  // Flag combinations that would send the kernel down a path its buffers do not back are
  // refused here, before anything is launched.
  const uint32_t stage = kp.flags & (MA_FLAG_FA_ONLY | MA_FLAG_AR_ONLY | MA_FLAG_NO_AR |
                                     MA_FLAG_OPROJ_ONLY);
  if (stage & (stage - 1u)) return MA_ERR_INVALID;              // at most one stage selector
  if ((kp.flags & MA_FLAG_AR_ONLY) && (kp.tp < 2 || kp.csym_mc == 0)) return MA_ERR_INVALID;
  if ((kp.flags & MA_FLAG_OPROJ_ONLY) && kp.tp != 1) return MA_ERR_INVALID;
  if ((kp.flags & MA_FLAG_AR_P2P) &&
      (kp.tp != 2 || !pl->desc.peer_csym[0] || !pl->desc.peer_csym[1]))
    return MA_ERR_INVALID;
  if (kp.flags & ~(MA_FLAG_FA_ONLY | MA_FLAG_DRAIN_FIRST | MA_FLAG_TILE_ORDER | MA_FLAG_AR_ONLY |
                   MA_FLAG_NO_AR | MA_FLAG_OPROJ_ONLY | MA_FLAG_AR_P2P))
    return MA_ERR_INVALID;
  if (kp.w_fa < 0 || kp.w_oproj < 0 || kp.w_ar < 0 || kp.w_fa + kp.w_oproj + kp.w_ar < 1)
    return MA_ERR_INVALID;
  int n = a->num_ctas > 0 ? a->num_ctas : pl->num_sms;
  if (n > pl->num_sms) n = pl->num_sms;          // one CTA per SM: every CTA must be resident (CTAs wait on each other's work)
  cudaError_t e = ma::launch_fused_prefill(pl->maps, kp, n, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MA_OK : MA_ERR_CUDA;
}

int ma_plan_set_inputs(ma_plan* pl, uint64_t Q, uint64_t K, uint64_t V, uint64_t W_o,
                       int64_t tot_q, int64_t tot_k, int64_t w_width) {
  if (!pl || !Q || !K || !V || !W_o) return MA_ERR_INVALID;
  const ma_plan_desc& d = pl->desc;
  if (tot_q < 1 || tot_k < 1 || w_width < d.hidden || w_width % 64) return MA_ERR_INVALID;
  if (d.page_table && tot_k % 128) return MA_ERR_INVALID;
  CUtensorMap fresh[6];
  const int rc = ma::encode_path_maps(fresh, Q, K, V, d.o_scratch, W_o,
                                      static_cast<uint64_t>(d.H_local),
                                      static_cast<uint64_t>(d.H_kv),
                                      static_cast<uint64_t>(tot_q), static_cast<uint64_t>(tot_k),
                                      static_cast<uint64_t>(d.max_row_tiles),
                                      static_cast<uint64_t>(w_width), d.csym,
                                      static_cast<uint64_t>(d.hidden),
                                      static_cast<uint64_t>(pl->kp.num_out) * 128);
  if (rc != MA_OK) return rc;
  pl->maps[0] = fresh[0]; pl->maps[1] = fresh[1]; pl->maps[2] = fresh[2]; pl->maps[4] = fresh[4];
  return MA_OK;
}

int ma_read_status(ma_plan* pl, void* stream, ma_status* out) {
  if (!pl || !out) return MA_ERR_INVALID;
  uint32_t h[4] = {0, 0, 0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(h, pl->kp.status, sizeof(h), cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return MA_ERR_CUDA;
  if (cudaStreamSynchronize(s) != cudaSuccess) return MA_ERR_CUDA;
  out->code = h[0]; out->site = h[1]; out->cta = h[2]; out->aux = h[3];
  return h[0] == 0 ? MA_OK : MA_ERR_DEVICE_TIMEOUT;
}

void ma_plan_destroy(ma_plan* pl) { delete pl; }

}  // extern "C"
