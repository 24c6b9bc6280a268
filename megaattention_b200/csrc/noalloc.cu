// ma_fused_prefill_noalloc: the fused prefill for callers that may not allocate device
// memory.  All scratch the kernel needs sits in one file-scope device array; see the
// declaration in include/megaattn_b200.h for who this is for, the limits and the rules
// (first call before any stream capture; a capturing stream is refused; calls share the
// array, overlapping calls race).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/megaattn_b200.h"
#include "kparams.h"

namespace ma {
cudaError_t launch_fused_prefill(const CUtensorMap* maps, const KParams& kp, int num_ctas,
                                 cudaStream_t stream);
int encode_path_maps(CUtensorMap* maps, uint64_t Q, uint64_t K, uint64_t V, uint64_t oscr,
                     uint64_t W, uint64_t H, uint64_t Hkv, uint64_t tot_q, uint64_t tot_k,
                     uint64_t row_tiles, uint64_t w_width, uint64_t csym, uint64_t hidden,
                     uint64_t csym_pitch);
}  // namespace ma

namespace {

// The one scratch array.  In host code this name is only a handle for the runtime, not a
// device address: the address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MA_NOALLOC_SCRATCH_BYTES];

// Layout of the first MA_NOALLOC_CONTROL_BYTES (byte offsets); O_scratch follows.
constexpr size_t kOffCtrl = 0;            // u32[8]
constexpr size_t kOffSync = 64;           // u32[3]
constexpr size_t kOffStatus = 128;        // u32[8]
constexpr size_t kOffNvl = 192;           // i32[2]
constexpr size_t kOffMeta = 256;          // packed i32: actv[8] | cu_q | cu_k | fa_b | fa_mb
constexpr size_t kMetaInts = 8 + 2 * (MA_NOALLOC_MAX_BATCH + 1) + 2 * MA_NOALLOC_MAX_ROW_TILES;
constexpr size_t kOffHeadReady = 8704;    // u32[MAX_ROW_TILES]
constexpr size_t kOffDoneBits = 10752;    // u64[MAX_SLOTS/64]
constexpr size_t kOffReadyBits = 11264;   // u64[MAX_SLOTS/64]
constexpr size_t kOffReadyCount = 11776;  // u32[MAX_SLOTS]
constexpr size_t kOffQueue = 28160;       // u32[MAX_SLOTS]
constexpr size_t kOffEnd = kOffQueue + 4 * MA_NOALLOC_MAX_SLOTS;
static_assert(kOffMeta + 4 * kMetaInts <= kOffHeadReady, "meta overlaps head_ready");
static_assert(kOffHeadReady + 4 * MA_NOALLOC_MAX_ROW_TILES <= kOffDoneBits, "layout");
static_assert(kOffDoneBits + MA_NOALLOC_MAX_SLOTS / 8 <= kOffReadyBits, "layout");
static_assert(kOffReadyBits + MA_NOALLOC_MAX_SLOTS / 8 <= kOffReadyCount, "layout");
static_assert(kOffReadyCount + 4 * MA_NOALLOC_MAX_SLOTS <= kOffQueue, "layout");
static_assert(kOffEnd <= MA_NOALLOC_CONTROL_BYTES, "control region too small");

unsigned char* g_scratch_addr[64] = {};   // per device, filled on the first call there

int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MA_ERR_CUDA;
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return MA_ERR_CUDA;
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return MA_OK;
}

}  // namespace

extern "C" int ma_fused_prefill_noalloc(const ma_noalloc_args* a, void* stream_) {
  if (!a || !a->seqlens_q || !a->Q || !a->K || !a->V || !a->W_o || !a->out) return MA_ERR_INVALID;
  if (a->H_local < 1 || a->H_kv < 1 || a->H_local % a->H_kv) return MA_ERR_INVALID;
  if (a->hidden < 64 || a->hidden % 64) return MA_ERR_INVALID;
  if (a->super_group_n_tiles < 1 || a->super_group_n_tiles > 4) return MA_ERR_INVALID;
  if (a->num_batch < 1) return MA_ERR_INVALID;
  if (a->num_batch > MA_NOALLOC_MAX_BATCH) return MA_ERR_CAPACITY;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  // ---- tile descriptors on the host (same arithmetic as metadata/row_desc.py)
  static thread_local int32_t meta[kMetaInts];
  const int B = a->num_batch;
  int32_t* actv = meta;
  int32_t* cu_q = meta + 8;
  int32_t* cu_k = cu_q + (B + 1);
  long long tq = 0, tk = 0;
  int R = 0;
  cu_q[0] = 0; cu_k[0] = 0;
  for (int b = 0; b < B; ++b) {
    const long long lq = a->seqlens_q[b];
    const long long lk = a->seqlens_k ? a->seqlens_k[b] : lq;
    if (lq <= 0 || lk < lq) return MA_ERR_INVALID;
    tq += lq; tk += lk;
    if (tq > 0x7fffffffLL || tk > 0x7fffffffLL) return MA_ERR_CAPACITY;
    cu_q[b + 1] = static_cast<int32_t>(tq);
    cu_k[b + 1] = static_cast<int32_t>(tk);
    R += static_cast<int>((lq + 127) / 128);
    if (R > MA_NOALLOC_MAX_ROW_TILES) return MA_ERR_CAPACITY;
  }
  int32_t* fa_b = cu_k + (B + 1);
  int32_t* fa_mb = fa_b + R;
  for (int b = 0, t = 0; b < B; ++b)
    for (int j = 0; j < (a->seqlens_q[b] + 127) / 128; ++j, ++t) { fa_b[t] = b; fa_mb[t] = j; }
  const int num_out = (a->hidden + 127) / 128;
  const int sg = a->super_group_n_tiles;
  const int nsg = (num_out + sg - 1) / sg;
  const long long total = static_cast<long long>(R) * nsg;
  if (total > MA_NOALLOC_MAX_SLOTS) return MA_ERR_CAPACITY;
  const int K_local = a->H_local * 128;
  if (static_cast<unsigned long long>(R) * 128ull * K_local * 2ull > MA_NOALLOC_OSCRATCH_BYTES)
    return MA_ERR_CAPACITY;
  actv[0] = R * a->H_local; actv[1] = static_cast<int32_t>(total); actv[2] = R;
  actv[3] = static_cast<int32_t>(total); actv[4] = static_cast<int32_t>((total + 63) / 64);
  actv[5] = static_cast<int32_t>(total); actv[6] = 0; actv[7] = 0;
  const size_t meta_ints = 8 + 2 * static_cast<size_t>(B + 1) + 2 * static_cast<size_t>(R);

  // ---- the device, then the scratch array's device address (set-up on the first call
  //      per device)
  int dev = 0, cc = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MA_ERR_CUDA;
  if (cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return MA_ERR_CUDA;
  if (cc != 10) return MA_ERR_NOT_SM100;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // The call copies this call's descriptors from a host buffer it reuses and, with
  // status_out, synchronises the stream: a stream that is being captured is refused.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) return MA_ERR_CUDA;
  if (cap != cudaStreamCaptureStatusNone) return MA_ERR_INVALID;
  unsigned char* scr = nullptr;
  int rc = scratch_for_current_device(&scr);
  if (rc != MA_OK) return rc;

  // ---- clear what must start at zero, then bring in this call's descriptors
  if (cudaMemsetAsync(scr, 0, MA_NOALLOC_CONTROL_BYTES, stream) != cudaSuccess) return MA_ERR_CUDA;
  if (cudaMemcpyAsync(scr + kOffMeta, meta, meta_ints * sizeof(int32_t), cudaMemcpyHostToDevice,
                      stream) != cudaSuccess)
    return MA_ERR_CUDA;

  ma::KParams k;
  memset(&k, 0, sizeof(k));
  k.H = a->H_local; k.Hkv = a->H_kv; k.q_per_kv = a->H_local / a->H_kv;
  k.K_local = K_local; k.hidden = a->hidden; k.num_out = num_out; k.sg = sg; k.nsg = nsg;
  k.tp = 1; k.rank = 0;
  k.w_fa = a->w_fa > 0 ? a->w_fa : 2; k.w_oproj = a->w_oproj > 0 ? a->w_oproj : 1; k.w_ar = 0;
  k.flags = 0;
  const float scale = a->softmax_scale > 0.f ? a->softmax_scale : 0.08838834764831845f;
  k.scale_log2 = scale * 1.4426950408889634f;
  k.pair = (k.q_per_kv % 2 == 0) ? 1 : 0;
  k.max_row_tiles = R;
  k.max_owner_slots = static_cast<int>(total);
  k.max_owner_words = static_cast<int>((total + 63) / 64);
  k.wait_limit_ns = 1000000ull * (a->wait_limit_ms ? a->wait_limit_ms : 2000u);
  int32_t* dmeta = reinterpret_cast<int32_t*>(scr + kOffMeta);
  k.o_scratch = reinterpret_cast<uint16_t*>(scr + MA_NOALLOC_CONTROL_BYTES);
  k.csym = reinterpret_cast<uint16_t*>(a->out);
  k.ctrl = reinterpret_cast<uint32_t*>(scr + kOffCtrl);
  k.sync_ctrl = reinterpret_cast<uint32_t*>(scr + kOffSync);
  k.status = reinterpret_cast<uint32_t*>(scr + kOffStatus);
  k.nvl_signal = reinterpret_cast<int*>(scr + kOffNvl);
  k.actv = dmeta;
  k.cu_q = dmeta + 8;
  k.cu_k = k.cu_q + (B + 1);
  k.fa_b = k.cu_k + (B + 1);
  k.fa_mb = k.fa_b + R;
  k.head_ready = reinterpret_cast<uint32_t*>(scr + kOffHeadReady);
  k.ar_done_bits = reinterpret_cast<unsigned long long*>(scr + kOffDoneBits);
  k.ready_count = reinterpret_cast<uint32_t*>(scr + kOffReadyCount);
  k.oproj_queue = reinterpret_cast<uint32_t*>(scr + kOffQueue);

  // ---- TMA descriptors over the caller's tensors and the scratch (host-side encoding)
  CUtensorMap maps[6];
  // W_o is read in 64-column panels straight from the caller's tensor: hidden % 64 == 0
  rc = ma::encode_path_maps(maps, a->Q, a->K, a->V, reinterpret_cast<uint64_t>(k.o_scratch), a->W_o,
                            static_cast<uint64_t>(a->H_local), static_cast<uint64_t>(a->H_kv),
                            static_cast<uint64_t>(tq), static_cast<uint64_t>(tk),
                            static_cast<uint64_t>(R), static_cast<uint64_t>(a->hidden), a->out,
                            static_cast<uint64_t>(a->hidden), static_cast<uint64_t>(num_out) * 128);
  if (rc != MA_OK) return rc;

  int n = a->num_ctas > 0 ? a->num_ctas : sms;
  if (n > sms) n = sms;
  if (ma::launch_fused_prefill(maps, k, n, stream) != cudaSuccess) return MA_ERR_CUDA;

  if (a->status_out) {
    uint32_t h[4] = {0, 0, 0, 0};
    if (cudaMemcpyAsync(h, k.status, sizeof(h), cudaMemcpyDeviceToHost, stream) != cudaSuccess)
      return MA_ERR_CUDA;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return MA_ERR_CUDA;
    a->status_out->code = h[0]; a->status_out->site = h[1];
    a->status_out->cta = h[2]; a->status_out->aux = h[3];
    if (h[0] != 0) return MA_ERR_DEVICE_TIMEOUT;
  }
  return MA_OK;
}
