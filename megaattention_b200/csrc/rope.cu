// Producer-side op of the fused launch: rotary position embedding on the packed varlen Q
// and on the NEW rows of K, in place, just before the launch reads them.
//
// The reference names the "QKV-proj / RoPE producer" as a step it has not built
// (README.md:41-44 of the reference); the projection itself is a plain library GEMM, the
// rotation is this kernel.  Rotate-half convention of the models the reference targets:
//   out[d]      = x[d] * cos(p w_d) - x[d + 64] * sin(p w_d)
//   out[d + 64] = x[d + 64] * cos(p w_d) + x[d] * sin(p w_d),   d < 64
// with the 64 frequencies w_d given by the caller as fp32 (theta^(-d/64), or a scaled
// variant), fp32 angles and products and one rounding to bf16.  Query row i of sequence b has
// position (k_len_b - q_len_b) + i; the K rows rotated are the last q_len_b rows of the
// sequence (the same positions): with q = k that is every K row, with a cached prefix the
// prefix was rotated when it was written.
//
// HBM bound (every element read and written once).  One CTA per token: 64 threads compute
// the token's 64 (cos, sin) pairs once, then all threads apply them to every head with
// 16-byte accesses.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/megaattn_b200.h"

namespace ma {
namespace {

constexpr int kRopeThreads = 128;

__device__ __forceinline__ float rb_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float rb_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t rb_pack(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__global__ void __launch_bounds__(kRopeThreads)
rope_kernel(uint16_t* q, uint16_t* k, const int* __restrict__ cu_q, const int* __restrict__ cu_k,
            const int* __restrict__ tok_b, const float* __restrict__ inv_freq, int tot_q, int H,
            int Hkv) {
  __shared__ float s_cos[64], s_sin[64];
  const int tid = threadIdx.x;
  for (int tok = blockIdx.x; tok < tot_q; tok += gridDim.x) {
    const int b = tok_b[tok];
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    const int k0 = cu_k[b], k_len = cu_k[b + 1] - k0;
    const int i = tok - q0;
    const int pos = (k_len - q_len) + i;
    __syncthreads();                         // the previous token's values are no longer read
    if (tid < 64) {
      // accurate sine and cosine: the angle reaches tens of thousands of radians at far
      // positions of the fast frequencies
      float sn, cs;
      sincosf(static_cast<float>(pos) * inv_freq[tid], &sn, &cs);
      s_cos[tid] = cs;
      s_sin[tid] = sn;
    }
    __syncthreads();
    uint16_t* qrow = q + static_cast<size_t>(tok) * H * 128;
    uint16_t* krow = k + static_cast<size_t>(k0 + pos) * Hkv * 128;
    const int nq = H * 8, nall = (H + Hkv) * 8;      // 16-byte chunks of the first halves
    for (int idx = tid; idx < nall; idx += kRopeThreads) {
      uint16_t* base = (idx < nq) ? qrow + (idx >> 3) * 128 : krow + ((idx - nq) >> 3) * 128;
      const int d = (idx & 7) * 8;
      uint4* plo = reinterpret_cast<uint4*>(base + d);
      uint4* phi = reinterpret_cast<uint4*>(base + d + 64);
      const uint4 lo = *plo, hi = *phi;
      const uint32_t lv[4] = {lo.x, lo.y, lo.z, lo.w}, hv[4] = {hi.x, hi.y, hi.z, hi.w};
      uint32_t ol[4], oh[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float c0 = s_cos[d + 2 * j], s0 = s_sin[d + 2 * j];
        const float c1 = s_cos[d + 2 * j + 1], s1 = s_sin[d + 2 * j + 1];
        const float a0 = rb_lo(lv[j]), a1 = rb_hi(lv[j]), b0 = rb_lo(hv[j]), b1 = rb_hi(hv[j]);
        ol[j] = rb_pack(a0 * c0 - b0 * s0, a1 * c1 - b1 * s1);
        oh[j] = rb_pack(b0 * c0 + a0 * s0, b1 * c1 + a1 * s1);
      }
      *plo = make_uint4(ol[0], ol[1], ol[2], ol[3]);
      *phi = make_uint4(oh[0], oh[1], oh[2], oh[3]);
    }
  }
}

}  // namespace
}  // namespace ma

extern "C" int ma_rope_qk(const ma_rope_args* a, void* stream) {
  if (!a || !a->q || !a->k || !a->cu_q || !a->cu_k || !a->token_batch || !a->inv_freq)
    return MA_ERR_INVALID;
  if (a->tot_q < 0 || a->H_local <= 0 || a->H_kv <= 0) return MA_ERR_INVALID;
  if ((a->q & 15u) || (a->k & 15u)) return MA_ERR_INVALID;            // 16-byte accesses
  if (a->tot_q == 0) return MA_OK;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return MA_ERR_CUDA;
  const int grid = a->tot_q < sms * 8 ? a->tot_q : sms * 8;
  ma::rope_kernel<<<grid, ma::kRopeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint16_t*>(a->q), reinterpret_cast<uint16_t*>(a->k),
      reinterpret_cast<const int*>(a->cu_q), reinterpret_cast<const int*>(a->cu_k),
      reinterpret_cast<const int*>(a->token_batch), reinterpret_cast<const float*>(a->inv_freq),
      a->tot_q, a->H_local, a->H_kv);
  return cudaGetLastError() == cudaSuccess ? MA_OK : MA_ERR_CUDA;
}
