// Consumer of the fused launch's output: residual add + RMSNorm over the hidden dimension,
// read straight from the tile-padded C_sym buffer (no de-tiling copy in between).
//
// The reference names this op as the next step after its fused kernel ("residual / RMSNorm
// consumer", README.md:41-44 of the reference) and ships no code for it; the arithmetic is
// the usual one of the models it targets: h = residual + y rounded to bf16 (the residual
// stream), out = h * rsqrt(mean(h^2) + eps) * weight in fp32, rounded once.
//
// HBM bound: every token row is read twice (y, residual) and written twice (residual,
// normed output), 8 bytes per element.  One CTA of 256 threads per token row, 16-byte
// accesses, the row's values kept in registers between the two passes; a persistent grid
// of a few CTAs per SM walks the 128-row tiles and skips the padding rows.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/megaattn_b200.h"

namespace ma {
namespace {

constexpr int kRnThreads = 256;

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// read once: do not keep in L1.  (Plain loads, not the read-only path: the residual may be
// updated in place, each thread writing back exactly the chunks it read.)
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// NCH: 16-byte chunks per thread, T: threads per CTA (hidden <= NCH * T * 8).  Rows wider
// than 8192 columns take 512 threads with four chunks each (two CTAs per SM) rather than
// 256 threads with eight: the latter needs 126 registers for the row and weight values.
template <int NCH, int T>
__global__ void __launch_bounds__(T, 1024 / T)
residual_rmsnorm_kernel(const uint16_t* __restrict__ csym, const uint16_t* res_in,
                        const uint16_t* __restrict__ weight, uint16_t* res_out,
                        uint16_t* __restrict__ normed, const int* __restrict__ cu_q,
                        const int* __restrict__ fa_b, const int* __restrict__ fa_mb,
                        int num_row_tiles, int hidden, int row_pitch, float eps) {
  __shared__ float s_part[2][T / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunk = hidden >> 3;
  uint4 w[NCH];
#pragma unroll
  for (int k = 0; k < NCH; ++k) {
    const int c = tid + k * T;
    w[k] = (c < nchunk) ? reinterpret_cast<const uint4*>(weight)[c] : make_uint4(0, 0, 0, 0);
  }
  const float inv_n = 1.f / static_cast<float>(hidden);
  uint32_t turn = 0;
  for (int slot = blockIdx.x; slot < num_row_tiles * 128; slot += gridDim.x) {
    const int t = slot >> 7, r = slot & 127;
    const int b = fa_b[t];
    const int q0 = cu_q[b];
    const int row = fa_mb[t] * 128 + r;
    if (row >= cu_q[b + 1] - q0) continue;          // padding row of a partial tile (whole CTA)
    const uint4* y4 = reinterpret_cast<const uint4*>(csym + static_cast<size_t>(slot) * row_pitch);
    const size_t tok = static_cast<size_t>(q0 + row) * hidden;
    const uint4* r4 = reinterpret_cast<const uint4*>(res_in + tok);
    uint4 h[NCH];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = tid + k * T;
      if (c < nchunk) {
        const uint4 a = ld_stream(y4 + c), d = ld_stream(r4 + c);
        const uint32_t av[4] = {a.x, a.y, a.z, a.w}, dv[4] = {d.x, d.y, d.z, d.w};
        uint32_t hv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hv[i] = pack_bf16(bf16_lo(av[i]) + bf16_lo(dv[i]), bf16_hi(av[i]) + bf16_hi(dv[i]));
          const float x0 = bf16_lo(hv[i]), x1 = bf16_hi(hv[i]);
          ss = fmaf(x0, x0, ss);
          ss = fmaf(x1, x1, ss);
        }
        h[k] = make_uint4(hv[0], hv[1], hv[2], hv[3]);
        reinterpret_cast<uint4*>(res_out + tok)[c] = h[k];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float* part = s_part[turn & 1u];                 // two buffers: one barrier per row
    ++turn;
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < T / 32; ++i) tot += part[i];
    const float rstd = rsqrtf(tot * inv_n + eps);
#pragma unroll
    for (int k = 0; k < NCH; ++k) {
      const int c = tid + k * T;
      if (c < nchunk) {
        const uint32_t hv[4] = {h[k].x, h[k].y, h[k].z, h[k].w};
        const uint32_t wv[4] = {w[k].x, w[k].y, w[k].z, w[k].w};
        uint32_t ov[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          ov[i] = pack_bf16(bf16_lo(hv[i]) * rstd * bf16_lo(wv[i]),
                            bf16_hi(hv[i]) * rstd * bf16_hi(wv[i]));
        reinterpret_cast<uint4*>(normed + tok)[c] = make_uint4(ov[0], ov[1], ov[2], ov[3]);
      }
    }
  }
}

}  // namespace
}  // namespace ma

extern "C" int ma_residual_rmsnorm(const ma_rmsnorm_args* a, void* stream) {
  if (!a || !a->csym || !a->residual_in || !a->weight || !a->residual_out || !a->normed_out ||
      !a->cu_q || !a->fa_b || !a->fa_mb)
    return MA_ERR_INVALID;
  if (a->num_row_tiles < 0 || a->hidden <= 0 || (a->hidden & 7) || a->row_pitch < a->hidden ||
      (a->row_pitch & 7) || !(a->eps >= 0.f))
    return MA_ERR_INVALID;
  if (a->hidden > 4 * 512 * 8) return MA_ERR_CAPACITY;                 // 16384 columns
  const uint64_t ptrs[] = {a->csym, a->residual_in, a->weight, a->residual_out, a->normed_out};
  for (uint64_t p : ptrs)
    if (p & 15u) return MA_ERR_INVALID;                                // 16-byte accesses
  if (a->num_row_tiles == 0) return MA_OK;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return MA_ERR_CUDA;
  const int rows = a->num_row_tiles * 128;
  const int nchunk = a->hidden / 8;
  const int threads = nchunk > 4 * ma::kRnThreads ? 2 * ma::kRnThreads : ma::kRnThreads;
  const int nch = (nchunk + threads - 1) / threads;
  const int per_sm = 1024 / threads;
  const int grid = rows < sms * per_sm ? rows : sms * per_sm;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define MA_RN_LAUNCH(N, T)                                                                       \
  ma::residual_rmsnorm_kernel<N, T><<<grid, T, 0, st>>>(                                        \
      reinterpret_cast<const uint16_t*>(a->csym), reinterpret_cast<const uint16_t*>(a->residual_in), \
      reinterpret_cast<const uint16_t*>(a->weight), reinterpret_cast<uint16_t*>(a->residual_out),   \
      reinterpret_cast<uint16_t*>(a->normed_out), reinterpret_cast<const int*>(a->cu_q),           \
      reinterpret_cast<const int*>(a->fa_b), reinterpret_cast<const int*>(a->fa_mb),               \
      a->num_row_tiles, a->hidden, a->row_pitch, a->eps)
  if (threads == 2 * ma::kRnThreads) MA_RN_LAUNCH(4, 512);
  else if (nch <= 1) MA_RN_LAUNCH(1, 256);
  else if (nch <= 2) MA_RN_LAUNCH(2, 256);
  else MA_RN_LAUNCH(4, 256);
#undef MA_RN_LAUNCH
  return cudaGetLastError() == cudaSuccess ? MA_OK : MA_ERR_CUDA;
}
