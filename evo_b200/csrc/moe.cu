// Expert router of a mixture-of-experts feed-forward: fp32 logits W.h, softmax over all experts, the `top` experts with the largest
// (score + correction) are chosen, and the output weights are the chosen experts' uncorrected scores times a constant (not
// renormalised).  One warp per token; the dense weight row (0 for experts that were not chosen) is what the grouped activation
// kernel multiplies into the expert columns, so that the experts' weighted sum is the K-reduction of one down-projection GEMM.
#include "common.cuh"
#include "../../include/evo_b200.h"
#include <math.h>

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }

constexpr int RW = 4;         // warps (tokens) per CTA
constexpr int EB = 16;        // experts whose partial sums a lane keeps at a time

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  return make_float4(bf_lo(u.x), bf_hi(u.x), bf_lo(u.y), bf_hi(u.y));
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(RW * 32) moe_route_kernel(const T* __restrict__ h, int64_t ldh, const bf16* __restrict__ rw, const bf16* __restrict__ corr,
                                                            float* __restrict__ weights, int32_t* __restrict__ chosen, int64_t rows, int D, int E, int top, float scale) {
  extern __shared__ float sm[];
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * RW + w;
  if (row >= rows) return;
  float* s = sm + (size_t)w * 2 * E;        // scores
  float* c = s + E;                         // choice scores (-inf once taken)
  const T* hr = h + row * ldh;
  // logits: the lanes split the row; EB experts share every load of h (their partial sums stay in registers until the row ends)
  float mx = -INFINITY;
  for (int e0 = 0; e0 < E; e0 += EB) {
    float acc[EB];
#pragma unroll
    for (int j = 0; j < EB; ++j) acc[j] = 0.f;
    if (VEC) {                               // D % 4 == 0, 8-byte (bf16) / 16-byte (fp32) aligned rows
      for (int k = lane * 4; k < D; k += 128) {
        const float4 h4 = ld4(hr + k);
#pragma unroll
        for (int j = 0; j < EB; ++j) {
          if (e0 + j < E) {
            const float4 w4 = ld4(rw + (int64_t)(e0 + j) * D + k);
            acc[j] = fmaf(h4.x, w4.x, fmaf(h4.y, w4.y, fmaf(h4.z, w4.z, fmaf(h4.w, w4.w, acc[j]))));
          }
        }
      }
    } else {
      for (int k = lane; k < D; k += 32) {
        const float hv = ldf(hr + k);
#pragma unroll
        for (int j = 0; j < EB; ++j)
          if (e0 + j < E) acc[j] = fmaf(hv, __bfloat162float(rw[(int64_t)(e0 + j) * D + k]), acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < EB; ++j) {
      float d = acc[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (e0 + j < E) {
        if (lane == 0) s[e0 + j] = d;
        mx = fmaxf(mx, d);
      }
    }
  }
  __syncwarp();
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float v = expf(s[e] - mx); s[e] = v; sum += v; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float* wrow = weights + row * E;
  for (int e = lane; e < E; e += 32) {
    const float v = s[e] * inv;
    s[e] = v;
    c[e] = v + (corr ? __bfloat162float(corr[e]) : 0.f);
    wrow[e] = 0.f;
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY; int bi = E;
    for (int e = lane; e < E; e += 32) if (c[e] > best) { best = c[e]; bi = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0 && bi < E) {
      wrow[bi] = s[bi] * scale;
      c[bi] = -INFINITY;
      if (chosen) chosen[row * top + k] = bi;
    }
    __syncwarp();
  }
}

}  // namespace

extern "C" int evo_moe_route(const void* h, int64_t ldh, const void* router_w, const void* correction, float* weights, int32_t* chosen,
                             int64_t rows, int D, int E, int top, float scale, int dtype, void* stream) {
  EVO_REQUIRE(h && router_w && weights && D > 0 && E > 0 && top > 0 && top <= E && ldh >= D, "evo_moe_route: bad arguments");
  EVO_REQUIRE(E <= 4096, "evo_moe_route: at most 4096 experts");
  if (rows == 0) return 0;
  const size_t smem = sizeof(float) * RW * 2 * (size_t)E;
  dim3 grid((unsigned)((rows + RW - 1) / RW)), block(RW * 32);
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = D % 4 == 0 && ldh % 4 == 0 && ((uintptr_t)h & (dtype ? 15 : 7)) == 0 && ((uintptr_t)router_w & 7) == 0;
  if (dtype) {
    if (vec) moe_route_kernel<float, true><<<grid, block, smem, st>>>((const float*)h, ldh, (const bf16*)router_w, (const bf16*)correction, weights, chosen, rows, D, E, top, scale);
    else moe_route_kernel<float, false><<<grid, block, smem, st>>>((const float*)h, ldh, (const bf16*)router_w, (const bf16*)correction, weights, chosen, rows, D, E, top, scale);
  } else {
    if (vec) moe_route_kernel<bf16, true><<<grid, block, smem, st>>>((const bf16*)h, ldh, (const bf16*)router_w, (const bf16*)correction, weights, chosen, rows, D, E, top, scale);
    else moe_route_kernel<bf16, false><<<grid, block, smem, st>>>((const bf16*)h, ldh, (const bf16*)router_w, (const bf16*)correction, weights, chosen, rows, D, E, top, scale);
  }
  return check_launch("evo_moe_route");
}
