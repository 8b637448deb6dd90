// Latent attention: keys and values of all heads are up-projections of one small latent per token, plus one rotated key part that
// all heads share; only [latent | rotated key part] is cached.
//
//   evo_latent_prep         one CTA per token: turns the rotated part of every query head in place (interleaved pairs, fp32 angles
//                           pos * freq[i]), RMS-norms the latent (fp32) and appends [latent | 0.. | turned key part] to the cache.
//   evo_latent_attn_decode  few query rows (the decoding step, short portions): the absorbed form.  A CTA owns one (query, head):
//                           ql = Uk_h^T q_a, scores straight against the cached latents (one warp per key, lanes across the latent),
//                           chunked streaming softmax, the weighted sum of latents, then o = Uv_h . sum -- the window's keys and
//                           values are never expanded.  Every intermediate is fp32.
// Prompts and long portions expand the visible rows of the cache with one GEMM against [Uk ; Uv] (the rotated part is carried into
// every head's key by identity rows of that weight) and run the windowed attention kernel on the result.
#include "common.cuh"
#include "../../include/evo_b200.h"
#include <math.h>

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// reductions over the block; every thread gets the result (red: 32 floats)
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[w] = v;
  __syncthreads();
  float t = -INFINITY;
  for (int i = 0; i < nw; ++i) t = fmaxf(t, red[i]);
  return t;
}

template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(evo_latent_prep_params p) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x, b = row / p.L, t = row % p.L;
  const int64_t pos = (p.pos_dev ? (int64_t)*p.pos_dev : p.pos0) + t;
  const float fpos = (float)pos;
  const int half = p.rot_dims / 2, hd = p.dim + p.rot;      // entries [rot_dims, rot) of a rotated part pass unchanged
  // queries: pair i of head h
  T* q = (T*)p.q + row * p.ldq;
  for (int idx = threadIdx.x; idx < p.H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half;
    float s, c;
    sincosf(fpos * p.freq[i], &s, &c);
    T* e = q + (int64_t)h * hd + p.dim + 2 * i;
    const float u = ldf(e), v = ldf(e + 1);
    stf(e, u * c - v * s);
    stf(e + 1, v * c + u * s);
  }
  const T* a = (const T*)p.dkv + row * p.ld_dkv;
  T* dst = (T*)p.cache + b * p.cache_batch_stride + pos * p.cache_row;
  float ss = 0.f;
  for (int c = threadIdx.x; c < p.rank; c += blockDim.x) { const float v = ldf(a + c); ss = fmaf(v, v, ss); }
  ss = block_sum(ss, red);
  const float rstd = 1.0f / sqrtf(ss / (float)p.rank + p.eps);
  const bf16* w = (const bf16*)p.norm_w;
  for (int c = threadIdx.x; c < p.rank_pad; c += blockDim.x) stf(dst + c, c < p.rank ? ldf(a + c) * rstd * __bfloat162float(w[c]) : 0.f);
  for (int i = threadIdx.x; i < p.rot / 2; i += blockDim.x) {
    float s = 0.f, c = 1.f;
    if (i < half) sincosf(fpos * p.freq[i], &s, &c);
    const float u = ldf(a + p.rank + 2 * i), v = ldf(a + p.rank + 2 * i + 1);
    stf(dst + p.rank_pad + 2 * i, u * c - v * s);
    stf(dst + p.rank_pad + 2 * i + 1, v * c + u * s);
  }
}

constexpr int DT = 256;       // threads of the decode CTA
constexpr int KC = 512;       // keys per softmax chunk
constexpr int RPT = 4;        // latent entries per thread (rank <= RPT * DT)

template <typename T>
__global__ void __launch_bounds__(DT) latent_decode_kernel(evo_latent_decode_params p, int nr, int ngrp) {
  extern __shared__ float sm[];
  float* qa = sm;                          // [dim]
  float* qr = qa + p.dim;                  // [rot]
  float* ql = qr + p.rot;                  // [rank]
  float* sc = ql + p.rank;                 // [KC]
  float* ol = sc + KC;                     // [ngrp][rank]
  __shared__ float red[32];
  const int rel = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int64_t row = (int64_t)b * p.Lq + rel;
  const int64_t i = (p.pos_dev ? (int64_t)*p.pos_dev : p.pos0) + rel;
  const int64_t lo = p.window > 0 ? max((int64_t)0, i - p.window + 1) : 0;
  const int64_t n = i - lo + 1;
  const int rank = p.rank, hd = p.dim + p.rot;
  const T* q = (const T*)p.q + row * p.ldq + (int64_t)h * hd;
  for (int e = tid; e < hd; e += DT) qa[e] = ldf(q + e);          // qa and qr are adjacent
  __syncthreads();
  const bf16* uk = (const bf16*)p.uk + (int64_t)h * p.dim * rank;
  for (int r = tid; r < rank; r += DT) {
    float acc = 0.f;
    for (int d = 0; d < p.dim; ++d) acc = fmaf(qa[d], __bfloat162float(uk[(int64_t)d * rank + r]), acc);
    ql[r] = acc;
  }
  __syncthreads();
  const T* cb = (const T*)p.cache + (int64_t)b * p.cache_batch_stride;
  const int grp = tid / nr, r0 = tid % nr;                         // threads past ngrp * nr take no part in the value sums
  float acc[RPT];
#pragma unroll
  for (int k = 0; k < RPT; ++k) acc[k] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  for (int64_t k0 = 0; k0 < n; k0 += KC) {
    const int nk = (int)min((int64_t)KC, n - k0);
    for (int jj = w; jj < nk; jj += DT / 32) {
      const T* c = cb + (lo + k0 + jj) * p.cache_row;
      float d = 0.f;
      for (int r = lane; r < rank; r += 32) d = fmaf(ql[r], ldf(c + r), d);
      for (int e = lane; e < p.rot; e += 32) d = fmaf(qr[e], ldf(c + p.rank_pad + e), d);
      d = warp_sum(d);
      if (lane == 0) sc[jj] = d * p.scale;
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int jj = tid; jj < nk; jj += DT) mx = fmaxf(mx, sc[jj]);
    const float m_new = fmaxf(m_run, block_max(mx, red));
    const float corr = expf(m_run - m_new);
    float ps = 0.f;
    for (int jj = tid; jj < nk; jj += DT) { const float e = expf(sc[jj] - m_new); sc[jj] = e; ps += e; }
    l_run = l_run * corr + block_sum(ps, red);                       // the barriers inside also publish sc
    m_run = m_new;
#pragma unroll
    for (int k = 0; k < RPT; ++k) acc[k] *= corr;
    if (grp < ngrp) {
      for (int jj = grp; jj < nk; jj += ngrp) {
        const T* c = cb + (lo + k0 + jj) * p.cache_row;
        const float pj = sc[jj];
#pragma unroll
        for (int k = 0; k < RPT; ++k) {
          const int r = r0 + k * nr;
          if (r < rank) acc[k] = fmaf(pj, ldf(c + r), acc[k]);
        }
      }
    }
    __syncthreads();
  }
  if (grp < ngrp) {
#pragma unroll
    for (int k = 0; k < RPT; ++k) {
      const int r = r0 + k * nr;
      if (r < rank) ol[grp * rank + r] = acc[k];
    }
  }
  __syncthreads();
  const float inv = 1.f / l_run;
  for (int r = tid; r < rank; r += DT) {
    float t = 0.f;
    for (int g = 0; g < ngrp; ++g) t += ol[g * rank + r];
    ql[r] = t * inv;                                                 // ql is free now: the normalised sum of latents
  }
  __syncthreads();
  float gate = 1.f;
  if (p.gate) gate = 1.f / (1.f + expf(-ldf((const T*)p.gate + row * p.ld_gate + h)));
  const bf16* uv = (const bf16*)p.uv + (int64_t)h * p.vdim * rank;
  T* orow = (T*)p.out + row * p.ldo;
  for (int v = w; v < p.vdim; v += DT / 32) {
    float d = 0.f;
    for (int r = lane; r < rank; r += 32) d = fmaf(__bfloat162float(uv[(int64_t)v * rank + r]), ql[r], d);
    d = warp_sum(d);
    if (lane == 0) stf(orow + (int64_t)h * p.vdim + v, d * gate);
  }
  if (h == p.H - 1)
    for (int64_t c = (int64_t)p.H * p.vdim + tid; c < p.ldo; c += DT) stf(orow + c, 0.f);
}

}  // namespace

extern "C" int evo_latent_prep(const evo_latent_prep_params* p, void* stream) {
  EVO_REQUIRE(p->q && p->dkv && p->norm_w && p->freq && p->cache, "evo_latent_prep: null argument");
  EVO_REQUIRE(p->H > 0 && p->dim >= 0 && p->rot >= 0 && p->rot % 2 == 0 && p->rot_dims % 2 == 0 && p->rot_dims >= 0 && p->rot_dims <= p->rot && p->rank > 0 && p->rank_pad >= p->rank, "evo_latent_prep: bad shape");
  EVO_REQUIRE(p->ldq >= (int64_t)p->H * (p->dim + p->rot) && p->ld_dkv >= p->rank + p->rot && p->cache_row >= p->rank_pad + p->rot, "evo_latent_prep: bad strides");
  if ((int64_t)p->B * p->L == 0) return 0;
  dim3 grid((unsigned)((int64_t)p->B * p->L)), block(128);
  if (p->dtype) latent_prep_kernel<float><<<grid, block, 0, (cudaStream_t)stream>>>(*p);
  else latent_prep_kernel<bf16><<<grid, block, 0, (cudaStream_t)stream>>>(*p);
  return check_launch("evo_latent_prep");
}

extern "C" int evo_latent_attn_decode(const evo_latent_decode_params* p, void* stream) {
  EVO_REQUIRE(p->q && p->cache && p->uk && p->uv && p->out, "evo_latent_attn_decode: null argument");
  EVO_REQUIRE(p->H > 0 && p->dim > 0 && p->rot >= 0 && p->rank > 0 && p->vdim > 0 && p->rank_pad >= p->rank, "evo_latent_attn_decode: bad shape");
  EVO_REQUIRE(p->rank <= RPT * DT, "evo_latent_attn_decode: latent size (%d) must be <= %d", p->rank, RPT * DT);
  EVO_REQUIRE(p->ldo >= (int64_t)p->H * p->vdim && p->H <= 65535 && p->B <= 65535, "evo_latent_attn_decode: bad output stride or grid");
  if ((int64_t)p->B * p->Lq == 0) return 0;
  const int nr = p->rank >= DT ? DT : (p->rank + 31) / 32 * 32;
  const int ngrp = DT / nr;
  const size_t smem = sizeof(float) * ((size_t)p->dim + p->rot + p->rank + KC + (size_t)ngrp * p->rank);
  EVO_REQUIRE(smem <= 200 * 1024, "evo_latent_attn_decode: head too large for shared memory (%zu bytes)", smem);
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid((unsigned)p->Lq, (unsigned)p->H, (unsigned)p->B);
  if (p->dtype) {
    if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(latent_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    latent_decode_kernel<float><<<grid, DT, smem, st>>>(*p, nr, ngrp);
  } else {
    if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(latent_decode_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    latent_decode_kernel<bf16><<<grid, DT, smem, st>>>(*p, nr, ngrp);
  }
  return check_launch("evo_latent_attn_decode");
}
