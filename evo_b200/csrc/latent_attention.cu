// Latent attention: keys and values of all heads are up-projections of one small latent per token, plus one rotated key part that
// all heads share; only [latent | rotated key part] is cached.
//
//   evo_latent_prep         one CTA per token: turns the rotated part of every query head in place (interleaved pairs, fp32 angles
//                           pos * freq[i]), RMS-norms the latent (fp32) and appends [latent | 0.. | turned key part] to the cache.
//   evo_latent_attn_decode  few query rows (the decoding step, short portions): the absorbed form, ql = Uk_h^T q_a, scores straight
//                           against the cached latents, streaming softmax, the weighted sum of latents, then o = Uv_h . sum -- the
//                           window's keys and values are never expanded, and every intermediate is fp32.  Four launches: absorb
//                           (Uk read once), a (key split, row, head group) kernel in which 8 or 16 heads share each tile of latents
//                           through shared memory, a merge of the splits, and the Uv product with the head gate (Uv read once).  Shapes that path does not
//                           cover run one CTA per (query, head) (latent_decode_kernel).
// Prompts and long portions expand the visible rows of the cache with one GEMM against [Uk ; Uv] (the rotated part is carried into
// every head's key by identity rows of that weight) and run the windowed attention kernel on the result.
#include "common.cuh"
#include "mma_sync.cuh"
#include "../../include/evo_b200.h"
#include <math.h>
#include <stdlib.h>
#include <algorithm>

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

// ---- few query rows, all heads of a group share every latent they read ------------------------------------------------------------
// (1) absorb: ql[row, h] = [Uk_h^T q_a | q_b]  (fp32, rank + rot entries).  grid (H, rank / 32); a CTA's 4 warps split the query
// dimension, lanes are 32 adjacent latent entries (coalesced weight rows); the weights are read once per 8 rows.
constexpr int AR = 8;         // rows per pass of the absorb kernel
// bf16 high part and bf16 remainder of v at entry e of a [2][kw] row (the tensor-core step kernel reads both with 16-byte copies)
__device__ __forceinline__ void put_split(bf16* row, int kw, int e, float v) {
  const bf16 hi = __float2bfloat16_rn(v);
  row[e] = hi;
  row[kw + e] = __float2bfloat16_rn(v - __bfloat162float(hi));
}
template <typename T>
__global__ void __launch_bounds__(128) latent_absorb_kernel(evo_latent_decode_params p, float* __restrict__ ql, bf16* __restrict__ qsplit) {
  extern __shared__ float qs[];             // [AR][dim], then [4][AR][32] partial sums
  float* ps = qs + AR * p.dim;
  const int h = blockIdx.x, lane = threadIdx.x & 31, dg = threadIdx.x >> 5, r = blockIdx.y * 32 + lane;
  const int hd = p.dim + p.rot, kw = p.rank + p.rot;
  const int64_t R = (int64_t)p.B * p.Lq;
  const bf16* uk = (const bf16*)p.uk + (int64_t)h * p.dim * p.rank;
  const int d_per = (p.dim + 3) / 4, d0 = dg * d_per, d1 = min(p.dim, d0 + d_per);
  for (int64_t row0 = 0; row0 < R; row0 += AR) {
    const int nr = (int)min((int64_t)AR, R - row0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < nr * p.dim; idx += 128) {
      const int i = idx / p.dim, d = idx % p.dim;
      qs[i * p.dim + d] = ldf((const T*)p.q + (row0 + i) * p.ldq + (int64_t)h * hd + d);
    }
    if (blockIdx.y == 0)
      for (int idx = threadIdx.x; idx < nr * p.rot; idx += 128) {
        const int i = idx / p.rot, e = idx % p.rot;
        const float v = ldf((const T*)p.q + (row0 + i) * p.ldq + (int64_t)h * hd + p.dim + e);
        ql[((row0 + i) * p.H + h) * kw + p.rank + e] = v;
        if (qsplit) put_split(qsplit + ((row0 + i) * p.H + h) * 2 * kw, kw, p.rank + e, v);
      }
    __syncthreads();
    float acc[AR];
#pragma unroll
    for (int i = 0; i < AR; ++i) acc[i] = 0.f;
    if (r < p.rank) {
#pragma unroll 4
      for (int d = d0; d < d1; ++d) {
        const float w = __bfloat162float(uk[(int64_t)d * p.rank + r]);
#pragma unroll
        for (int i = 0; i < AR; ++i) acc[i] = fmaf(qs[(i < nr ? i : 0) * p.dim + d], w, acc[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < AR; ++i) ps[(dg * AR + i) * 32 + lane] = acc[i];
    __syncthreads();
    for (int idx = threadIdx.x; idx < nr * 32; idx += 128) {
      const int i = idx >> 5, l = idx & 31;
      if (blockIdx.y * 32 + l < p.rank) {
        const float v = ps[i * 32 + l] + ps[(AR + i) * 32 + l] + ps[(2 * AR + i) * 32 + l] + ps[(3 * AR + i) * 32 + l];
        ql[((row0 + i) * p.H + h) * kw + blockIdx.y * 32 + l] = v;
        if (qsplit) put_split(qsplit + ((row0 + i) * p.H + h) * 2 * kw, kw, blockIdx.y * 32 + l, v);
      }
    }
  }
}

// (2) scores and value sums of one (key split, row, head group): tiles of KT = 256 / HG latents go through shared memory once for all HG heads.
// Rows in shared memory are [latent, padded to 4 | rotated part, padded to 4] with a row stride of 4 mod 32 floats, so that the 16-byte
// reads of both phases are conflict-free: thread (head, key) scores its key with float4 dot products; thread (head, kk) accumulates the
// latent entries 4 (kk + KT k) .. + 3.  One partial (max, sum, acc) per split.
constexpr int SPLIT_T = 256;
constexpr int RMAX = 32;      // latent entries per thread
struct SplitLayout { int rp4, kwp, tw; };
__host__ __device__ inline SplitLayout split_layout(int rank, int rot) {
  SplitLayout l;
  l.rp4 = (rank + 3) / 4 * 4;
  l.kwp = l.rp4 + (rot + 3) / 4 * 4;
  l.tw = l.kwp + (36 - l.kwp % 32) % 32;
  return l;
}
template <typename T, int HG>
__global__ void __launch_bounds__(SPLIT_T) latent_split_kernel(evo_latent_decode_params p, const float* __restrict__ ql, float* __restrict__ part, int n_split, int pairs) {
  constexpr int KT = SPLIT_T / HG;          // keys per tile = threads per head (16 or 32: a head's threads sit in one warp)
  extern __shared__ __align__(16) float sm[];
  const SplitLayout lay = split_layout(p.rank, p.rot);
  const int kw = p.rank + p.rot, kwp = lay.kwp, tw = lay.tw, rp4 = lay.rp4;
  float* qs = sm;                           // [HG][kwp]
  float* tile = qs + HG * kwp;              // [KT][tw]
  float* pb = tile + KT * tw;               // [HG][KT]
  const int split = blockIdx.x, hg = blockIdx.z;
  const int64_t row = blockIdx.y, b = row / p.Lq, rel = row % p.Lq;
  const int tid = threadIdx.x, hl = tid / KT, kk = tid % KT, w = tid >> 5, lane = tid & 31;
  const int h = hg * HG + hl;
  const int64_t i = (p.pos_dev ? (int64_t)*p.pos_dev : p.pos0) + rel;
  const int64_t lo = p.window > 0 ? max((int64_t)0, i - p.window + 1) : 0;
  const int64_t n = i - lo + 1;
  const int64_t tiles = (n + KT - 1) / KT, per = (tiles + n_split - 1) / n_split;
  const int64_t t_begin = split * per, t_end = min(tiles, t_begin + per);
  for (int idx = tid; idx < HG * kwp + KT * tw; idx += SPLIT_T) sm[idx] = 0.f;       // pads stay zero
  __syncthreads();
  for (int idx = tid; idx < HG * kw; idx += SPLIT_T) {
    const int hh = idx / kw, e = idx % kw;
    if (hg * HG + hh < p.H) qs[hh * kwp + (e < p.rank ? e : rp4 + e - p.rank)] = ql[(row * p.H + hg * HG + hh) * kw + e];
  }
  const T* cb = (const T*)p.cache + b * p.cache_batch_stride;
  float acc[RMAX / 4][4];
#pragma unroll
  for (int k = 0; k < RMAX / 4; ++k) acc[k][0] = acc[k][1] = acc[k][2] = acc[k][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  for (int64_t t = t_begin; t < t_end; ++t) {
    const int64_t k0 = lo + t * KT;
    const int nk = (int)min((int64_t)KT, i + 1 - k0);
    __syncthreads();
    for (int key = w; key < nk; key += SPLIT_T / 32) {
      const T* c = cb + (k0 + key) * p.cache_row;
      float* dst = tile + key * tw;
      if (pairs) {                          // even sizes and strides: two entries per load
        for (int e = lane * 2; e < p.rank; e += 64) {
          if (sizeof(T) == 2) { const uint32_t u = *reinterpret_cast<const uint32_t*>(c + e); dst[e] = bf_lo(u); dst[e + 1] = bf_hi(u); }
          else { const float2 u = *reinterpret_cast<const float2*>(c + e); dst[e] = u.x; dst[e + 1] = u.y; }
        }
        for (int e = lane * 2; e < p.rot; e += 64) {
          if (sizeof(T) == 2) { const uint32_t u = *reinterpret_cast<const uint32_t*>(c + p.rank_pad + e); dst[rp4 + e] = bf_lo(u); dst[rp4 + e + 1] = bf_hi(u); }
          else { const float2 u = *reinterpret_cast<const float2*>(c + p.rank_pad + e); dst[rp4 + e] = u.x; dst[rp4 + e + 1] = u.y; }
        }
      } else {
        for (int e = lane; e < p.rank; e += 32) dst[e] = ldf(c + e);
        for (int e = lane; e < p.rot; e += 32) dst[rp4 + e] = ldf(c + p.rank_pad + e);
      }
    }
    __syncthreads();
    float sc = -INFINITY;
    if (kk < nk) {
      float d = 0.f;
      const float4* qv = reinterpret_cast<const float4*>(qs + hl * kwp);
      const float4* cv = reinterpret_cast<const float4*>(tile + kk * tw);
#pragma unroll 4
      for (int e = 0; e < kwp / 4; ++e) {
        const float4 a = qv[e], c4 = cv[e];
        d = fmaf(a.x, c4.x, fmaf(a.y, c4.y, fmaf(a.z, c4.z, fmaf(a.w, c4.w, d))));
      }
      sc = d * p.scale;
    }
    float mx = sc;
#pragma unroll
    for (int o = KT / 2; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float m_new = fmaxf(m_run, mx);               // finite: every tile of the range has a visible key
    const float corr = expf(m_run - m_new);
    const float pj = kk < nk ? expf(sc - m_new) : 0.f;
    float ps = pj;
#pragma unroll
    for (int o = KT / 2; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l_run = l_run * corr + ps;
    m_run = m_new;
    pb[hl * KT + kk] = pj;
    __syncwarp();                                       // a head's KT probabilities are written and read by lanes of one warp
#pragma unroll
    for (int k = 0; k < RMAX / 4; ++k) { acc[k][0] *= corr; acc[k][1] *= corr; acc[k][2] *= corr; acc[k][3] *= corr; }
    for (int key = 0; key < nk; ++key) {
      const float pk = pb[hl * KT + key];
      const float4* cv = reinterpret_cast<const float4*>(tile + key * tw) + kk;
#pragma unroll
      for (int k = 0; k < RMAX / 4; ++k) {
        if ((kk + k * KT) * 4 < rp4) {
          const float4 c4 = cv[k * KT];
          acc[k][0] = fmaf(pk, c4.x, acc[k][0]); acc[k][1] = fmaf(pk, c4.y, acc[k][1]);
          acc[k][2] = fmaf(pk, c4.z, acc[k][2]); acc[k][3] = fmaf(pk, c4.w, acc[k][3]);
        }
      }
    }
  }
  if (h >= p.H) return;
  float* dst = part + (((int64_t)split * gridDim.y + row) * p.H + h) * (p.rank + 2);
  if (kk == 0) { dst[0] = m_run; dst[1] = l_run; }
#pragma unroll
  for (int k = 0; k < RMAX / 4; ++k)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = (kk + k * KT) * 4 + j;
      if (r < p.rank) dst[2 + r] = acc[k][j];
    }
}

// (2b) the same partial on the tensor cores, for bf16 caches, groups of 16 heads and latents of 64 / 128 / 256 / 512 entries: the 16 heads are
// the M dimension of mma.sync.m16n8k16.  q_l enters as a bf16 high part plus a bf16 remainder (two MMAs; products with the bf16 latents are
// exact, sums fp32), the scores of a 64-key tile go through shared memory in fp32, every warp rebuilds the tile's softmax weights in
// fragment layout (fp32), and the weights enter the value sum as high + remainder against the SAME tile (read transposed by ldmatrix).
// The four warps split the keys for the scores and the latent columns for the values.  NV8 = rank / 32 (8-column tiles per warp).
constexpr int MK = 64;        // keys per tile
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, int src_bytes) {      // src_bytes 0: zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(smem_u32(smem_dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}
template <int NV8>
__global__ void __launch_bounds__(128) latent_split_mma_kernel(evo_latent_decode_params p, const bf16* __restrict__ qsplit, float* __restrict__ part, int n_split) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int kw = p.rank + p.rot, st = kw + 8;             // row stride in bf16: 16 bytes of padding, conflict-free fragment reads
  bf16* Qh = reinterpret_cast<bf16*>(smraw);              // [16][st] high parts of [q_l | q_b]
  bf16* Ql = Qh + 16 * st;                                // [16][st] remainders
  bf16* Ks = Ql + 16 * st;                                // [MK][st] latents and rotated key parts of the tile
  float* Ss = reinterpret_cast<float*>(Ks + MK * st);     // [16][MK + 2] scores (base-2 exponent units)
  constexpr int sst = MK + 2;
  const int split = blockIdx.x, hg = blockIdx.z;
  const int64_t row = blockIdx.y, b = row / p.Lq, rel = row % p.Lq;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, qr = lane >> 2, qc = (lane & 3) * 2;
  const int64_t i = (p.pos_dev ? (int64_t)*p.pos_dev : p.pos0) + rel;
  const int64_t lo = p.window > 0 ? max((int64_t)0, i - p.window + 1) : 0;
  const int64_t n = i - lo + 1;
  const int64_t tiles = (n + MK - 1) / MK, per = (tiles + n_split - 1) / n_split;
  const int64_t t_begin = split * per, t_end = min(tiles, t_begin + per);
  const int c16 = kw / 8;                                        // 16-byte chunks per row
  // both query parts of the 16 heads: asynchronous 16-byte copies (zero-filled past the last head), in flight together with the first tile
  for (int rr = w; rr < 32; rr += 4) {
    const int hh = rr & 15, part_ = rr >> 4, h = hg * 16 + hh;
    const bf16* src = qsplit + ((row * p.H + (h < p.H ? h : 0)) * 2 + part_) * kw;
    bf16* dst = (part_ ? Ql : Qh) + hh * st;
    for (int c = lane; c < c16; c += 32) cp_async16(dst + c * 8, src + c * 8, h < p.H ? 16 : 0);
  }
  const bf16* cb = (const bf16*)p.cache + b * p.cache_batch_stride;
  float O[NV8][4];
#pragma unroll
  for (int nn = 0; nn < NV8; ++nn) O[nn][0] = O[nn][1] = O[nn][2] = O[nn][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows qr and qr + 8 (the same in every warp)
  const float scale2 = p.scale * 1.4426950408889634f;
  for (int64_t t = t_begin; t < t_end; ++t) {
    const int64_t k0 = lo + t * MK;
    const int nk = (int)min((int64_t)MK, i + 1 - k0);
    __syncthreads();
    for (int r = w; r < MK; r += 4) {                       // a warp per key row, 16 bytes per lane, zero-filled past the last key
      const bf16* src = cb + (k0 + (r < nk ? r : 0)) * p.cache_row;
      for (int c = lane; c < c16; c += 32) cp_async16(Ks + r * st + c * 8, src + c * 8, r < nk ? 16 : 0);
    }
    cp_async_wait_all();
    __syncthreads();
    // scores of keys [16 w, 16 w + 16): S = (Qh + Ql) . K^T
    float S[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) S[u][0] = S[u][1] = S[u][2] = S[u][3] = 0.f;
    for (int ks = 0; ks < kw / 16; ++ks) {
      uint32_t ah[4], al[4], kf[4];
      const bf16* qa = Qh + ks * 16 + qc;
      ah[0] = *reinterpret_cast<const uint32_t*>(qa + qr * st);
      ah[1] = *reinterpret_cast<const uint32_t*>(qa + (qr + 8) * st);
      ah[2] = *reinterpret_cast<const uint32_t*>(qa + qr * st + 8);
      ah[3] = *reinterpret_cast<const uint32_t*>(qa + (qr + 8) * st + 8);
      const bf16* qb = Ql + ks * 16 + qc;
      al[0] = *reinterpret_cast<const uint32_t*>(qb + qr * st);
      al[1] = *reinterpret_cast<const uint32_t*>(qb + (qr + 8) * st);
      al[2] = *reinterpret_cast<const uint32_t*>(qb + qr * st + 8);
      al[3] = *reinterpret_cast<const uint32_t*>(qb + (qr + 8) * st + 8);
      ldmatrix_x4(kf, Ks + ((2 * w + (lane >> 4)) * 8 + (lane & 7)) * st + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(S[0], ah, kf[0], kf[1]); mma_bf16(S[0], al, kf[0], kf[1]);
      mma_bf16(S[1], ah, kf[2], kf[3]); mma_bf16(S[1], al, kf[2], kf[3]);
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int col = (2 * w + u) * 8 + qc;
      Ss[qr * sst + col] = col < nk ? S[u][0] * scale2 : -INFINITY;
      Ss[qr * sst + col + 1] = col + 1 < nk ? S[u][1] * scale2 : -INFINITY;
      Ss[(qr + 8) * sst + col] = col < nk ? S[u][2] * scale2 : -INFINITY;
      Ss[(qr + 8) * sst + col + 1] = col + 1 < nk ? S[u][3] * scale2 : -INFINITY;
    }
    __syncthreads();
    // the tile's weights in A-fragment layout: P[kk] = rows (qr, qr + 8) x keys 16 kk + qc + {0, 1, 8, 9}
    float P[MK / 16][8];
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int kk = 0; kk < MK / 16; ++kk) {
      const float2 a0 = *reinterpret_cast<const float2*>(Ss + qr * sst + kk * 16 + qc), a1 = *reinterpret_cast<const float2*>(Ss + qr * sst + kk * 16 + 8 + qc);
      const float2 b0 = *reinterpret_cast<const float2*>(Ss + (qr + 8) * sst + kk * 16 + qc), b1 = *reinterpret_cast<const float2*>(Ss + (qr + 8) * sst + kk * 16 + 8 + qc);
      P[kk][0] = a0.x; P[kk][1] = a0.y; P[kk][2] = b0.x; P[kk][3] = b0.y; P[kk][4] = a1.x; P[kk][5] = a1.y; P[kk][6] = b1.x; P[kk][7] = b1.y;
      mx0 = fmaxf(mx0, fmaxf(fmaxf(a0.x, a0.y), fmaxf(a1.x, a1.y)));
      mx1 = fmaxf(mx1, fmaxf(fmaxf(b0.x, b0.y), fmaxf(b1.x, b1.y)));
    }
    mx0 = quad_max(mx0); mx1 = quad_max(mx1);
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);          // finite: every tile of the range has a visible key
    const float c0 = ex2(m0 - n0), c1 = ex2(m1 - n1);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int kk = 0; kk < MK / 16; ++kk) {
      P[kk][0] = ex2(P[kk][0] - n0); P[kk][1] = ex2(P[kk][1] - n0); P[kk][4] = ex2(P[kk][4] - n0); P[kk][5] = ex2(P[kk][5] - n0);
      P[kk][2] = ex2(P[kk][2] - n1); P[kk][3] = ex2(P[kk][3] - n1); P[kk][6] = ex2(P[kk][6] - n1); P[kk][7] = ex2(P[kk][7] - n1);
      s0 += P[kk][0] + P[kk][1] + P[kk][4] + P[kk][5];
      s1 += P[kk][2] + P[kk][3] + P[kk][6] + P[kk][7];
    }
    l0 = l0 * c0 + quad_sum(s0); l1 = l1 * c1 + quad_sum(s1);
    m0 = n0; m1 = n1;
#pragma unroll
    for (int nn = 0; nn < NV8; ++nn) { O[nn][0] *= c0; O[nn][1] *= c0; O[nn][2] *= c1; O[nn][3] *= c1; }
    // O[:, columns of this warp] += P . C
#pragma unroll
    for (int kk = 0; kk < MK / 16; ++kk) {
      uint32_t ah[4], al[4];
      split_pack(P[kk][0], P[kk][1], ah[0], al[0]);
      split_pack(P[kk][2], P[kk][3], ah[1], al[1]);
      split_pack(P[kk][4], P[kk][5], ah[2], al[2]);
      split_pack(P[kk][6], P[kk][7], ah[3], al[3]);
#pragma unroll
      for (int nn = 0; nn < NV8; nn += 2) {
        uint32_t bv[4];
        ldmatrix_x4_trans(bv, Ks + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * st + (w * NV8 + nn + (lane >> 4)) * 8);
        mma_bf16(O[nn], ah, bv[0], bv[1]); mma_bf16(O[nn], al, bv[0], bv[1]);
        mma_bf16(O[nn + 1], ah, bv[2], bv[3]); mma_bf16(O[nn + 1], al, bv[2], bv[3]);
      }
    }
  }
  cp_async_wait_all();                                           // a split without tiles still has its query copies in flight
  // partials in natural-exponent units, as the merge kernel expects
  const float ln2 = 0.6931471805599453f;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int h = hg * 16 + qr + 8 * half;
    if (h >= p.H) continue;
    float* dst = part + (((int64_t)split * gridDim.y + row) * p.H + h) * (p.rank + 2);
    if (w == 0 && qc == 0) { dst[0] = (half ? m1 : m0) * ln2; dst[1] = half ? l1 : l0; }
#pragma unroll
    for (int nn = 0; nn < NV8; ++nn) {
      const int r = (w * NV8 + nn) * 8 + qc;
      dst[2 + r] = O[nn][2 * half]; dst[2 + r + 1] = O[nn][2 * half + 1];
    }
  }
}

// (3) merge of the splits: ol[row, h, :] = sum / l   (one CTA per (row, head); ol has the row stride of ql)
__global__ void __launch_bounds__(128) latent_merge_kernel(evo_latent_decode_params p, const float* __restrict__ part, int n_split, float* __restrict__ ol) {
  const int64_t row = blockIdx.x;
  const int h = blockIdx.y, tid = threadIdx.x;
  const int64_t R = gridDim.x, stride = (int64_t)p.rank + 2;
  float mx = -INFINITY;
  for (int s = 0; s < n_split; ++s) mx = fmaxf(mx, part[(((int64_t)s * R + row) * p.H + h) * stride]);
  float l = 0.f;
  for (int s = 0; s < n_split; ++s) {
    const float* src = part + (((int64_t)s * R + row) * p.H + h) * stride;
    if (src[0] != -INFINITY) l = fmaf(src[1], expf(src[0] - mx), l);
  }
  const float inv = 1.f / l;
  float* dst = ol + (row * p.H + h) * (p.rank + p.rot);
  for (int r = tid; r < p.rank; r += 128) {
    float t = 0.f;
    for (int s = 0; s < n_split; ++s) {
      const float* src = part + (((int64_t)s * R + row) * p.H + h) * stride;
      if (src[0] != -INFINITY) t = fmaf(src[2 + r], expf(src[0] - mx), t);
    }
    dst[r] = t * inv;
  }
}

// (4) o = Uv_h . ol, head gate, store: grid (H, vdim / 8), one value row of Uv per warp, read once for up to 16 query rows
constexpr int UR = 16;        // query rows per pass
template <typename T>
__global__ void __launch_bounds__(256) latent_uv_kernel(evo_latent_decode_params p, const float* __restrict__ ol) {
  extern __shared__ float os[];             // [UR][rank]
  const int h = blockIdx.x, tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  const int kw = p.rank + p.rot;
  const int64_t R = (int64_t)p.B * p.Lq;
  const bf16* uv = (const bf16*)p.uv + (int64_t)h * p.vdim * p.rank;
  for (int64_t row0 = 0; row0 < R; row0 += UR) {
    const int nr = (int)min((int64_t)UR, R - row0);
    __syncthreads();
    for (int idx = tid; idx < nr * p.rank; idx += 256) {
      const int i = idx / p.rank, r = idx % p.rank;
      os[i * p.rank + r] = ol[((row0 + i) * p.H + h) * kw + r];
    }
    __syncthreads();
    for (int v = blockIdx.y * 8 + w; v < min(p.vdim, (int)(blockIdx.y + 1) * 8); v += 8) {
      float d[UR];
#pragma unroll
      for (int i = 0; i < UR; ++i) d[i] = 0.f;
      for (int r = lane; r < p.rank; r += 32) {
        const float wv = __bfloat162float(uv[(int64_t)v * p.rank + r]);
#pragma unroll
        for (int i = 0; i < UR; ++i) d[i] = fmaf(wv, os[(i < nr ? i : 0) * p.rank + r], d[i]);
      }
#pragma unroll
      for (int i = 0; i < UR; ++i) d[i] = warp_sum(d[i]);
      if (lane == 0)
        for (int i = 0; i < nr; ++i) {
          const int64_t row = row0 + i;
          float gate = 1.f;
          if (p.gate) gate = 1.f / (1.f + expf(-ldf((const T*)p.gate + row * p.ld_gate + h)));
          stf((T*)p.out + row * p.ldo + (int64_t)h * p.vdim + v, d[i] * gate);
        }
    }
    if (h == p.H - 1 && blockIdx.y == 0)
      for (int i = 0; i < nr; ++i)
        for (int64_t c = (int64_t)p.H * p.vdim + tid; c < p.ldo; c += 256) stf((T*)p.out + (row0 + i) * p.ldo + c, 0.f);
  }
}

// plan of the shared-heads path: heads per group (0: not covered, the per-head kernel runs) and the number of key splits
struct SplitPlan { int hg, n_split, mma; size_t smem, ws; };
inline SplitPlan split_plan(const evo_latent_decode_params* p) {
  SplitPlan pl = {0, 1, 0, 0, 0};
  if (p->H >= 12 && p->rank <= 16 * RMAX) pl.hg = 16;
  else if (p->rank <= 32 * RMAX) pl.hg = 8;
  else return pl;
  int kt = SPLIT_T / pl.hg;
  const int kw = p->rank + p->rot;
  const SplitLayout lay = split_layout(p->rank, p->rot);
  pl.smem = sizeof(float) * ((size_t)pl.hg * lay.kwp + (size_t)kt * lay.tw + SPLIT_T);
  // tensor-core form: bf16 cache rows that are [latent | rotated part] without padding in between, 16-byte chunks
  const size_t smem_mma = sizeof(bf16) * (size_t)(32 + MK) * (kw + 8) + sizeof(float) * 16 * (MK + 2);
  if (p->dtype == 0 && pl.hg == 16 && (p->rank == 64 || p->rank == 128 || p->rank == 256 || p->rank == 512) && p->rot % 16 == 0 && p->rank_pad == p->rank &&
      p->cache_row % 8 == 0 && p->cache_batch_stride % 8 == 0 && ((uintptr_t)p->cache & 15) == 0 && smem_mma <= 200 * 1024) {
    pl.mma = 1; pl.smem = smem_mma; kt = MK;
  }
  if (pl.smem > 200 * 1024) { pl.hg = 0; return pl; }
  const int64_t R = (int64_t)p->B * p->Lq, groups = (p->H + pl.hg - 1) / pl.hg;
  const int64_t keys = p->max_keys > 0 ? (p->window > 0 ? std::min<int64_t>(p->window, p->max_keys) : p->max_keys) : (p->window > 0 ? p->window : 1024);
  const int64_t tiles = (keys + kt - 1) / kt;
  int64_t s = ((pl.mma ? 1 : 3) * 148 + R * groups - 1) / (R * groups);          // CTAs that fit the GPU at once (shared memory)
  s = std::max<int64_t>(1, std::min<int64_t>(s, pl.mma ? tiles : (tiles + 1) / 2));
  pl.n_split = (int)std::min<int64_t>(s, 64);
  pl.ws = sizeof(float) * (((size_t)R * p->H * kw + (size_t)pl.n_split * R * p->H * (p->rank + 2) + 3) / 4 * 4);
  if (pl.mma) pl.ws += sizeof(bf16) * 2 * (size_t)R * p->H * kw;          // the absorbed queries as bf16 high parts and remainders
  return pl;
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

extern "C" size_t evo_latent_attn_decode_workspace(const evo_latent_decode_params* p) {
  return split_plan(p).ws;
}

extern "C" int evo_latent_attn_decode(const evo_latent_decode_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  EVO_REQUIRE(p->q && p->cache && p->uk && p->uv && p->out, "evo_latent_attn_decode: null argument");
  EVO_REQUIRE(p->H > 0 && p->dim > 0 && p->rot >= 0 && p->rank > 0 && p->vdim > 0 && p->rank_pad >= p->rank, "evo_latent_attn_decode: bad shape");
  EVO_REQUIRE(p->ldo >= (int64_t)p->H * p->vdim && p->H <= 65535 && p->B <= 65535, "evo_latent_attn_decode: bad output stride or grid");
  if ((int64_t)p->B * p->Lq == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const SplitPlan pl = split_plan(p);
  if (pl.hg && workspace && workspace_bytes >= pl.ws) {
    const int64_t R = (int64_t)p->B * p->Lq;
    EVO_REQUIRE(R <= 65535, "evo_latent_attn_decode: too many query rows");
    const int kw = p->rank + p->rot;
    float* ql = (float*)workspace;
    float* part = ql + (size_t)R * p->H * kw;
    const size_t sm_a = sizeof(float) * ((size_t)AR * p->dim + 4 * AR * 32);
    dim3 ga((unsigned)p->H, (unsigned)((p->rank + 31) / 32));
    dim3 gs((unsigned)pl.n_split, (unsigned)R, (unsigned)((p->H + pl.hg - 1) / pl.hg));
    dim3 gm((unsigned)R, (unsigned)p->H);
    dim3 gu((unsigned)p->H, (unsigned)((p->vdim + 7) / 8));
    const size_t sm_u = sizeof(float) * UR * p->rank;
    EVO_REQUIRE(sm_u <= 200 * 1024, "evo_latent_attn_decode: latent too large");
    const int esz = p->dtype ? 4 : 2;
    const int pairs = p->rank % 2 == 0 && p->rot % 2 == 0 && p->rank_pad % 2 == 0 && p->cache_row % 2 == 0 && p->cache_batch_stride % 2 == 0 &&
                      ((uintptr_t)p->cache & (uintptr_t)(2 * esz - 1)) == 0;
#define EVO_LATENT_SPLIT(T)                                                                                                          \
    latent_absorb_kernel<T><<<ga, 128, sm_a, st>>>(*p, ql, nullptr);                                                                 \
    if (pl.hg == 16) {                                                                                                               \
      if (pl.smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(latent_split_kernel<T, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem)); \
      latent_split_kernel<T, 16><<<gs, SPLIT_T, pl.smem, st>>>(*p, ql, part, pl.n_split, pairs);                                    \
    } else {                                                                                                                         \
      if (pl.smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(latent_split_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));  \
      latent_split_kernel<T, 8><<<gs, SPLIT_T, pl.smem, st>>>(*p, ql, part, pl.n_split, pairs);                                     \
    }                                                                                                                                \
    latent_merge_kernel<<<gm, 128, 0, st>>>(*p, part, pl.n_split, ql);                                                               \
    if (sm_u > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(latent_uv_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_u));                \
    latent_uv_kernel<T><<<gu, 256, sm_u, st>>>(*p, ql);
#define EVO_LATENT_MMA(NV8)                                                                                                          \
    { if (pl.smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(latent_split_mma_kernel<NV8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem)); \
      latent_split_mma_kernel<NV8><<<gs, 128, pl.smem, st>>>(*p, qsplit, part, pl.n_split); }
    if (pl.mma) {
      bf16* qsplit = (bf16*)(ql + ((size_t)R * p->H * kw + (size_t)pl.n_split * R * p->H * (p->rank + 2) + 3) / 4 * 4);
      latent_absorb_kernel<bf16><<<ga, 128, sm_a, st>>>(*p, ql, qsplit);
      switch (p->rank) {
        case 64: EVO_LATENT_MMA(2) break;
        case 128: EVO_LATENT_MMA(4) break;
        case 256: EVO_LATENT_MMA(8) break;
        default: EVO_LATENT_MMA(16) break;
      }
      latent_merge_kernel<<<gm, 128, 0, st>>>(*p, part, pl.n_split, ql);
      if (sm_u > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(latent_uv_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_u));
      latent_uv_kernel<bf16><<<gu, 256, sm_u, st>>>(*p, ql);
    } else if (p->dtype) { EVO_LATENT_SPLIT(float) } else { EVO_LATENT_SPLIT(bf16) }
#undef EVO_LATENT_MMA
#undef EVO_LATENT_SPLIT
    return check_launch("evo_latent_attn_decode");
  }
  EVO_REQUIRE(p->rank <= RPT * DT, "evo_latent_attn_decode: latent size (%d) must be <= %d", p->rank, RPT * DT);
  const int nr = p->rank >= DT ? DT : (p->rank + 31) / 32 * 32;
  const int ngrp = DT / nr;
  const size_t smem = sizeof(float) * ((size_t)p->dim + p->rot + p->rank + KC + (size_t)ngrp * p->rank);
  EVO_REQUIRE(smem <= 200 * 1024, "evo_latent_attn_decode: head too large for shared memory (%zu bytes)", smem);
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
