// minGRU: an element-wise gated recurrence whose gate and candidate read only the current token,
//   a_t = sigmoid(z_t + bz),  c_t = u_t + bu,  cand_t = c_t + 1/2 (c_t >= 0) | sigmoid(c_t) (c_t < 0),
//   S_t = (1 - a_t) S_{t-1} + a_t cand_t,   out_t = S_t * silu(g_t),
// with z, u, g the raw projections of the token (bf16 or fp32) and the gates, the candidate and the state in fp32.
//
// The recurrence is linear in S, S_t = p_t S_{t-1} + q_t, so a sequence is cut into chunks of CH tokens: a first kernel reduces every
// chunk to its (product of p, end value from a zero start), a second kernel folds the chunks before its own into the carried-in
// state (a few fused multiply-adds per chunk) and then walks its chunk token by token, writing the outputs.  z and u are read
// twice, g and the output once; the single-token step and short portions run the second kernel alone.  One thread owns two adjacent
// channels of one chunk (one when sizes or alignment forbid), consecutive threads consecutive channels (coalesced rows).
#include "common.cuh"
#include "../../include/evo_b200.h"

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int CH = 64;        // tokens per chunk
constexpr int TPB = 128;      // threads per CTA

// IEEE exp and division for fp32 activations (the all-fp32 mode); the hardware approximations (relative error ~1e-6) for bf16 ones
template <typename T> __device__ __forceinline__ float sigmoidf_(float v);
template <> __device__ __forceinline__ float sigmoidf_<float>(float v) { return 1.f / (1.f + expf(-v)); }
template <> __device__ __forceinline__ float sigmoidf_<bf16>(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }

// (p, q) of one token: S <- p S + q
template <typename T>
__device__ __forceinline__ void gate_pair(float z, float u, float bz, float bu, float& pp, float& qq) {
  const float a = sigmoidf_<T>(z + bz);
  const float c = u + bu;
  const float cand = c >= 0.f ? c + 0.5f : sigmoidf_<T>(c);
  pp = 1.f - a;
  qq = a * cand;
}

// two adjacent channels of a row as floats (4-byte bf16 / 8-byte fp32 accesses), or one when VW == 1
template <typename T, int VW> struct Ch;
template <typename T> struct Ch<T, 1> {
  static __device__ __forceinline__ void ld(const T* p, float* o) { o[0] = ldf(p); }
  static __device__ __forceinline__ void st(T* p, const float* v) { stf(p, v[0]); }
};
template <> struct Ch<bf16, 2> {
  static __device__ __forceinline__ void ld(const bf16* p, float* o) { const uint32_t u = *reinterpret_cast<const uint32_t*>(p); o[0] = bf_lo(u); o[1] = bf_hi(u); }
  static __device__ __forceinline__ void st(bf16* p, const float* v) { *reinterpret_cast<uint32_t*>(p) = pack_bf16(v[0], v[1]); }
};
template <> struct Ch<float, 2> {
  static __device__ __forceinline__ void ld(const float* p, float* o) { const float2 u = *reinterpret_cast<const float2*>(p); o[0] = u.x; o[1] = u.y; }
  static __device__ __forceinline__ void st(float* p, const float* v) { *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]); }
};

template <typename T, int VW>
__global__ void __launch_bounds__(TPB) mingru_chunk_kernel(evo_mingru_params p, int64_t chunk, int n_chunks, float2* __restrict__ agg, float* __restrict__ init) {
  const int ch = (blockIdx.x * TPB + threadIdx.x) * VW;
  if (ch >= p.W) return;
  const int c = blockIdx.y, b = blockIdx.z;
  const int64_t t0 = (int64_t)c * chunk, t1 = min(p.L, t0 + chunk);
  float bz[VW], bu[VW], P[VW], S[VW];
#pragma unroll
  for (int k = 0; k < VW; ++k) {
    bz[k] = p.z_bias ? __bfloat162float(((const bf16*)p.z_bias)[ch + k]) : 0.f;
    bu[k] = p.u_bias ? __bfloat162float(((const bf16*)p.u_bias)[ch + k]) : 0.f;
    // the carried-in state is copied aside: the second kernel's last chunk overwrites p.state while other chunks may not have started
    if (c == 0) init[(int64_t)b * p.W + ch + k] = (p.state && !p.zero_start) ? p.state[(int64_t)b * p.W + ch + k] : 0.f;
    P[k] = 1.f; S[k] = 0.f;
  }
  const T* z = (const T*)p.z + ((int64_t)b * p.L + t0) * p.ld + ch;
  const T* u = (const T*)p.u + ((int64_t)b * p.L + t0) * p.ld + ch;
#pragma unroll 8
  for (int64_t t = t0; t < t1; ++t, z += p.ld, u += p.ld) {
    float zv[VW], uv[VW];
    Ch<T, VW>::ld(z, zv); Ch<T, VW>::ld(u, uv);
#pragma unroll
    for (int k = 0; k < VW; ++k) {
      float pp, qq;
      gate_pair<T>(zv[k], uv[k], bz[k], bu[k], pp, qq);
      S[k] = fmaf(pp, S[k], qq);
      P[k] *= pp;
    }
  }
#pragma unroll
  for (int k = 0; k < VW; ++k) agg[((int64_t)b * n_chunks + c) * p.W + ch + k] = make_float2(P[k], S[k]);
}

template <typename T, int VW>
__global__ void __launch_bounds__(TPB) mingru_apply_kernel(evo_mingru_params p, int64_t chunk, int n_chunks, const float2* __restrict__ agg, const float* __restrict__ init) {
  const int ch = (blockIdx.x * TPB + threadIdx.x) * VW;
  const int c = blockIdx.y, b = blockIdx.z;
  const int64_t t0 = (int64_t)c * chunk, t1 = min(p.L, t0 + chunk);
  T* __restrict__ o = (T*)p.out + ((int64_t)b * p.L + t0) * p.ldo + ch;
  if (ch >= p.W) {                          // pad columns of the output (W and ldo are even when VW == 2)
    const float zero[2] = {0.f, 0.f};
    if (ch < p.ldo) for (int64_t t = t0; t < t1; ++t, o += p.ldo) Ch<T, VW>::st(o, zero);
    return;
  }
  float bz[VW], bu[VW], S[VW];
#pragma unroll
  for (int k = 0; k < VW; ++k) {
    bz[k] = p.z_bias ? __bfloat162float(((const bf16*)p.z_bias)[ch + k]) : 0.f;
    bu[k] = p.u_bias ? __bfloat162float(((const bf16*)p.u_bias)[ch + k]) : 0.f;
    S[k] = n_chunks > 1 ? init[(int64_t)b * p.W + ch + k] : ((p.state && !p.zero_start) ? p.state[(int64_t)b * p.W + ch + k] : 0.f);
  }
  for (int j = 0; j < c; ++j) {
#pragma unroll
    for (int k = 0; k < VW; ++k) {
      const float2 a = agg[((int64_t)b * n_chunks + j) * p.W + ch + k];
      S[k] = fmaf(a.x, S[k], a.y);
    }
  }
  const T* __restrict__ z = (const T*)p.z + ((int64_t)b * p.L + t0) * p.ld + ch;
  const T* __restrict__ u = (const T*)p.u + ((int64_t)b * p.L + t0) * p.ld + ch;
  const T* __restrict__ g = (const T*)p.g + ((int64_t)b * p.L + t0) * p.ld + ch;
#pragma unroll 4
  for (int64_t t = t0; t < t1; ++t, z += p.ld, u += p.ld, g += p.ld, o += p.ldo) {
    float zv[VW], uv[VW], gv[VW], ov[VW];
    Ch<T, VW>::ld(z, zv); Ch<T, VW>::ld(u, uv); Ch<T, VW>::ld(g, gv);
#pragma unroll
    for (int k = 0; k < VW; ++k) {
      float pp, qq;
      gate_pair<T>(zv[k], uv[k], bz[k], bu[k], pp, qq);
      S[k] = fmaf(pp, S[k], qq);
      ov[k] = S[k] * (gv[k] * sigmoidf_<T>(gv[k]));
    }
    Ch<T, VW>::st(o, ov);
  }
  if (c == n_chunks - 1 && p.state) {
#pragma unroll
    for (int k = 0; k < VW; ++k) p.state[(int64_t)b * p.W + ch + k] = S[k];
  }
}

inline void plan(const evo_mingru_params* p, int64_t& chunk, int& n_chunks) {
  if (p->L <= 2 * CH) { chunk = p->L > 0 ? p->L : 1; n_chunks = 1; return; }
  chunk = CH;
  n_chunks = (int)((p->L + CH - 1) / CH);
  if (n_chunks > 65535) { n_chunks = 65535; chunk = (p->L + n_chunks - 1) / n_chunks; n_chunks = (int)((p->L + chunk - 1) / chunk); }
}

}  // namespace

extern "C" size_t evo_mingru_workspace(const evo_mingru_params* p) {
  int64_t chunk; int n_chunks;
  plan(p, chunk, n_chunks);
  return n_chunks > 1 ? sizeof(float2) * (size_t)p->B * n_chunks * p->W + sizeof(float) * (size_t)p->B * p->W : 0;
}

extern "C" int evo_mingru_fwd(const evo_mingru_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  EVO_REQUIRE(p->z && p->u && p->g && p->out && p->W > 0 && p->B >= 0 && p->L >= 0 && p->ld >= p->W && p->ldo >= p->W, "evo_mingru_fwd: bad arguments");
  EVO_REQUIRE(p->B <= 65535, "evo_mingru_fwd: batch too large");
  if ((int64_t)p->B * p->L == 0) return 0;
  int64_t chunk; int n_chunks;
  plan(p, chunk, n_chunks);
  const size_t need = evo_mingru_workspace(p);
  EVO_REQUIRE(need == 0 || (workspace && workspace_bytes >= need), "evo_mingru_fwd: workspace too small (%zu < %zu)", workspace_bytes, need);
  cudaStream_t st = (cudaStream_t)stream;
  float2* agg = (float2*)workspace;
  float* init = n_chunks > 1 ? (float*)(agg + (size_t)p->B * n_chunks * p->W) : nullptr;
  const int esz = p->dtype ? 4 : 2;
  auto al = [esz](const void* q) { return ((uintptr_t)q & (uintptr_t)(2 * esz - 1)) == 0; };
  const bool two = p->W % 2 == 0 && p->ld % 2 == 0 && p->ldo % 2 == 0 && al(p->z) && al(p->u) && al(p->g) && al(p->out);
  const int per = TPB * (two ? 2 : 1);
  if (n_chunks > 1) {
    dim3 grid((unsigned)((p->W + per - 1) / per), (unsigned)n_chunks, (unsigned)p->B);
    if (p->dtype) { if (two) mingru_chunk_kernel<float, 2><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); else mingru_chunk_kernel<float, 1><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); }
    else { if (two) mingru_chunk_kernel<bf16, 2><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); else mingru_chunk_kernel<bf16, 1><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); }
    if (int rc = check_launch("evo_mingru_fwd")) return rc;
  }
  dim3 grid((unsigned)((p->ldo + per - 1) / per), (unsigned)n_chunks, (unsigned)p->B);
  if (p->dtype) { if (two) mingru_apply_kernel<float, 2><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); else mingru_apply_kernel<float, 1><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); }
  else { if (two) mingru_apply_kernel<bf16, 2><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); else mingru_apply_kernel<bf16, 1><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init); }
  return check_launch("evo_mingru_fwd");
}
