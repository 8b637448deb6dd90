// minGRU: an element-wise gated recurrence whose gate and candidate read only the current token,
//   a_t = sigmoid(z_t + bz),  c_t = u_t + bu,  cand_t = c_t + 1/2 (c_t >= 0) | sigmoid(c_t) (c_t < 0),
//   S_t = (1 - a_t) S_{t-1} + a_t cand_t,   out_t = S_t * silu(g_t),
// with z, u, g the raw projections of the token (bf16 or fp32) and the gates, the candidate and the state in fp32.
//
// The recurrence is linear in S, S_t = p_t S_{t-1} + q_t, so a sequence is cut into chunks of CH tokens: a first kernel reduces every
// chunk to its (product of p, end value from a zero start), a second kernel folds the chunks before its own into the carried-in
// state (a few fused multiply-adds per chunk) and then walks its chunk token by token, writing the outputs.  z and u are read
// twice, g and the output once; the single-token step and short portions run the second kernel alone.  One thread owns one
// channel of one chunk, consecutive threads consecutive channels (coalesced rows).
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
constexpr int TPB = 128;      // channels per CTA

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }

// (p, q) of one token: S <- p S + q
__device__ __forceinline__ void gate_pair(float z, float u, float bz, float bu, float& pp, float& qq) {
  const float a = sigmoidf_(z + bz);
  const float c = u + bu;
  const float cand = c >= 0.f ? c + 0.5f : sigmoidf_(c);
  pp = 1.f - a;
  qq = a * cand;
}

template <typename T>
__global__ void __launch_bounds__(TPB) mingru_chunk_kernel(evo_mingru_params p, int64_t chunk, int n_chunks, float2* __restrict__ agg, float* __restrict__ init) {
  const int ch = blockIdx.x * TPB + threadIdx.x;
  if (ch >= p.W) return;
  const int c = blockIdx.y, b = blockIdx.z;
  const int64_t t0 = (int64_t)c * chunk, t1 = min(p.L, t0 + chunk);
  const float bz = p.z_bias ? __bfloat162float(((const bf16*)p.z_bias)[ch]) : 0.f;
  const float bu = p.u_bias ? __bfloat162float(((const bf16*)p.u_bias)[ch]) : 0.f;
  const T* z = (const T*)p.z + ((int64_t)b * p.L + t0) * p.ld + ch;
  const T* u = (const T*)p.u + ((int64_t)b * p.L + t0) * p.ld + ch;
  // the carried-in state is copied aside: the second kernel's last chunk overwrites p.state while other chunks may not have started
  if (c == 0) init[(int64_t)b * p.W + ch] = (p.state && !p.zero_start) ? p.state[(int64_t)b * p.W + ch] : 0.f;
  float P = 1.f, S = 0.f;
#pragma unroll 4
  for (int64_t t = t0; t < t1; ++t, z += p.ld, u += p.ld) {
    float pp, qq;
    gate_pair(ldf(z), ldf(u), bz, bu, pp, qq);
    S = fmaf(pp, S, qq);
    P *= pp;
  }
  agg[((int64_t)b * n_chunks + c) * p.W + ch] = make_float2(P, S);
}

template <typename T>
__global__ void __launch_bounds__(TPB) mingru_apply_kernel(evo_mingru_params p, int64_t chunk, int n_chunks, const float2* __restrict__ agg, const float* __restrict__ init) {
  const int ch = blockIdx.x * TPB + threadIdx.x;
  const int c = blockIdx.y, b = blockIdx.z;
  const int64_t t0 = (int64_t)c * chunk, t1 = min(p.L, t0 + chunk);
  T* o = (T*)p.out + ((int64_t)b * p.L + t0) * p.ldo + ch;
  if (ch >= p.W) {                          // pad columns of the output
    if (ch < p.ldo) for (int64_t t = t0; t < t1; ++t, o += p.ldo) stf(o, 0.f);
    return;
  }
  const float bz = p.z_bias ? __bfloat162float(((const bf16*)p.z_bias)[ch]) : 0.f;
  const float bu = p.u_bias ? __bfloat162float(((const bf16*)p.u_bias)[ch]) : 0.f;
  float S = n_chunks > 1 ? init[(int64_t)b * p.W + ch] : ((p.state && !p.zero_start) ? p.state[(int64_t)b * p.W + ch] : 0.f);
  for (int k = 0; k < c; ++k) {
    const float2 a = agg[((int64_t)b * n_chunks + k) * p.W + ch];
    S = fmaf(a.x, S, a.y);
  }
  const T* z = (const T*)p.z + ((int64_t)b * p.L + t0) * p.ld + ch;
  const T* u = (const T*)p.u + ((int64_t)b * p.L + t0) * p.ld + ch;
  const T* g = (const T*)p.g + ((int64_t)b * p.L + t0) * p.ld + ch;
#pragma unroll 4
  for (int64_t t = t0; t < t1; ++t, z += p.ld, u += p.ld, g += p.ld, o += p.ldo) {
    float pp, qq;
    gate_pair(ldf(z), ldf(u), bz, bu, pp, qq);
    S = fmaf(pp, S, qq);
    const float gv = ldf(g);
    stf(o, S * (gv * sigmoidf_(gv)));
  }
  if (c == n_chunks - 1 && p.state) p.state[(int64_t)b * p.W + ch] = S;
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
  if (n_chunks > 1) {
    dim3 grid((unsigned)((p->W + TPB - 1) / TPB), (unsigned)n_chunks, (unsigned)p->B);
    if (p->dtype) mingru_chunk_kernel<float><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init);
    else mingru_chunk_kernel<bf16><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init);
    if (int rc = check_launch("evo_mingru_fwd")) return rc;
  }
  dim3 grid((unsigned)((p->ldo + TPB - 1) / TPB), (unsigned)n_chunks, (unsigned)p->B);
  if (p->dtype) mingru_apply_kernel<float><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init);
  else mingru_apply_kernel<bf16><<<grid, TPB, 0, st>>>(*p, chunk, n_chunks, agg, init);
  return check_launch("evo_mingru_fwd");
}
