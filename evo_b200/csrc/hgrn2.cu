// Gated linear recurrence (HGRN2) as one fused kernel: gate activation (sigmoid with a learned lower bound), query
// activation (SiLU), the matrix-state recurrence S <- diag(g) S + (1 - g) v^T, the read-out o = S^T q and the per-head
// RMS norm with weight.  Everything after the raw projections is fp32, and the state stays in registers for the whole
// sequence: HBM sees q, f, v once, the output once and the state once per call.
//
// One CTA per (head, sequence).  A thread owns RPT consecutive state rows of one value channel: thread (kp, j) holds
// S[kp*RPT .. kp*RPT+RPT) [j]; 16 tokens of activated gates / queries / values are staged in shared memory per round, so the
// time loop runs without barriers; partial read-outs of the dk/RPT row groups are folded after each round.
// Measured on B200: the time loop is bound by instruction issue and by the shared-memory -> register path of the (gate, query)
// pairs, and it wants many resident warps: 1024 threads with 16 state rows each beat 512 threads x 32 rows, 256 threads x
// (16 rows x 4 value channels) and a register-prefetched staging (3.1 vs 3.8, 4.7 and 6.3 ms per 4 x 4096 tokens x 32 heads of 128 x 128).
// The same kernel serves the single-token step (L == 1): the state is then streamed through once.
// Value channels are independent in the recurrence, so a head whose state does not fit one CTA's registers is split over
// several CTAs by value channel; the read-outs then go to an fp32 workspace and a second small kernel applies the head norm.
#include "common.cuh"
#include "../../include/evo_b200.h"
#include <algorithm>

using namespace evo;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int TCH = 16;      // tokens staged per round

template <typename T, int RPT>
__global__ void __launch_bounds__(RPT <= 16 ? 1024 : (RPT == 32 ? 512 : 256), 1) hgrn2_kernel(evo_hgrn2_params p, int KP, int dvp, float* __restrict__ raw, int4 steps) {
  extern __shared__ __align__(16) float smem[];
  const int dk = p.dk, dv = p.dv, dkp = KP * RPT;
  float2* fq = reinterpret_cast<float2*>(smem);            // [TCH][dkp]  (gate, activated query)
  float* vv = smem + 2 * TCH * dkp;                        // [TCH][dvp]
  float* op = vv + TCH * dvp;                              // [TCH][KP][dvp]
  const int h = blockIdx.x, b = blockIdx.y;
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int j0 = blockIdx.z * dvp;                         // first value channel of this CTA
  const int j = j0 + tid % dvp, kp = tid / dvp;
  const bool live = j < dv;
  const T* qp = (const T*)p.q + h * dk;
  const T* fp = (const T*)p.f + h * dk;
  const T* vp = (const T*)p.v + h * dv;
  const bf16* fb = (const bf16*)p.f_bias + h * dk;
  const bf16* lo = (const bf16*)p.lower + h * dk;
  const bf16* nw = (const bf16*)p.norm_w;
  float* Sg = p.state ? p.state + ((int64_t)b * p.H + h) * dk * (int64_t)dv : nullptr;

  float S[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int k = kp * RPT + r;
    S[r] = (Sg && !p.zero_start && live && k < dk) ? Sg[(int64_t)k * dv + j] : 0.f;
  }

  for (int64_t t0 = 0; t0 < p.L; t0 += TCH) {
    const int nt = (int)min((int64_t)TCH, p.L - t0);
    const int64_t row0 = (int64_t)b * p.L + t0;
    __syncthreads();                                   // the previous round's read-outs have been folded
    // (token, channel) of this thread's first element; steps = blockDim / and % the row widths, from the host: no division inside the loops
    for (int tt = tid / dkp, k = tid % dkp; tt < nt; ) {
      float2 e = make_float2(0.f, 0.f);
      if (k < dk) {
        const float l = __bfloat162float(lo[k]);
        const float fr = ldf(fp + (row0 + tt) * p.ld + k) + __bfloat162float(fb[k]);
        const float qr = ldf(qp + (row0 + tt) * p.ld + k);
        e.x = l + (1.f - l) / (1.f + expf(-fr));
        e.y = qr / (1.f + expf(-qr));
      }
      fq[tt * dkp + k] = e;
      tt += steps.x; k += steps.y;
      if (k >= dkp) { k -= dkp; ++tt; }
    }
    for (int tt = tid / dvp, c = tid % dvp; tt < nt; ) {
      vv[tt * dvp + c] = j0 + c < dv ? ldf(vp + (row0 + tt) * p.ld + j0 + c) : 0.f;
      tt += steps.z; c += steps.w;
      if (c >= dvp) { c -= dvp; ++tt; }
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float v = vv[tt * dvp + (j - j0)];
      const float4* e = reinterpret_cast<const float4*>(fq + tt * dkp + kp * RPT);       // two state rows per 16-byte read
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < RPT / 2; ++r) {
        const float4 g = e[r];
        S[2 * r] = fmaf(g.x, S[2 * r] - v, v);         // g S + (1 - g) v
        o = fmaf(S[2 * r], g.y, o);
        S[2 * r + 1] = fmaf(g.z, S[2 * r + 1] - v, v);
        o = fmaf(S[2 * r + 1], g.w, o);
      }
      op[(tt * KP + kp) * dvp + (j - j0)] = o;
    }
    __syncthreads();
    // fold the row groups, norm over the head's dv values, store: one warp per token
    for (int tt = tid >> 5; tt < nt; tt += nthr >> 5) {
      const int lane = tid & 31;
      if (raw) {                                       // split head: un-normed read-outs, the norm follows in head_norm_kernel
        for (int c = lane; c < dvp && j0 + c < dv; c += 32) {
          float o = 0.f;
          for (int q = 0; q < KP; ++q) o += op[(tt * KP + q) * dvp + c];
          raw[((row0 + tt) * p.H + h) * dv + j0 + c] = o;
        }
        continue;
      }
      float ss = 0.f;
      for (int c = lane; c < dv; c += 32) {
        float o = 0.f;
        for (int q = 0; q < KP; ++q) o += op[(tt * KP + q) * dvp + c];
        op[(tt * KP) * dvp + c] = o;                   // this lane re-reads its own columns below
        ss = fmaf(o, o, ss);
      }
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
      const float rstd = 1.0f / sqrtf(ss / (float)dv + p.eps);
      T* orow = (T*)p.out + (row0 + tt) * p.ldo;
      for (int c = lane; c < dv; c += 32) stf(orow + h * dv + c, op[(tt * KP) * dvp + c] * rstd * __bfloat162float(nw[c]));
      if (h == p.H - 1)
        for (int64_t c = (int64_t)p.H * dv + lane; c < p.ldo; c += 32) stf(orow + c, 0.f);
    }
  }
  if (Sg && live) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int k = kp * RPT + r;
      if (k < dk) Sg[(int64_t)k * dv + j] = S[r];
    }
  }
}

// second pass of a split head: out = raw / sqrt(mean(raw^2) + eps) * norm_w, one warp per (row, head)
template <typename T>
__global__ void head_norm_kernel(evo_hgrn2_params p, const float* __restrict__ raw) {
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= (int64_t)p.B * p.L * p.H) return;
  const int64_t row = wid / p.H; const int h = (int)(wid % p.H);
  const float* r = raw + wid * p.dv;
  float ss = 0.f;
  for (int c = lane; c < p.dv; c += 32) ss = fmaf(r[c], r[c], ss);
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s);
  const float rstd = 1.0f / sqrtf(ss / (float)p.dv + p.eps);
  T* orow = (T*)p.out + row * p.ldo;
  const bf16* nw = (const bf16*)p.norm_w;
  for (int c = lane; c < p.dv; c += 32) stf(orow + h * p.dv + c, r[c] * rstd * __bfloat162float(nw[c]));
  if (h == p.H - 1)
    for (int64_t c = (int64_t)p.H * p.dv + lane; c < p.ldo; c += 32) stf(orow + c, 0.f);
}

struct Plan { int rpt, KP, dvc, chunks; };
// fewest state rows per thread that still fit one CTA (more threads hide the shared-memory latency of the time loop);
// heads too large for that are split by value channel with 64 rows per thread
inline Plan plan(int dk, int dv, int64_t ctas, int64_t L) {
  const int dvp = (dv + 31) / 32 * 32;
  for (int rpt : {8, 16, 32, 64}) {
    const int KP = (dk + rpt - 1) / rpt;
    if ((int64_t)KP * dvp <= (rpt <= 16 ? 1024 : (rpt == 32 ? 512 : 256))) {      // register budget: rpt state rows per thread
      // long sequences on few (head, sequence) pairs: spread the value channels over more CTAs so that every SM has one
      // (the extra fp32 round trip of the read-outs is small against a scan that leaves SMs idle)
      int chunks = 1;
      if (L >= 256 && ctas * 2 <= device_sm_count() && dvp >= 64) chunks = (int)std::min<int64_t>(dvp / 32, device_sm_count() / ctas);
      const int dvc = (dvp / 32 + chunks - 1) / chunks * 32;
      // a split CTA has fewer value channels: give its threads fewer rows again so that it keeps as many warps
      if (chunks > 1)
        for (int r2 : {8, 16})
          if (r2 < rpt && (int64_t)((dk + r2 - 1) / r2) * dvc <= 1024) return {r2, (dk + r2 - 1) / r2, dvc, (dv + dvc - 1) / dvc};
      return {rpt, KP, dvc, (dv + dvc - 1) / dvc};
    }
  }
  const int KP = (dk + 63) / 64;
  const int dvc = 256 / KP / 32 * 32;
  if (dvc < 32) return {0, 0, 0, 0};
  return {64, KP, dvc, (dv + dvc - 1) / dvc};
}

template <typename T, int RPT>
int launch(const evo_hgrn2_params* p, int KP, int dvp, int chunks, float* raw, cudaStream_t st) {
  const size_t smem = sizeof(float) * ((size_t)2 * TCH * KP * RPT + (size_t)TCH * dvp + (size_t)TCH * KP * dvp);
  auto kern = hgrn2_kernel<T, RPT>;
  if (smem > 48 * 1024) EVO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int nthr = KP * dvp, dkp = KP * RPT;
  kern<<<dim3(p->H, p->B, chunks), dim3(nthr), smem, st>>>(*p, KP, dvp, raw, make_int4(nthr / dkp, nthr % dkp, nthr / dvp, nthr % dvp));
  int rc = check_launch("evo_hgrn2_fwd");
  if (rc || !raw) return rc;
  const int64_t warps = (int64_t)p->B * p->L * p->H;
  head_norm_kernel<T><<<(unsigned)((warps + 7) / 8), 256, 0, st>>>(*p, raw);
  return check_launch("evo_hgrn2_fwd");
}

template <typename T>
int dispatch(const evo_hgrn2_params* p, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  const Plan pl = plan(p->dk, p->dv, (int64_t)p->B * p->H, p->L);
  if (pl.rpt == 0) { set_error("evo_hgrn2_fwd: dk (%d) must be <= 512", p->dk); return -1; }
  float* raw = nullptr;
  if (pl.chunks > 1) {
    const size_t need = sizeof(float) * (size_t)p->B * p->L * p->H * p->dv;
    if (!workspace || workspace_bytes < need) { set_error("evo_hgrn2_fwd: workspace too small (%zu < %zu)", workspace_bytes, need); return -1; }
    raw = (float*)workspace;
  }
  if (pl.rpt == 8) return launch<T, 8>(p, pl.KP, pl.dvc, pl.chunks, raw, st);
  if (pl.rpt == 16) return launch<T, 16>(p, pl.KP, pl.dvc, pl.chunks, raw, st);
  if (pl.rpt == 32) return launch<T, 32>(p, pl.KP, pl.dvc, pl.chunks, raw, st);
  return launch<T, 64>(p, pl.KP, pl.dvc, pl.chunks, raw, st);
}

}  // namespace

extern "C" size_t evo_hgrn2_workspace(const evo_hgrn2_params* p) {
  const Plan pl = plan(p->dk, p->dv, (int64_t)p->B * p->H, p->L);
  return pl.chunks > 1 ? sizeof(float) * (size_t)p->B * p->L * p->H * p->dv : 0;
}

extern "C" int evo_hgrn2_fwd(const evo_hgrn2_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  EVO_REQUIRE(p->q && p->f && p->v && p->f_bias && p->lower && p->norm_w && p->out, "evo_hgrn2_fwd: null argument");
  EVO_REQUIRE(p->B >= 0 && p->L >= 0 && p->H > 0 && p->dk > 0 && p->dv > 0 && p->ldo >= (int64_t)p->H * p->dv, "evo_hgrn2_fwd: bad shape");
  if (p->B == 0 || p->L == 0) return 0;
  return p->dtype ? dispatch<float>(p, workspace, workspace_bytes, (cudaStream_t)stream) : dispatch<bf16>(p, workspace, workspace_bytes, (cudaStream_t)stream);
}
