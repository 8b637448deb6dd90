// C (M, N) = A (M, K) . W (N, K)^T with plain fp32 multiply-add on the CUDA cores: the linear layer of the all-fp32 mode
// (tensor cores would round the operands to bf16 or tf32) and a shape-agnostic comparator for the tcgen05 GEMMs.
// A and C are bf16 or fp32, W is bf16 as stored; any M, N, K and any leading dimensions.
//   M >  8: 64 x 64 tiles, 16-deep k-slices through shared memory, 4 x 4 outputs per thread;
//   M <= 8: one warp per output column streams its weight row once (the single-token step is a stream of the weights).
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

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const T* __restrict__ A, int64_t lda, const bf16* __restrict__ W, int64_t ldw,
                                                        T* __restrict__ C, int64_t ldc, int64_t M, int64_t N, int64_t K) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Ws[TK][TN + 4];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = tid + i * 256, r = idx >> 4, kk = idx & 15;
      const int64_t k = k0 + kk;
      As[kk][r] = (m0 + r < M && k < K) ? ldf(A + (m0 + r) * lda + k) : 0.f;
      Ws[kk][r] = (n0 + r < N && k < K) ? __bfloat162float(W[(n0 + r) * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; w[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n < N) stf(C + m * ldc + n, acc[i][j]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gemv_simt_kernel(const T* __restrict__ A, int64_t lda, const bf16* __restrict__ W, int64_t ldw,
                                                        T* __restrict__ C, int64_t ldc, int M, int64_t N, int64_t K) {
  const int64_t n = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (n >= N) return;
  const int lane = threadIdx.x & 31;
  float acc[8] = {};
  const bf16* w = W + n * ldw;
  for (int64_t k = lane; k < K; k += 32) {
    const float wv = __bfloat162float(w[k]);
#pragma unroll
    for (int m = 0; m < 8; ++m)
      if (m < M) acc[m] = fmaf(ldf(A + m * lda + k), wv, acc[m]);
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    float v = acc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && m < M) stf(C + m * ldc + n, v);
  }
}

template <typename T>
int run(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  if (M <= 8) {
    gemv_simt_kernel<T><<<(unsigned)((N + 7) / 8), 256, 0, st>>>((const T*)A, lda, (const bf16*)W, ldw, (T*)C, ldc, (int)M, N, K);
  } else {
    dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM));
    gemm_simt_kernel<T><<<grid, 256, 0, st>>>((const T*)A, lda, (const bf16*)W, ldw, (T*)C, ldc, M, N, K);
  }
  return check_launch("evo_gemm_simt");
}

}  // namespace

extern "C" int evo_gemm_simt(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K, int dtype, void* stream) {
  EVO_REQUIRE(A && W && C && M >= 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N, "evo_gemm_simt: bad arguments");
  EVO_REQUIRE((M + TM - 1) / TM <= 65535, "evo_gemm_simt: M too large");
  if (M == 0) return 0;
  return dtype ? run<float>(A, lda, W, ldw, C, ldc, M, N, K, (cudaStream_t)stream) : run<bf16>(A, lda, W, ldw, C, ldc, M, N, K, (cudaStream_t)stream);
}
