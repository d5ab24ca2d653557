// The projections either side of attention: out [M, N] = act(a [M, K] * b [K, N] + bias)
// + addend, and the greedy head argmax_v (w [V, N] . x [N]).  They replace the 'matmul'
// op (fused qkv / q / kv / o_proj with its residual addend; packages/runntime/src/core/
// graph/ops/matmul.ts:28-99, dispatch packages/runntime/src/core/gpu/dispatch/
// matmul.ts:64-92) and 'argmaxDot' (packages/runntime/src/core/kernels/matmul/
// argmaxDot.ts).
//
// Two kernels, both on the FP32 pipes with f32 accumulation:
//  - skinny (M <= 16, the decode step): weight-bandwidth bound.  A block owns a strip of
//    32 sixteen-byte column groups; its eight warps split K, every warp streaming whole
//    512-byte row pieces of b with 16-byte loads while the few rows of a come from L1;
//    the warps' sums meet in shared memory.  b is read once (twice for M > 8).
//  - tiled (any M): 64 x 64 output tile per block, 16-deep K steps through shared memory,
//    4 x 4 outputs per thread.  This is the general fallback, not a tensor-core GEMM.
#include <cfloat>
#include "common.cuh"

namespace rt {
namespace {

// Activation codes: packages/runntime/src/core/kernels/activations.ts:6-14,29-86.
__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case 1: return tanhf(x);
    case 2: {  // gelu with the reference's erf polynomial (Abramowitz-Stegun 7.1.26)
      const float z = x * 0.70710678118654752f, az = fabsf(z);
      const float t = 1.f / (1.f + az * 0.3275911f);
      const float poly = t * (0.254829592f + t * (-0.284496736f + t * (1.421413741f +
                         t * (-1.453152027f + t * 1.061405429f))));
      const float erf = copysignf(1.f - poly * __expf(-az * az), z);
      return 0.5f * x * (1.f + erf);
    }
    case 3: return x / (1.f + __expf(-x));
    case 4: return fmaxf(x, 0.f);
    case 5: {  // torch's gelu(approximate='tanh'), tanh as 1 - 2/(e^{2u} + 1)
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      const float th = 1.f - 2.f / (__expf(2.f * u) + 1.f);
      return 0.5f * x * (1.f + th);
    }
    case 6: return fmaxf(x, 0.f) + (__expf(fminf(x, 0.f)) - 1.f);
    default: return x;
  }
}

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[16 / sizeof(T)]);
template <>
__device__ __forceinline__ void load_vec<float>(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
template <>
__device__ __forceinline__ void load_vec<__half>(const __half* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}

// ---- skinny: M <= MR rows per pass, N a multiple of the vector width -----------------
constexpr int kSkinnyThreads = 256;
constexpr int kSkinnyRows = 8;

template <typename T>
__global__ void __launch_bounds__(kSkinnyThreads)
matmul_skinny_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ bias,
                     const T* __restrict__ addend, T* __restrict__ out, int m0, int M, int64_t K,
                     int64_t N, int act) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float sAcc[kSkinnyRows][32 * V];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t col = ((int64_t)blockIdx.x * 32 + lane) * V;
  const int rows = min(kSkinnyRows, M - m0);
  for (int i = threadIdx.x; i < kSkinnyRows * 32 * V; i += kSkinnyThreads)
    (&sAcc[0][0])[i] = 0.f;
  __syncthreads();
  float acc[kSkinnyRows][V];
#pragma unroll
  for (int r = 0; r < kSkinnyRows; r++)
#pragma unroll
    for (int v = 0; v < V; v++) acc[r][v] = 0.f;
  if (col < N) {
    const T* ap = a + (int64_t)m0 * K;
    for (int64_t k = warp; k < K; k += kSkinnyThreads / 32) {
      float bv[V];
      load_vec<T>(b + k * N + col, bv);
#pragma unroll
      for (int r = 0; r < kSkinnyRows; r++) {
        if (r < rows) {
          const float av = to_f32<T>(ap[(int64_t)r * K + k]);  // same address across the warp
#pragma unroll
          for (int v = 0; v < V; v++) acc[r][v] = fmaf(av, bv[v], acc[r][v]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kSkinnyRows; r++)
      if (r < rows)
#pragma unroll
        for (int v = 0; v < V; v++) atomicAdd(&sAcc[r][lane * V + v], acc[r][v]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rows * 32 * V; i += kSkinnyThreads) {
    const int r = i / (32 * V), c = i - r * (32 * V);
    const int64_t n = (int64_t)blockIdx.x * 32 * V + c;
    if (n >= N) continue;
    float y = sAcc[r][c];
    if (bias) y += to_f32<T>(bias[n]);
    y = apply_act(y, act);
    if (addend) y += to_f32<T>(addend[(int64_t)(m0 + r) * N + n]);
    out[(int64_t)(m0 + r) * N + n] = from_f32<T>(y);
  }
}

// ---- tiled: any shape -------------------------------------------------------------------
constexpr int TM = 64, TN = 64, TK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
matmul_tiled_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ bias,
                    const T* __restrict__ addend, T* __restrict__ out, int64_t M, int64_t K,
                    int64_t N, int act) {
  __shared__ float sA[TK][TM + 1], sB[TK][TN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  const int64_t row0 = (int64_t)blockIdx.y * TM, col0 = (int64_t)blockIdx.x * TN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int r = i / TK, kk = i - r * TK;
      const int64_t gr = row0 + r, gk = k0 + kk;
      sA[kk][r] = (gr < M && gk < K) ? to_f32<T>(a[gr * K + gk]) : 0.f;
    }
    for (int i = threadIdx.x; i < TK * TN; i += 256) {
      const int kk = i / TN, c = i - kk * TN;
      const int64_t gk = k0 + kk, gc = col0 + c;
      sB[kk][c] = (gk < K && gc < N) ? to_f32<T>(b[gk * N + gc]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; kk++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = sA[kk][ty * 4 + i], bv[i] = sB[kk][tx * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t r = row0 + ty * 4 + i;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int64_t c = col0 + tx * 4 + j;
      if (c >= N) continue;
      float y = acc[i][j];
      if (bias) y += to_f32<T>(bias[c]);
      y = apply_act(y, act);
      if (addend) y += to_f32<T>(addend[r * N + c]);
      out[r * N + c] = from_f32<T>(y);
    }
  }
}

// ---- argmaxDot ------------------------------------------------------------------------
// Key that orders by value, then by lower row index: (orderable float bits, ~index).
__device__ __forceinline__ unsigned long long argmax_key(float v, uint32_t idx) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (0xffffffffu - idx);
}

template <typename T>
__global__ void __launch_bounds__(256)
argmax_dot_kernel(const T* __restrict__ w, const T* __restrict__ x, int64_t V, int64_t N,
                  unsigned long long* best) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  unsigned long long mine = 0ull;
  for (int64_t v = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); v < V; v += warps) {
    const T* row = w + v * N;
    float s = 0.f;
    for (int64_t n = lane; n < N; n += 32) s = fmaf(to_f32<T>(row[n]), to_f32<T>(x[n]), s);
    s = warp_sum(s);
    const unsigned long long key = argmax_key(s, (uint32_t)v);
    if (key > mine) mine = key;
  }
  if (lane == 0 && mine) atomicMax(best, mine);
}

__global__ void argmax_finish_kernel(const unsigned long long* best, float* out) {
  out[0] = (float)(0xffffffffu - (uint32_t)(*best & 0xffffffffull));
}

}  // namespace

cudaError_t launch_matmul(const void* a, const void* b, const void* bias, const void* addend,
                          void* out, int64_t M, int64_t K, int64_t N, int act, int dtype,
                          cudaStream_t s) {
  const int esize = dtype == RT_F16 ? 2 : 4;
  const int V = 16 / esize;
  const bool vecOk = N % V == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0;
  if (M <= 2 * kSkinnyRows && vecOk) {
    const unsigned grid = (unsigned)((N + 32 * V - 1) / (32 * V));
    for (int m0 = 0; m0 < M; m0 += kSkinnyRows) {
      if (dtype == RT_F16)
        matmul_skinny_kernel<__half><<<grid, kSkinnyThreads, 0, s>>>(
            static_cast<const __half*>(a), static_cast<const __half*>(b),
            static_cast<const __half*>(bias), static_cast<const __half*>(addend),
            static_cast<__half*>(out), m0, (int)M, K, N, act);
      else
        matmul_skinny_kernel<float><<<grid, kSkinnyThreads, 0, s>>>(
            static_cast<const float*>(a), static_cast<const float*>(b),
            static_cast<const float*>(bias), static_cast<const float*>(addend),
            static_cast<float*>(out), m0, (int)M, K, N, act);
    }
    return cudaGetLastError();
  }
  const dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM));
  if (grid.y > 65535) return cudaErrorInvalidValue;
  if (dtype == RT_F16)
    matmul_tiled_kernel<__half><<<grid, 256, 0, s>>>(
        static_cast<const __half*>(a), static_cast<const __half*>(b),
        static_cast<const __half*>(bias), static_cast<const __half*>(addend),
        static_cast<__half*>(out), M, K, N, act);
  else
    matmul_tiled_kernel<float><<<grid, 256, 0, s>>>(
        static_cast<const float*>(a), static_cast<const float*>(b), static_cast<const float*>(bias),
        static_cast<const float*>(addend), static_cast<float*>(out), M, K, N, act);
  return cudaGetLastError();
}

cudaError_t launch_argmax_dot(const void* w, const void* x, float* out, int64_t V, int64_t N,
                              int dtype, unsigned long long* scratch, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(unsigned long long), s);
  if (e != cudaSuccess) return e;
  int64_t blocks = (V + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (dtype == RT_F16)
    argmax_dot_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(
        static_cast<const __half*>(w), static_cast<const __half*>(x), V, N, scratch);
  else
    argmax_dot_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(
        static_cast<const float*>(w), static_cast<const float*>(x), V, N, scratch);
  argmax_finish_kernel<<<1, 1, 0, s>>>(scratch, out);
  return cudaGetLastError();
}

}  // namespace rt
