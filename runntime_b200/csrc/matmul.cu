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
//    row pieces of b (8 or 16 bytes per lane) while the few rows of a come from L1;
//    the warps' sums meet in shared memory.  b is read once (twice for M > 8).
//  - tiled (any M): 64 x 64 output tile per block, 16-deep K steps through shared memory,
//    4 x 4 outputs per thread.  This is the general fallback, not a tensor-core GEMM.
#include <cfloat>
#include <type_traits>
#include "common.cuh"
#include "sm100.cuh"

namespace rt {
namespace {

// Runtime activation code, for epilogues that touch a handful of elements per thread.
__device__ __noinline__ float apply_act(float x, int act) {
  float y = x;
  act_dispatch(act, [&](auto code) { y = act_apply<decltype(code)::value>(x); });
  return y;
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

// ---- skinny: M <= 8 rows per pass, N a multiple of the vector width ----------------------
// A block owns a strip of 256 sixteen-byte column groups (4 KB of every row of b,
// contiguous in memory: narrow strips waste most of each DRAM page) and a slice of K.
// Every thread keeps its own 8 x V accumulators, takes eight rows of b per step (eight
// 16-byte loads in flight, kept packed until used) and reads a from shared memory, where
// the block's rows of a for its K slice are staged as f32 once.  With one slice the
// epilogue is applied here; with more, the sums are added into `partial` [M][N] f32
// (zeroed before the launch) and matmul_skinny_finish_kernel applies the epilogue.
constexpr int kSkinnyThreads = 256;
constexpr int kSkinnyRows = 8;
constexpr int kSkinnyU = 8;
constexpr int kSkinnyBlocksPerSm = 2;   // measured: 2.01 TB/s against 1.85 with one

template <typename T>
__global__ void __launch_bounds__(kSkinnyThreads, 2)
matmul_skinny_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ bias,
                     const T* __restrict__ addend, T* __restrict__ out, float* __restrict__ partial,
                     int m0, int M, int64_t K, int64_t N, int kPerSlice, int act) {
  constexpr int V = 16 / sizeof(T), U = kSkinnyU;
  extern __shared__ __align__(16) float sA[];          // [kSkinnyRows][kPad]
  const int64_t col = ((int64_t)blockIdx.x * kSkinnyThreads + threadIdx.x) * V;
  const int rows = min(kSkinnyRows, M - m0);
  const int64_t kBegin = (int64_t)blockIdx.y * kPerSlice;
  const int kLen = (int)min((int64_t)kPerSlice, K - kBegin);
  const int kPad = (kPerSlice + U - 1) / U * U;
  for (int i = threadIdx.x; i < kSkinnyRows * kPad; i += kSkinnyThreads) {
    const int r = i / kPad, kk = i - r * kPad;
    sA[i] = (r < rows && kk < kLen) ? to_f32<T>(a[(int64_t)(m0 + r) * K + kBegin + kk]) : 0.f;
  }
  __syncthreads();
  const bool inRange = col < N;
  float acc[kSkinnyRows][V];
#pragma unroll
  for (int r = 0; r < kSkinnyRows; r++)
#pragma unroll
    for (int v = 0; v < V; v++) acc[r][v] = 0.f;
  const T* bp = b + kBegin * N + col;
  for (int k0 = 0; inRange && k0 < kLen; k0 += U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      raw[u] = make_uint4(0, 0, 0, 0);
      if (k0 + u < kLen) raw[u] = *reinterpret_cast<const uint4*>(bp + (int64_t)(k0 + u) * N);
    }
#pragma unroll
    for (int u4 = 0; u4 < U; u4 += 4) {
      float bv[4][V];
#pragma unroll
      for (int u = 0; u < 4; u++) load_vec<T>(reinterpret_cast<const T*>(&raw[u4 + u]), bv[u]);
#pragma unroll
      for (int r = 0; r < kSkinnyRows; r++) {
        // four consecutive k of row r in one broadcast load; rows past M hold zeros
        const float4 av = *reinterpret_cast<const float4*>(&sA[r * kPad + k0 + u4]);
        const float a4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
          for (int v = 0; v < V; v++) acc[r][v] = fmaf(a4[u], bv[u][v], acc[r][v]);
      }
    }
  }
  if (partial) {
    // Row by row through shared memory, so that the adds into the f32 accumulator are
    // coalesced (a lane per consecutive column) instead of eight columns per lane.
    __syncthreads();                         // everybody is done reading sA
    float* sRow = sA;                        // kSkinnyThreads * V floats fit: see the launcher
#pragma unroll
    for (int r = 0; r < kSkinnyRows; r++) {
      if (r >= rows) break;
#pragma unroll
      for (int v = 0; v < V; v++) sRow[threadIdx.x * V + v] = acc[r][v];
      __syncthreads();
      const int64_t n0 = (int64_t)blockIdx.x * kSkinnyThreads * V;
      for (int c = threadIdx.x; c < kSkinnyThreads * V; c += kSkinnyThreads)
        if (n0 + c < N) atomicAdd(&partial[(int64_t)(m0 + r) * N + n0 + c], sRow[c]);
      __syncthreads();
    }
    return;
  }
  if (!inRange) return;
#pragma unroll
  for (int r = 0; r < kSkinnyRows; r++) {
    if (r >= rows) continue;
#pragma unroll
    for (int v = 0; v < V; v++) {
      const int64_t n = col + v;
      float y = acc[r][v];
      if (bias) y += to_f32<T>(bias[n]);
      y = apply_act(y, act);
      if (addend) y += to_f32<T>(addend[(int64_t)(m0 + r) * N + n]);
      out[(int64_t)(m0 + r) * N + n] = from_f32<T>(y);
    }
  }
}

// ---- skinny, fed by a bulk-copy ring ---------------------------------------------------
// The same decomposition (a block = 4 KB of every row of b in a slice of K), but the rows
// arrive in shared memory through a ring of cp.async.bulk stages issued by a producer
// warp, so that tens of kilobytes per SM are in flight however few registers the
// consumers have; the consumers (one per sixteen-byte column group) read their piece of
// each row from shared memory.  Needs N * sizeof(T) a multiple of 16 and aligned bases.
constexpr int kRingRows = 4;      // rows of b per stage (16 KB)
constexpr int kRingStages = 5;    // 80 KB of b in flight per block, two blocks per SM

template <typename T>
__global__ void __launch_bounds__(kSkinnyThreads + 32, 2)
matmul_skinny_ring_kernel(const T* __restrict__ a, const T* __restrict__ b,
                          const T* __restrict__ bias, const T* __restrict__ addend,
                          T* __restrict__ out, float* __restrict__ partial, int m0, int M, int64_t K,
                          int64_t N, int kPerSlice, int act) {
  using namespace sm100;
  constexpr int V = 16 / sizeof(T), R = kRingRows, S = kRingStages;
  constexpr int kStripBytes = kSkinnyThreads * 16;             // 4 KB of one row
  extern __shared__ __align__(128) unsigned char smemRaw[];
  __shared__ __align__(8) uint64_t sFull[S], sEmpty[S];
  __shared__ int sAbort;
  unsigned char* ring = smemRaw;                                // [S][R][kStripBytes]
  float* sA = reinterpret_cast<float*>(smemRaw + (size_t)S * R * kStripBytes);  // [rows][kPad]
  const int tid = threadIdx.x;
  const int64_t col0 = (int64_t)blockIdx.x * kSkinnyThreads * V;
  const int64_t colsHere = min((int64_t)kSkinnyThreads * V, N - col0);
  const uint32_t rowBytes = (uint32_t)(colsHere * sizeof(T));    // a multiple of 16
  const int rows = min(kSkinnyRows, M - m0);
  const int64_t kBegin = (int64_t)blockIdx.y * kPerSlice;
  const int kLen = (int)min((int64_t)kPerSlice, K - kBegin);
  const int kPad = (kPerSlice + 3) / 4 * 4;
  const int nTiles = (kLen + R - 1) / R;
  if (tid == 0) {
    sAbort = 0;
    for (int i = 0; i < S; i++) {
      mbar_init(smem_u32(&sFull[i]), 1);
      mbar_init(smem_u32(&sEmpty[i]), kSkinnyThreads / 32);
    }
    fence_barrier_init();
  }
  for (int i = tid; i < kSkinnyRows * kPad; i += kSkinnyThreads + 32) {
    const int r = i / kPad, kk = i - r * kPad;
    sA[i] = (r < rows && kk < kLen) ? to_f32<T>(a[(int64_t)(m0 + r) * K + kBegin + kk]) : 0.f;
  }
  __syncthreads();

  if (tid >= kSkinnyThreads) {
    // ---------------- producer warp ----------------
    if (tid == kSkinnyThreads) {
      const T* src = b + kBegin * N + col0;
      for (int it = 0; it < nTiles; it++) {
        const int st = it % S;
        if (it >= S && !mbar_wait(smem_u32(&sEmpty[st]), ((it / S) - 1) & 1, &sAbort)) break;
        const int nr = min(R, kLen - it * R);
        mbar_expect_tx(smem_u32(&sFull[st]), (uint32_t)nr * rowBytes);
        for (int r = 0; r < nr; r++)
          bulk_g2s(smem_u32(ring + ((size_t)st * R + r) * kStripBytes),
                   src + (int64_t)(it * R + r) * N, rowBytes, smem_u32(&sFull[st]));
      }
    }
    return;
  }

  // ---------------- consumers: one sixteen-byte column group each ----------------
  const bool inRange = (int64_t)tid * V < colsHere;
  float acc[kSkinnyRows][V];
#pragma unroll
  for (int r = 0; r < kSkinnyRows; r++)
#pragma unroll
    for (int v = 0; v < V; v++) acc[r][v] = 0.f;
  bool ok = true;
  for (int it = 0; it < nTiles; it++) {
    const int st = it % S;
    if (!mbar_wait(smem_u32(&sFull[st]), (it / S) & 1, &sAbort)) { ok = false; break; }
    const int nr = min(R, kLen - it * R);
    if (inRange) {
#pragma unroll
      for (int u = 0; u < R; u++) {
        if (u < nr) {
          float bv[V];
          load_vec<T>(reinterpret_cast<const T*>(ring + ((size_t)st * R + u) * kStripBytes) + tid * V, bv);
#pragma unroll
          for (int r = 0; r < kSkinnyRows; r++) {
            const float av = sA[r * kPad + it * R + u];  // broadcast; rows past M hold zeros
#pragma unroll
            for (int v = 0; v < V; v++) acc[r][v] = fmaf(av, bv[v], acc[r][v]);
          }
        }
      }
    }
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(smem_u32(&sEmpty[st]));
  }
  // Every consumer comes here, also one whose wait ran out (the others' waits then end at
  // their next look at the abort word), so the decision below is the same for all.
  (void)ok;
  named_barrier_sync(1, kSkinnyThreads);
  if (sAbort) return;          // a bounded wait ran out: leave the output untouched
  const int64_t col = col0 + (int64_t)tid * V;
  if (partial) {
    // Row by row through shared memory (the ring is free now), so that the adds into the
    // f32 accumulator are coalesced: a lane per consecutive column.
    float* sRow = reinterpret_cast<float*>(ring);
#pragma unroll
    for (int r = 0; r < kSkinnyRows; r++) {
      if (r >= rows) break;
#pragma unroll
      for (int v = 0; v < V; v++) sRow[tid * V + v] = acc[r][v];
      named_barrier_sync(1, kSkinnyThreads);
      for (int c = tid; c < colsHere; c += kSkinnyThreads)
        atomicAdd(&partial[(int64_t)(m0 + r) * N + col0 + c], sRow[c]);
      named_barrier_sync(1, kSkinnyThreads);
    }
    return;
  }
  if (!inRange) return;
#pragma unroll
  for (int r = 0; r < kSkinnyRows; r++) {
    if (r >= rows) continue;
#pragma unroll
    for (int v = 0; v < V; v++) {
      const int64_t n = col + v;
      float y = acc[r][v];
      if (bias) y += to_f32<T>(bias[n]);
      y = apply_act(y, act);
      if (addend) y += to_f32<T>(addend[(int64_t)(m0 + r) * N + n]);
      out[(int64_t)(m0 + r) * N + n] = from_f32<T>(y);
    }
  }
}

template <typename T>
__global__ void matmul_skinny_finish_kernel(const float* __restrict__ partial,
                                            const T* __restrict__ bias,
                                            const T* __restrict__ addend, T* __restrict__ out,
                                            int64_t M, int64_t N, int act) {
  const int64_t total = M * N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    float y = partial[i];
    if (bias) y += to_f32<T>(bias[i % N]);
    y = apply_act(y, act);
    if (addend) y += to_f32<T>(addend[i]);
    out[i] = from_f32<T>(y);
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
                  unsigned long long* best, bool vec) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  unsigned long long mine = 0ull;
  for (int64_t v = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); v < V; v += warps) {
    const T* row = w + v * N;
    float s = 0.f;
    if (vec) {
      constexpr int VV = 16 / sizeof(T);
      for (int64_t n = (int64_t)lane * VV; n < N; n += 32 * VV) {
        float wv[VV], xv[VV];
        load_vec<T>(row + n, wv);
        load_vec<T>(x + n, xv);
#pragma unroll
        for (int e = 0; e < VV; e++) s = fmaf(wv[e], xv[e], s);
      }
    } else {
      for (int64_t n = lane; n < N; n += 32) s = fmaf(to_f32<T>(row[n]), to_f32<T>(x[n]), s);
    }
    s = warp_sum(s);
    const unsigned long long key = argmax_key(s, (uint32_t)v);
    if (key > mine) mine = key;
  }
  if (lane == 0 && mine) atomicMax(best, mine);
}

__global__ void argmax_finish_kernel(const unsigned long long* best, float* out) {
  out[0] = (float)(0xffffffffu - (uint32_t)(*best & 0xffffffffull));
}


// K slices for the skinny kernel: enough blocks for two per SM, at least 32 rows
// each, and few enough rows that the slice of a fits shared memory.
int skinny_slices(int64_t K, int64_t strips) {
  int64_t want = (kSkinnyBlocksPerSm * 148 + strips - 1) / strips;
  const int64_t maxByRows = K / 32 > 0 ? K / 32 : 1;
  if (want > maxByRows) want = maxByRows;
  const int64_t minBySmem = (K + 1023) / 1024;
  if (want < minBySmem) want = minBySmem;
  return (int)(want < 1 ? 1 : want);
}

bool skinny_ok(int64_t M, int64_t N, const void* b, int esize) {
  return M <= 2 * kSkinnyRows && N % (16 / esize) == 0 && reinterpret_cast<uintptr_t>(b) % 16 == 0;
}

template <typename T>
cudaError_t matmul_typed(const void* a, const void* b, const void* bias, const void* addend,
                         void* out, int64_t M, int64_t K, int64_t N, int act, float* scratch,
                         cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  auto* ai = static_cast<const T*>(a);
  auto* bi = static_cast<const T*>(b);
  auto* ci = static_cast<const T*>(bias);
  auto* di = static_cast<const T*>(addend);
  auto* oi = static_cast<T*>(out);
  if (skinny_ok(M, N, b, sizeof(T))) {
    const int64_t strips = (N + kSkinnyThreads * V - 1) / (kSkinnyThreads * V);
    const int slices = skinny_slices(K, strips);
    if (slices > 1 && !scratch) return cudaErrorInvalidValue;
    const int kPerSlice = (int)((K + slices - 1) / slices);
    const dim3 grid((unsigned)strips, (unsigned)slices);
    float* partial = slices > 1 ? scratch : nullptr;
    if (partial) {
      cudaError_t e = cudaMemsetAsync(partial, 0, (size_t)M * N * sizeof(float), s);
      if (e != cudaSuccess) return e;
    }
    size_t smem = (size_t)kSkinnyRows * ((kPerSlice + kSkinnyU - 1) / kSkinnyU * kSkinnyU) * 4;
    if (smem < (size_t)kSkinnyThreads * V * 4) smem = (size_t)kSkinnyThreads * V * 4;
    // The ring kernel when a's slice fits beside the ring (two blocks per SM).
    const size_t ringBytes = (size_t)kRingStages * kRingRows * kSkinnyThreads * 16;
    const size_t ringSmem = ringBytes + (size_t)kSkinnyRows * ((kPerSlice + 3) / 4 * 4) * 4;
    const bool useRing = ringSmem <= 110 * 1024 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    if (useRing) {
      auto kern = matmul_skinny_ring_kernel<T>;
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)ringSmem);
      if (e != cudaSuccess) return e;
      for (int m0 = 0; m0 < M; m0 += kSkinnyRows)
        kern<<<grid, kSkinnyThreads + 32, ringSmem, s>>>(ai, bi, ci, di, oi, partial, m0, (int)M, K,
                                                         N, kPerSlice, act);
    } else {
      for (int m0 = 0; m0 < M; m0 += kSkinnyRows)
        matmul_skinny_kernel<T><<<grid, kSkinnyThreads, smem, s>>>(ai, bi, ci, di, oi, partial, m0,
                                                                  (int)M, K, N, kPerSlice, act);
    }
    if (partial) {
      int64_t blocks = (M * N + 255) / 256;
      if (blocks > 148 * 8) blocks = 148 * 8;
      matmul_skinny_finish_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(partial, ci, di, oi, M, N, act);
    }
    return cudaGetLastError();
  }
  const dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM));
  if (grid.y > 65535) return cudaErrorInvalidValue;
  matmul_tiled_kernel<T><<<grid, 256, 0, s>>>(ai, bi, ci, di, oi, M, K, N, act);
  return cudaGetLastError();
}

}  // namespace

size_t matmul_scratch_need(int64_t M, int64_t K, int64_t N, int dtype) {
  const int esize = dtype == RT_F16 ? 2 : 4;
  if (M > 2 * kSkinnyRows || N % (16 / esize) != 0) return 0;
  const int64_t strips = (N + kSkinnyThreads * (16 / esize) - 1) / (kSkinnyThreads * (16 / esize));
  return skinny_slices(K, strips) > 1 ? (size_t)M * N * sizeof(float) : 0;
}

cudaError_t launch_matmul(const void* a, const void* b, const void* bias, const void* addend,
                          void* out, int64_t M, int64_t K, int64_t N, int act, int dtype,
                          float* scratch, cudaStream_t s) {
  return dtype == RT_F16
             ? matmul_typed<__half>(a, b, bias, addend, out, M, K, N, act, scratch, s)
             : matmul_typed<float>(a, b, bias, addend, out, M, K, N, act, scratch, s);
}

cudaError_t launch_argmax_dot(const void* w, const void* x, float* out, int64_t V, int64_t N,
                              int dtype, unsigned long long* scratch, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(unsigned long long), s);
  if (e != cudaSuccess) return e;
  int64_t blocks = (V + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const int vv = 16 / (dtype == RT_F16 ? 2 : 4);
  const bool vec = N % vv == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(x) % 16 == 0;
  if (dtype == RT_F16)
    argmax_dot_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(
        static_cast<const __half*>(w), static_cast<const __half*>(x), V, N, scratch, vec);
  else
    argmax_dot_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(
        static_cast<const float*>(w), static_cast<const float*>(x), V, N, scratch, vec);
  argmax_finish_kernel<<<1, 1, 0, s>>>(scratch, out);
  return cudaGetLastError();
}

}  // namespace rt
