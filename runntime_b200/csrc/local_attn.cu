// Local attention over a fused qkv slab [T, 3*heads*headDim]: query t of each
// head sees keys t-window+1 .. t (window <= 32), nothing ahead.  The score of
// the key j rows back is
//     cap * tanh( sum_d (q_d * qScale_d) * (k_d * kScale + rel[j][d]) / cap ),
// then softmax over the keys and the weighted sum of their values
// (packages/runntime/src/core/kernels/attention/attnLocal.ts:58-123; op
// packages/runntime/src/core/graph/ops/attention.ts:255-300).
//
// Tiled kernel (heads up to 512 wide): a CTA takes a run of consecutive rows of
// one head and stages their K and V rows, the window-1 rows before them and the
// head's bias rows in shared memory once, so every K/V row leaves L2 once per
// CTA instead of once per query that sees it (window times).  One warp per row
// inside the tile: each lane owns four-element words of the head, keeps its
// share of q * qScale in registers, adds its share of every distance's dot
// product from shared memory, and the partial sums are reduced across the warp.
// HBM-bound: the slab is read once (plus (window-1)/tileRows of K and V again at
// tile seams) and the output written once.
//
// Row kernel (any head width): one warp per (row, head), operands straight from
// global memory; every K/V row is re-read by the `window` queries that see it,
// which L1/L2 absorb.  Used when a tile would not fit shared memory.
#include <type_traits>
#include "common.cuh"

namespace rt {
namespace {

constexpr int kMaxWindow = 32;
constexpr int kWarps = 8;
constexpr int kRegWords = 4;  // words of q kept per lane: heads up to 4*32*4 = 512 wide

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__half>(const __half* p) {
  const uint2 w = *reinterpret_cast<const uint2*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&w);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 v) {
  *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* p, float4 v) {
  uint2 w;
  __half2* h = reinterpret_cast<__half2*>(&w);
  h[0] = __floats2half2_rn(v.x, v.y);
  h[1] = __floats2half2_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = w;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
local_attn_kernel(const T* __restrict__ qkv, const float* __restrict__ rel,
                  const float* __restrict__ qScale, T* __restrict__ out, int64_t rows, int heads,
                  int hd, int window, float kScale, float softcap) {
  const int lane = threadIdx.x & 31;
  const int64_t g = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
  if (g >= rows * heads) return;  // uniform per warp
  const int64_t t = g / heads;
  const int h = (int)(g - t * heads);
  const int words = hd >> 2;
  const int64_t width = (int64_t)heads * hd, rowElems = 3 * width;
  const int n = (int)min((int64_t)window, t + 1);  // key t-j exists for j <= t

  const T* qp = qkv + t * rowElems + (int64_t)h * hd;
  float4 qreg[kRegWords];
#pragma unroll
  for (int i = 0; i < kRegWords; i++) {
    const int w = lane + 32 * i;
    qreg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (w < words) {
      const float4 q = load4<T>(qp + 4 * w), sc = load4<float>(qScale + 4 * w);
      qreg[i] = make_float4(q.x * sc.x, q.y * sc.y, q.z * sc.z, q.w * sc.w);
    }
  }

  // This lane's share of every distance's dot product.
  float part[kMaxWindow];
#pragma unroll
  for (int j = 0; j < kMaxWindow; j++) {
    part[j] = 0.f;
    if (j < n) {
      const T* kp = qkv + (t - j) * rowElems + width + (int64_t)h * hd;
      const float* rp = rel + (int64_t)j * width + (int64_t)h * hd;
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < kRegWords; i++) {
        const int w = lane + 32 * i;
        if (w < words) {
          const float4 k = load4<T>(kp + 4 * w), r = load4<float>(rp + 4 * w);
          const float4 q = qreg[i];
          s = fmaf(q.x, fmaf(k.x, kScale, r.x), s);
          s = fmaf(q.y, fmaf(k.y, kScale, r.y), s);
          s = fmaf(q.z, fmaf(k.z, kScale, r.z), s);
          s = fmaf(q.w, fmaf(k.w, kScale, r.w), s);
        }
      }
      for (int w = lane + 32 * kRegWords; w < words; w += 32) {  // heads wider than 512
        const float4 q = load4<T>(qp + 4 * w), sc = load4<float>(qScale + 4 * w);
        const float4 k = load4<T>(kp + 4 * w), r = load4<float>(rp + 4 * w);
        s = fmaf(q.x * sc.x, fmaf(k.x, kScale, r.x), s);
        s = fmaf(q.y * sc.y, fmaf(k.y, kScale, r.y), s);
        s = fmaf(q.z * sc.z, fmaf(k.z, kScale, r.z), s);
        s = fmaf(q.w * sc.w, fmaf(k.w, kScale, r.w), s);
      }
      part[j] = s;
    }
  }
  // Reduce across the warp; every lane ends with every score.
  float m = -3.402823466e38f;
#pragma unroll
  for (int j = 0; j < kMaxWindow; j++) {
    if (j < n) {  // n is uniform across the warp
      float s = part[j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      s = softcap * tanhf(s / softcap);
      part[j] = s;
      m = fmaxf(m, s);
    }
  }
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxWindow; j++) {
    if (j < n) {
      part[j] = expf(part[j] - m);
      sum += part[j];
    }
  }
  const float inv = 1.f / sum;  // distance 0 always exists, so sum >= 1

  T* op = out + t * width + (int64_t)h * hd;
  for (int w = lane; w < words; w += 32) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < kMaxWindow; j++) {
      if (j < n) {
        const float4 v = load4<T>(qkv + (t - j) * rowElems + 2 * width + (int64_t)h * hd + 4 * w);
        acc.x = fmaf(part[j], v.x, acc.x);
        acc.y = fmaf(part[j], v.y, acc.y);
        acc.z = fmaf(part[j], v.z, acc.z);
        acc.w = fmaf(part[j], v.w, acc.w);
      }
    }
    store4<T>(op + 4 * w, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
  }
}

// ---- tiled kernel ------------------------------------------------------------------
constexpr int kTileThreads = 256;

template <typename T, int WMAX>
__global__ void __launch_bounds__(kTileThreads)
local_attn_tiled_kernel(const T* __restrict__ qkv, const float* __restrict__ rel,
                        const float* __restrict__ qScale, T* __restrict__ out, int64_t rows,
                        int heads, int hd, int window, int tileRows, float kScale, float softcap) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * tileRows;            // first query row of the tile
  const int64_t first = t0 - (window - 1) > 0 ? t0 - (window - 1) : 0;  // first staged key row
  const int nq = (int)min((int64_t)tileRows, rows - t0);
  const int staged = (int)(t0 + nq - first);
  const int words = hd >> 2;
  const int64_t width = (int64_t)heads * hd, rowElems = 3 * width;
  const int maxStaged = tileRows + window - 1;
  T* sK = reinterpret_cast<T*>(smem);
  T* sV = sK + (size_t)maxStaged * hd;
  float* sRel = reinterpret_cast<float*>(sV + (size_t)maxStaged * hd);

  // Stage K and V rows [first, first + staged) of this head and the head's bias rows.
  for (int i = threadIdx.x; i < staged * words; i += kTileThreads) {
    const int r = i / words, w = i - r * words;
    const T* src = qkv + (first + r) * rowElems + width + (int64_t)h * hd + 4 * w;
    using Word = typename std::conditional<sizeof(T) == 2, uint2, uint4>::type;
    *reinterpret_cast<Word*>(sK + (size_t)r * hd + 4 * w) = *reinterpret_cast<const Word*>(src);
    *reinterpret_cast<Word*>(sV + (size_t)r * hd + 4 * w) = *reinterpret_cast<const Word*>(src + width);
  }
  for (int i = threadIdx.x; i < window * words; i += kTileThreads) {
    const int j = i / words, w = i - j * words;
    *reinterpret_cast<float4*>(sRel + (size_t)j * hd + 4 * w) =
        *reinterpret_cast<const float4*>(rel + (int64_t)j * width + (int64_t)h * hd + 4 * w);
  }
  __syncthreads();

  for (int r = warp; r < nq; r += kTileThreads / 32) {
    const int64_t t = t0 + r;
    const int n = (int)min((int64_t)window, t + 1);
    const int kr = (int)(t - first);  // staged index of key t
    const T* qp = qkv + t * rowElems + (int64_t)h * hd;
    float4 qreg[kRegWords];
#pragma unroll
    for (int i = 0; i < kRegWords; i++) {
      const int w = lane + 32 * i;
      qreg[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (w < words) {
        const float4 q = load4<T>(qp + 4 * w), sc = load4<float>(qScale + 4 * w);
        qreg[i] = make_float4(q.x * sc.x, q.y * sc.y, q.z * sc.z, q.w * sc.w);
      }
    }
    // Lane j ends up with the score of distance j: every lane adds its share of each
    // dot product, the shares are summed across the warp, and lane j keeps sum j.
    float mine = 0.f;
#pragma unroll
    for (int j = 0; j < WMAX; j++) {
      if (j < n) {
        const T* kp = sK + (size_t)(kr - j) * hd;
        const float* rp = sRel + (size_t)j * hd;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < kRegWords; i++) {
          const int w = lane + 32 * i;
          if (w < words) {
            const float4 k = load4<T>(kp + 4 * w), rl = load4<float>(rp + 4 * w);
            const float4 q = qreg[i];
            s = fmaf(q.x, fmaf(k.x, kScale, rl.x), s);
            s = fmaf(q.y, fmaf(k.y, kScale, rl.y), s);
            s = fmaf(q.z, fmaf(k.z, kScale, rl.z), s);
            s = fmaf(q.w, fmaf(k.w, kScale, rl.w), s);
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == j) mine = s;
      }
    }
    // Softcap, softmax: one tanh and one exp per lane instead of `window` of each.
    const float sc = lane < n ? softcap * tanhf(mine / softcap) : -3.402823466e38f;
    float m = sc;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float pr = lane < n ? expf(sc - m) : 0.f;
    float sum = pr;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float pn = pr / sum;  // distance 0 always exists, so sum >= 1
    T* op = out + t * width + (int64_t)h * hd;
    float4 acc[kRegWords];
#pragma unroll
    for (int i = 0; i < kRegWords; i++) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < WMAX; j++) {
      if (j < n) {
        const float pj = __shfl_sync(0xffffffffu, pn, j);
        const T* vp = sV + (size_t)(kr - j) * hd;
#pragma unroll
        for (int i = 0; i < kRegWords; i++) {
          const int w = lane + 32 * i;
          if (w < words) {
            const float4 v = load4<T>(vp + 4 * w);
            acc[i].x = fmaf(pj, v.x, acc[i].x);
            acc[i].y = fmaf(pj, v.y, acc[i].y);
            acc[i].z = fmaf(pj, v.z, acc[i].z);
            acc[i].w = fmaf(pj, v.w, acc[i].w);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kRegWords; i++) {
      const int w = lane + 32 * i;
      if (w < words) store4<T>(op + 4 * w, acc[i]);
    }
  }
}

// Rows per tile: the largest tile whose K, V and bias rows fit 28 KB, so that eight CTAs
// (all 64 warps) share an SM — the kernel is a chain of dependent shuffles and small
// shared-memory loads per row, which only occupancy hides; else the largest tile within
// `budget`; 0 if not even 8 rows fit.
int tile_rows_for(int hd, int window, int esize, size_t budget) {
  const size_t relBytes = (size_t)window * hd * 4;
  auto need = [&](int tr) { return 2 * (size_t)(tr + window - 1) * hd * esize + relBytes; };
  for (int tr : {64, 32, 16}) if (need(tr) <= 28 * 1024) return tr;
  for (int tr : {64, 32, 16, 8}) if (need(tr) <= budget) return tr;
  return 0;
}

template <typename T>
cudaError_t launch_tiled(const void* qkv, const float* rel, const float* qScale, void* out,
                         int64_t rows, int heads, int hd, int window, int tileRows, float kScale,
                         float softcap, cudaStream_t s) {
  const size_t smemBytes = 2 * (size_t)(tileRows + window - 1) * hd * sizeof(T) +
                           (size_t)window * hd * 4;
  auto kern = window <= 16 ? local_attn_tiled_kernel<T, 16> : local_attn_tiled_kernel<T, 32>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smemBytes);
  if (e != cudaSuccess) return e;
  const dim3 grid((unsigned)((rows + tileRows - 1) / tileRows), (unsigned)heads);
  kern<<<grid, kTileThreads, smemBytes, s>>>(static_cast<const T*>(qkv), rel, qScale,
                                             static_cast<T*>(out), rows, heads, hd, window,
                                             tileRows, kScale, softcap);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_local_attn(const void* qkv, const float* rel, const float* qScale, void* out,
                              int64_t rows, int heads, int hd, int window, float kScale,
                              float softcap, int dtype, cudaStream_t s) {
  // The tiled kernel wants the head in registers (<= 512 wide), a grid within the
  // y limit and a tile that fits shared memory beside a second resident CTA.
  const int esize = dtype == RT_F16 ? 2 : 4;
  const int tileRows = (hd <= 128 * kRegWords && heads <= 65535)
                           ? tile_rows_for(hd, window, esize, 100 * 1024) : 0;
  if (tileRows > 0 && (rows + tileRows - 1) / tileRows <= 0x7fffffffll) {
    return dtype == RT_F16
               ? launch_tiled<__half>(qkv, rel, qScale, out, rows, heads, hd, window, tileRows,
                                      kScale, softcap, s)
               : launch_tiled<float>(qkv, rel, qScale, out, rows, heads, hd, window, tileRows,
                                     kScale, softcap, s);
  }
  const int64_t blocks = (rows * heads + kWarps - 1) / kWarps;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  if (dtype == RT_F16)
    local_attn_kernel<__half><<<(unsigned)blocks, kWarps * 32, 0, s>>>(
        static_cast<const __half*>(qkv), rel, qScale, static_cast<__half*>(out), rows, heads, hd,
        window, kScale, softcap);
  else
    local_attn_kernel<float><<<(unsigned)blocks, kWarps * 32, 0, s>>>(
        static_cast<const float*>(qkv), rel, qScale, static_cast<float*>(out), rows, heads, hd,
        window, kScale, softcap);
  return cudaGetLastError();
}

}  // namespace rt
