// Row-wise softmax over the last dim, optionally masked by a [start, end) key
// range per row and a window around the diagonal: the probabilities of the
// matmul-attention path that callers keep beside the fused 'attn' op
// (packages/runntime/src/core/graph/ops/reduce.ts:12-39; kernel
// packages/runntime/src/core/kernels/reduce/softmax.ts:111-186).
//
// HBM-bound: one read and one write of the scores.  A row is handled by one
// warp (rows up to kWarpRowCols wide, eight rows per CTA) or by one CTA; the
// first pass keeps a running (max, sum) per thread, the second re-reads the row
// (it is in L1/L2 by then) and writes exp(x - max) / sum.  Four elements per
// access when the width is a multiple of four and the rows are aligned.
#include "common.cuh"

namespace rt {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpRowCols = 2048;
constexpr float kNegMax = -3.402823466e38f;

template <typename T>
struct Quad;
template <>
struct Quad<float> {
  using type = float4;
  static __device__ __forceinline__ void unpack(const float4& v, float (&f)[4]) {
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
  }
  static __device__ __forceinline__ float4 pack(const float (&f)[4]) {
    return make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <>
struct Quad<__half> {
  using type = uint2;
  static __device__ __forceinline__ void unpack(const uint2& v, float (&f)[4]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
    f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
  }
  static __device__ __forceinline__ uint2 pack(const float (&f)[4]) {
    uint2 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
    h[0] = __floats2half2_rn(f[0], f[1]);
    h[1] = __floats2half2_rn(f[2], f[3]);
    return v;
  }
};

__device__ __forceinline__ void fold(float& m, float& s, float v) {
  const float mNew = fmaxf(m, v);
  s = s * __expf(m - mNew) + __expf(v - mNew);
  m = mNew;
}

__device__ __forceinline__ void combine(float& m, float& s, float m2, float s2) {
  const float mNew = fmaxf(m, m2);
  s = s * __expf(m - mNew) + s2 * __expf(m2 - mNew);
  m = mNew;
}

// WARP: one warp per row, else one CTA per row.  VEC4: four elements per access.
template <typename T, bool WARP, bool VEC4>
__global__ void __launch_bounds__(kThreads)
softmax_kernel(const T* __restrict__ x, T* __restrict__ out, const float* __restrict__ segs,
               int64_t rows, int64_t cols, int64_t wl, int64_t wr) {
  using Q = Quad<T>;
  using QV = typename Q::type;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = WARP ? (int64_t)blockIdx.x * (kThreads / 32) + warp : (int64_t)blockIdx.x;
  if (row >= rows) return;  // uniform per warp (WARP) or per CTA
  const int t = WARP ? lane : threadIdx.x;
  const int span = WARP ? 32 : kThreads;

  // Kept columns [lo, hi).
  int64_t lo = 0, hi = cols;
  if (segs) {
    const int64_t s0 = (int64_t)segs[2 * row], s1 = (int64_t)segs[2 * row + 1];
    lo = max(s0, row - min(row, wl));
    hi = min(s1, row + min(cols - row, wr + 1));
  }

  const T* xr = x + row * cols;
  T* orow = out + row * cols;
  float m = kNegMax, s = 0.f;
  // Quads of columns [q0, q1) touch the kept range; only the first and the last of them
  // can hold masked columns (32-bit column arithmetic: the launcher takes this path only for
  // rows shorter than 2^31).
  const int lo32 = (int)lo, hi32 = (int)hi;
  const int q0 = lo32 >> 2, q1 = hi32 > lo32 ? (hi32 + 3) >> 2 : q0;
  if (VEC4) {
    const QV* xq = reinterpret_cast<const QV*>(xr);
    for (int i = q0 + t; i < q1; i += span) {
      float f[4];
      Q::unpack(xq[i], f);
      const int j = i * 4;
      const bool inner = j >= lo32 && j + 4 <= hi32;
      if (!inner) {
#pragma unroll
        for (int e = 0; e < 4; e++)
          if (j + e < lo32 || j + e >= hi32) f[e] = kNegMax;
      }
      // one running-sum rescale per quad instead of per element: five exponentials for four columns
      const float mNew = fmaxf(m, fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3])));
      float add = 0.f;
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float pe = __expf(f[e] - mNew);
        add += (inner || (j + e >= lo32 && j + e < hi32)) ? pe : 0.f;
      }
      s = s * __expf(m - mNew) + add;
      m = mNew;
    }
  } else {
    for (int64_t j = lo + t; j < hi; j += span) fold(m, s, to_f32<T>(xr[j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    combine(m, s, __shfl_xor_sync(0xffffffffu, m, o), __shfl_xor_sync(0xffffffffu, s, o));
  if (!WARP) {
    __shared__ float sM[kThreads / 32], sS[kThreads / 32];
    if (lane == 0) sM[warp] = m, sS[warp] = s;
    __syncthreads();
    m = sM[0], s = sS[0];
#pragma unroll
    for (int w = 1; w < kThreads / 32; w++) combine(m, s, sM[w], sS[w]);
  }
  const float inv = s > 0.f ? 1.f / s : 0.f;

  if (VEC4) {
    const QV* xq = reinterpret_cast<const QV*>(xr);
    QV* oq = reinterpret_cast<QV*>(orow);
    const int nq = (int)(cols >> 2);
    // zeros either side of the kept range: stores only
    const float z4[4] = {0.f, 0.f, 0.f, 0.f};
    const QV zero = Q::pack(z4);
#pragma unroll 4
    for (int i = t; i < q0; i += span) oq[i] = zero;
#pragma unroll 4
    for (int i = q1 + t; i < nq; i += span) oq[i] = zero;
    for (int i = q0 + t; i < q1; i += span) {
      float f[4];
      Q::unpack(xq[i], f);
      const int j = i * 4;
      if (j >= lo32 && j + 4 <= hi32) {
#pragma unroll
        for (int e = 0; e < 4; e++) f[e] = __expf(f[e] - m) * inv;
      } else {
#pragma unroll
        for (int e = 0; e < 4; e++)
          f[e] = (j + e >= lo32 && j + e < hi32) ? __expf(f[e] - m) * inv : 0.f;
      }
      oq[i] = Q::pack(f);
    }
  } else {
    for (int64_t j = t; j < cols; j += span) {
      float pr = 0.f;
      if (j >= lo && j < hi) pr = __expf(to_f32<T>(xr[j]) - m) * inv;
      orow[j] = from_f32<T>(pr);
    }
  }
}

template <typename T>
cudaError_t softmax_typed(const void* x, void* out, const float* segs, int64_t rows, int64_t cols,
                          int64_t wl, int64_t wr, cudaStream_t s) {
  auto* xi = static_cast<const T*>(x);
  auto* oi = static_cast<T*>(out);
  const uintptr_t quad = 4 * sizeof(T);
  const bool vec4 = cols % 4 == 0 && cols < (1ll << 31) - 8 && reinterpret_cast<uintptr_t>(x) % quad == 0 &&
                    reinterpret_cast<uintptr_t>(out) % quad == 0;
  const bool warpRows = cols <= kWarpRowCols;
  const int64_t blocks = warpRows ? (rows + kThreads / 32 - 1) / (kThreads / 32) : rows;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  const unsigned g = (unsigned)blocks;
  if (warpRows) {
    if (vec4) softmax_kernel<T, true, true><<<g, kThreads, 0, s>>>(xi, oi, segs, rows, cols, wl, wr);
    else softmax_kernel<T, true, false><<<g, kThreads, 0, s>>>(xi, oi, segs, rows, cols, wl, wr);
  } else {
    if (vec4) softmax_kernel<T, false, true><<<g, kThreads, 0, s>>>(xi, oi, segs, rows, cols, wl, wr);
    else softmax_kernel<T, false, false><<<g, kThreads, 0, s>>>(xi, oi, segs, rows, cols, wl, wr);
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_softmax(const void* x, void* out, const float* segs, int64_t rows, int64_t cols,
                           int64_t wl, int64_t wr, int dtype, cudaStream_t s) {
  return dtype == RT_F16 ? softmax_typed<__half>(x, out, segs, rows, cols, wl, wr, s)
                         : softmax_typed<float>(x, out, segs, rows, cols, wl, wr, s);
}

}  // namespace rt
