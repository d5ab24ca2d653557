// Local attention over a fused qkv slab [T, 3*heads*headDim]: query t of each
// head sees keys t-window+1 .. t (window <= 32), nothing ahead.  The score of
// the key j rows back is
//     cap * tanh( sum_d (q_d * qScale_d) * (k_d * kScale + rel[j][d]) / cap ),
// then softmax over the keys and the weighted sum of their values
// (packages/runntime/src/core/kernels/attention/attnLocal.ts:58-123; op
// packages/runntime/src/core/graph/ops/attention.ts:255-300).
//
// One warp per (row, head), eight per CTA.  Each lane owns four-element words of
// the head: it keeps its share of q * qScale in registers (heads up to 512 wide,
// re-read beyond), adds its share of every distance's dot product, and the
// `window` partial sums are then reduced across the warp together.  K, V and the
// bias rows are read with 8- or 16-byte accesses; every K/V row is re-read by the
// `window` queries that see it, which L1/L2 absorb (the window's rows are
// adjacent), so HBM sees the slab once and the output once.
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

}  // namespace

cudaError_t launch_local_attn(const void* qkv, const float* rel, const float* qScale, void* out,
                              int64_t rows, int heads, int hd, int window, float kScale,
                              float softcap, int dtype, cudaStream_t s) {
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
