// Small kernels beside attention: the standalone KV-cache append (writeRows)
// and the cross-device merge of (m, l, acc) partials.
#include "common.cuh"

namespace rt {
namespace {

// dst[offset + i] = src[i]; packages/runntime/src/core/kernels/shape/rows.ts:143-162.
// Bytes are copied 16 at a time when the three of offset, size and pointers allow.
template <typename V>
__global__ void write_rows_kernel(V* __restrict__ dst, const V* __restrict__ src, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = src[i];
}

// One warp per unit (one query head of one sequence): M = max m_p,
// L = sum l_p e^(m_p - M), o = sum acc_p e^(m_p - M) / L — the algebra of
// packages/runntime/src/core/kernels/attention/attnDecode.ts:405-422.
template <typename T>
__global__ void merge_partials_kernel(const float* __restrict__ partials, int parts,
                                      int64_t units, int hd, T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (u >= units) return;
  const int64_t stride = 2 + hd;
  float M = kNegSeed;
  for (int p = lane; p < parts; p += 32) M = fmaxf(M, partials[((int64_t)p * units + u) * stride]);
  M = warp_max(M);
  float L = 0.f;
  for (int p = lane; p < parts; p += 32) {
    const float* r = partials + ((int64_t)p * units + u) * stride;
    L += r[1] * __expf(r[0] - M);
  }
  L = warp_sum(L);
  const float invL = L > 0.f ? 1.f / L : 0.f;
  for (int x = lane; x < hd; x += 32) {
    float o = 0.f;
    for (int p = 0; p < parts; p++) {
      const float* r = partials + ((int64_t)p * units + u) * stride;
      o = fmaf(r[2 + x], __expf(r[0] - M), o);
    }
    out[u * hd + x] = from_f32<T>(o * invL);
  }
}

}  // namespace

cudaError_t launch_write_rows(void* dst, const void* src, int64_t dstOffsetBytes, int64_t bytes,
                              cudaStream_t s) {
  if (bytes <= 0) return cudaSuccess;
  char* d = static_cast<char*>(dst) + dstOffsetBytes;
  const uintptr_t mis = reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(src) |
                        (uintptr_t)bytes;
  const int threads = 256;
  auto blocks = [&](int64_t n) {
    int64_t b = (n + threads - 1) / threads;
    return (unsigned)(b > 148 * 16 ? 148 * 16 : b);
  };
  if ((mis & 15) == 0) {
    const int64_t n = bytes / 16;
    write_rows_kernel<uint4><<<blocks(n), threads, 0, s>>>(reinterpret_cast<uint4*>(d),
                                                          static_cast<const uint4*>(src), n);
  } else if ((mis & 3) == 0) {
    const int64_t n = bytes / 4;
    write_rows_kernel<uint32_t><<<blocks(n), threads, 0, s>>>(
        reinterpret_cast<uint32_t*>(d), static_cast<const uint32_t*>(src), n);
  } else {
    const int64_t n = bytes / 2;  // element sizes are 2 or 4, so bytes is even
    write_rows_kernel<uint16_t><<<blocks(n), threads, 0, s>>>(
        reinterpret_cast<uint16_t*>(d), static_cast<const uint16_t*>(src), n);
  }
  return cudaGetLastError();
}

cudaError_t launch_merge_partials(const float* partials, int parts, int64_t units, int hd,
                                  void* out, int dtype, cudaStream_t s) {
  const int warps = 8;
  const unsigned grid = (unsigned)((units + warps - 1) / warps);
  if (dtype == RT_F16)
    merge_partials_kernel<__half><<<grid, warps * 32, 0, s>>>(partials, parts, units, hd,
                                                               static_cast<__half*>(out));
  else
    merge_partials_kernel<float><<<grid, warps * 32, 0, s>>>(partials, parts, units, hd,
                                                              static_cast<float*>(out));
  return cudaGetLastError();
}

}  // namespace rt
