// Small kernels beside attention: the standalone KV-cache append (writeRows),
// the rotary embedding that precedes it, and the cross-device merge of
// (m, l, acc) partials.
#include <type_traits>
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

// out[r, c] = x[rowStart + r, colStart + c] in units of V (1 to 16 bytes):
// packages/runntime/src/core/kernels/shape/columns.ts, rows.ts (sliceCols / sliceRows).
template <typename V>
__global__ void slice_kernel(V* __restrict__ out, const V* __restrict__ x, int64_t rows,
                             int64_t width, int64_t srcCols, int64_t srcOffset) {
  const int64_t total = rows * width;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / width, c = i - r * width;
    out[i] = x[srcOffset + r * srcCols + c];
  }
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

// Merge of the rows the ranks exchanged, on the rank that owns the sequences.  `buffer` is
// this rank's exchange buffer: two halves (by step parity) of [world][per * heads][2+hd],
// source rank p's rows for this rank's `per` sequences; the half of the step just computed
// is *step & 1 (the decode kernel's last block has moved *step before this kernel starts).
// Each block first waits until every rank's arrival word has reached *step: a rank
// publishes it after all of its rows for this owner have landed here.  The wait is bounded
// (`limit` polls, about a second by default), then the block records the failure in *status
// and writes zeros.  Output rows: sequences [firstSeq, firstSeq + owned) of `out`.
template <typename T>
__global__ void merge_exchanged_kernel(const float* __restrict__ buffer,
                                       const uint32_t* __restrict__ flags,
                                       const uint32_t* __restrict__ step, int world, int per,
                                       int owned, int firstSeq, int heads, int hd,
                                       T* __restrict__ out, int* status, int limit) {
  __shared__ int sOk;
  // A programmatic dependent of the decode kernel: resident early, reading nothing before
  // that grid has finished; the kernel after this one may be made resident at once.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(step);
  if (threadIdx.x == 0) sOk = 1;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    // An acquire load at system scope pairs with the peer's fence + release store: once the
    // word is seen, the rows stored before it are visible too.
    const uint32_t* f = flags + threadIdx.x;
    bool arrived = false;
    for (int i = 0; i < limit; i++) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
      // signed distance: a peer may already be a step ahead
      if ((int32_t)(seen - epoch) >= 0) { arrived = true; break; }
      __nanosleep(i < 64 ? 100 : 1000);
    }
    if (!arrived) sOk = 0;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t units = (int64_t)owned * heads;
  const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  T* dst = out + ((int64_t)firstSeq * heads + u) * hd;
  if (!sOk) {
    if (threadIdx.x == 0) atomicOr(status, kStatusWaitTimeout);
    if (u < units)
      for (int x = lane; x < hd; x += 32) dst[x] = from_f32<T>(0.f);
    return;
  }
  if (u >= units) return;
  const int64_t stride = 2 + hd;
  const int64_t slot = (int64_t)per * heads * stride;   // one source rank's rows
  const float* partials = buffer + (int64_t)(epoch & 1u) * world * slot + u * stride;
  // One round trip to memory: every load of the unit goes out before the first is used (the
  // rows came in through peer stores, so they are read from L2 or DRAM, and loads that wait
  // for one another would add a microsecond each).  Lane p holds rank p's (m, l); lane x
  // holds output columns x, x+32, ... of every rank's row.
  constexpr int kCols = 4;   // head sizes up to 128
  float mv = kNegSeed, lv = 0.f;
  if (lane < world) {
    mv = __ldcg(partials + lane * slot);
    lv = __ldcg(partials + lane * slot + 1);
  }
  float val[kCols][RT_MAX_PEERS];
#pragma unroll
  for (int c = 0; c < kCols; c++) {
    const int x = lane + 32 * c;
#pragma unroll
    for (int p = 0; p < RT_MAX_PEERS; p++)
      val[c][p] = (x < hd && p < world) ? __ldcg(partials + p * slot + 2 + x) : 0.f;
  }
  const float M = warp_max(mv);
  const float w = lane < world ? __expf(mv - M) : 0.f;
  const float L = warp_sum(lv * w);
  const float invL = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
  for (int c = 0; c < kCols; c++) {
    const int x = lane + 32 * c;
    float o = 0.f;
#pragma unroll
    for (int p = 0; p < RT_MAX_PEERS; p++) o = fmaf(val[c][p], __shfl_sync(0xffffffffu, w, p), o);
    if (x < hd) dst[x] = from_f32<T>(o * invL);
  }
}

// Rotary embedding, one thread per interleaved pair of a column window of x:
// (x0, x1) -> (x0 c - x1 s, x1 c + x0 s) with pair-duplicated f32 tables
// [rows, headDim]; packages/runntime/src/core/kernels/attention/rope.ts:36-70.
template <typename T> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<__half> { using type = __half2; };

// PAIRED: every pair of x and out sits on a pair-sized boundary (even row strides,
// aligned bases), so a pair moves as one 8- or 4-byte access.
template <typename T, bool PAIRED>
__global__ void rope_kernel(const T* __restrict__ x, const float* __restrict__ cosT,
                            const float* __restrict__ sinT, T* __restrict__ out, int64_t rows,
                            int64_t srcCols, int hd, int64_t srcStart, int64_t width) {
  using P = typename Pair<T>::type;
  const int64_t pairs = width / 2, total = rows * pairs;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / pairs, col0 = (i - row * pairs) * 2;
    const int dcol = (int)(col0 % hd);
    const float c = cosT[row * hd + dcol], s = sinT[row * hd + dcol];
    const T* src = x + row * srcCols + srcStart + col0;
    T* dst = out + row * width + col0;
    T a, b;
    if (PAIRED) {
      const P v = *reinterpret_cast<const P*>(src);
      a = v.x, b = v.y;
    } else {
      a = src[0], b = src[1];
    }
    const float x0 = to_f32<T>(a), x1 = to_f32<T>(b);
    float f0, f1;
    rope_pair(x0, x1, c, s, f0, f1);
    const T r0 = from_f32<T>(f0), r1 = from_f32<T>(f1);
    if (PAIRED) {
      P v;
      v.x = r0, v.y = r1;
      *reinterpret_cast<P*>(dst) = v;
    } else {
      dst[0] = r0, dst[1] = r1;
    }
  }
}

// Vector path: a thread takes one 16-byte (or, for heads like 36 and 52 halves wide,
// 8-byte) group of columns of a head for one row, loads the row's cos/sin for those columns once and
// walks over the heads of the window, so the tables cost one read per row and column
// group instead of one per element.  Needs headDim, srcStart, the row strides and the
// base addresses on boundaries of the group size.
template <typename T, int V>   // V elements (V*sizeof(T) = 16 or 8 bytes) per thread and access
__global__ void rope_vec_kernel(const T* __restrict__ x, const float* __restrict__ cosT,
                                const float* __restrict__ sinT, T* __restrict__ out, int64_t rows,
                                int64_t srcCols, int hd, int64_t srcStart, int64_t width) {
  using Word = typename std::conditional<V * sizeof(T) == 16, uint4, uint2>::type;
  const int groups = hd / V;
  const int nHeads = (int)(width / hd);
  const int64_t total = rows * groups;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / groups;
    const int c0 = (int)(i - row * groups) * V;
    float c[V / 2], sn[V / 2];
#pragma unroll
    for (int e = 0; e < V / 2; e += 2) {  // tables are pair-duplicated: entries 0, 2 of a float4
      const float4 cv = *reinterpret_cast<const float4*>(cosT + row * hd + c0 + 2 * e);
      const float4 sv = *reinterpret_cast<const float4*>(sinT + row * hd + c0 + 2 * e);
      c[e] = cv.x, c[e + 1] = cv.z, sn[e] = sv.x, sn[e + 1] = sv.z;
    }
    const T* src = x + row * srcCols + srcStart + c0;
    T* dst = out + row * width + c0;
    // Four heads per round, their loads issued together: one 16-byte load in flight per
    // thread does not cover the DRAM latency (measured 4.4 TB/s against 5.x with four).
    constexpr int U = 4;
    for (int h0 = 0; h0 < nHeads; h0 += U) {
      Word raw[U];
#pragma unroll
      for (int u = 0; u < U; u++)
        if (h0 + u < nHeads) raw[u] = *reinterpret_cast<const Word*>(src + (int64_t)(h0 + u) * hd);
#pragma unroll
      for (int u = 0; u < U; u++) {
        if (h0 + u < nHeads) {
          T* v = reinterpret_cast<T*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < V / 2; e++) {
            float r0, r1;
            rope_pair(to_f32<T>(v[2 * e]), to_f32<T>(v[2 * e + 1]), c[e], sn[e], r0, r1);
            v[2 * e] = from_f32<T>(r0), v[2 * e + 1] = from_f32<T>(r1);
          }
          *reinterpret_cast<Word*>(dst + (int64_t)(h0 + u) * hd) = raw[u];
        }
      }
    }
  }
}

template <typename T>
void rope_launch(const void* x, const float* cosT, const float* sinT, void* out, int64_t rows,
                 int64_t srcCols, int hd, int64_t srcStart, int64_t width, unsigned blocks,
                 cudaStream_t s) {
  const uintptr_t pairBytes = 2 * sizeof(T);
  const bool paired = (srcCols % 2 == 0) && (reinterpret_cast<uintptr_t>(x) % pairBytes == 0) &&
                      (reinterpret_cast<uintptr_t>(out) % pairBytes == 0);
  auto* xi = static_cast<const T*>(x);
  auto* oi = static_cast<T*>(out);
  const auto aligned = [&](int v) {
    const uintptr_t bytes = v * sizeof(T);
    return hd % v == 0 && hd % 4 == 0 && srcStart % v == 0 && srcCols % v == 0 && width % v == 0 &&
           reinterpret_cast<uintptr_t>(x) % bytes == 0 && reinterpret_cast<uintptr_t>(out) % bytes == 0 &&
           reinterpret_cast<uintptr_t>(cosT) % 16 == 0 && reinterpret_cast<uintptr_t>(sinT) % 16 == 0;
  };
  const auto vblocks = [&](int v) {
    const int64_t vb = (rows * (hd / v) + 255) / 256;
    return (unsigned)(vb > 148 * 32 ? 148 * 32 : vb);
  };
  constexpr int V16 = 16 / sizeof(T);
  if (aligned(V16)) {
    rope_vec_kernel<T, V16><<<vblocks(V16), 256, 0, s>>>(xi, cosT, sinT, oi, rows, srcCols, hd,
                                                         srcStart, width);
    return;
  }
  if (sizeof(T) == 2 && aligned(4)) {
    rope_vec_kernel<T, 4><<<vblocks(4), 256, 0, s>>>(xi, cosT, sinT, oi, rows, srcCols, hd,
                                                     srcStart, width);
    return;
  }
  if (paired)
    rope_kernel<T, true><<<blocks, 256, 0, s>>>(xi, cosT, sinT, oi, rows, srcCols, hd, srcStart, width);
  else
    rope_kernel<T, false><<<blocks, 256, 0, s>>>(xi, cosT, sinT, oi, rows, srcCols, hd, srcStart, width);
}

}  // namespace

cudaError_t launch_rope(const void* x, const float* cosT, const float* sinT, void* out,
                        int64_t rows, int64_t srcCols, int hd, int64_t srcStart, int64_t width,
                        int dtype, cudaStream_t s) {
  const int64_t total = rows * (width / 2);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == RT_F16)
    rope_launch<__half>(x, cosT, sinT, out, rows, srcCols, hd, srcStart, width, (unsigned)blocks, s);
  else
    rope_launch<float>(x, cosT, sinT, out, rows, srcCols, hd, srcStart, width, (unsigned)blocks, s);
  return cudaGetLastError();
}

cudaError_t launch_slice(const void* x, void* out, int64_t rows, int64_t srcColBytes,
                         int64_t offsetBytes, int64_t widthBytes, cudaStream_t s) {
  const uintptr_t mis = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out) |
                        (uintptr_t)srcColBytes | (uintptr_t)offsetBytes | (uintptr_t)widthBytes;
  auto run = [&](auto tag) {
    using V = decltype(tag);
    const int64_t u = sizeof(V), total = rows * (widthBytes / u);
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    slice_kernel<V><<<(unsigned)blocks, 256, 0, s>>>(static_cast<V*>(out), static_cast<const V*>(x),
                                                     rows, widthBytes / u, srcColBytes / u,
                                                     offsetBytes / u);
  };
  if ((mis & 15) == 0) run(uint4{});
  else if ((mis & 3) == 0) run(uint32_t{});
  else run(uint16_t{});
  return cudaGetLastError();
}

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

cudaError_t launch_merge_exchanged(const float* buffer, const uint32_t* flags, const uint32_t* step,
                                   int world, int per, int owned, int firstSeq, int heads, int hd,
                                   void* out, int dtype, int* status, int limit, cudaStream_t s) {
  if (owned <= 0) return cudaSuccess;   // this rank owns none of the sequences: nothing to merge
  const int warps = 8;
  const int64_t units = (int64_t)owned * heads;
  const unsigned grid = (unsigned)((units + warps - 1) / warps);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(warps * 32);
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (dtype == RT_F16)
    return cudaLaunchKernelEx(&cfg, merge_exchanged_kernel<__half>, buffer, flags, step, world, per, owned,
                              firstSeq, heads, hd, static_cast<__half*>(out), status, limit);
  return cudaLaunchKernelEx(&cfg, merge_exchanged_kernel<float>, buffer, flags, step, world, per, owned,
                            firstSeq, heads, hd, static_cast<float*>(out), status, limit);
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
