// Pieces shared by the tensor-core prefill kernels: TMEM load/store wrappers,
// packed-fp32 helpers, tcgen05 descriptors and the host-side TMA tensor maps.
#pragma once

#include <cudaTypedefs.h>

#include <mutex>
#include <string>

#include "common.cuh"
#include "sm100.cuh"

namespace rt {
namespace tc {

// Optional timeline instrumentation for kernel development (off unless the
// translation unit is compiled with RT_TC_TRACE): lane 0 of every warp of CTA
// (0,0) stores (clock, tag, index) records into its own slice of a device buffer
// (plain stores, no atomics, so the timeline is barely disturbed).
#ifdef RT_TC_TRACE
#ifndef RT_TC_TRACE_X0
#define RT_TC_TRACE_X0 0u   // first of the two traced CTAs (blockIdx.x; blockIdx.y is 0)
#endif
constexpr int kTraceWarps = 32, kTracePerWarp = 1024;
__device__ long long gTraceBuf[kTraceWarps * kTracePerWarp * 2];
#define TC_TRACE_DECL int traceSeq_ = 0;
// CTAs (X0,0) and (X0+1,0): the second one's warps use slots 16 and up.
#define TC_TRACE(tag, idx)                                                                  \
  do {                                                                                      \
    if (blockIdx.x - RT_TC_TRACE_X0 <= 1u && blockIdx.y == 0 && (threadIdx.x & 31) == 0 &&  \
        traceSeq_ < kTracePerWarp) {                                                        \
      long long* r_ = gTraceBuf + (((blockIdx.x - RT_TC_TRACE_X0) * 16 + (threadIdx.x >> 5)) * \
                                       kTracePerWarp + traceSeq_++) * 2;                     \
      r_[0] = clock64();                                                                    \
      r_[1] = (long long)(tag)*100000 + (idx) + 1;                                          \
    }                                                                                       \
  } while (0)
#else
#define TC_TRACE_DECL
#define TC_TRACE(tag, idx) \
  do {                     \
  } while (0)
#endif

constexpr int BM = 128;                   // query rows per MMA tile (= TMEM lanes)
// log2 units: the accumulator is rescaled when a row's maximum has grown this far past
// its reference point.  P = 2^(s - reference) is stored as f16, so 2^threshold must stay
// below 65504; f16 keeps its relative precision over that whole range.
#ifndef RT_RESCALE_THRESHOLD
#define RT_RESCALE_THRESHOLD 13
#endif
constexpr float kRescaleThreshold = (float)RT_RESCALE_THRESHOLD;

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(taddr)
      : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Packed fp32 pairs: two FMAs (adds) per instruction.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<const uint64_t*>(&a)), "l"(*reinterpret_cast<const uint64_t*>(&b)),
        "l"(*reinterpret_cast<const uint64_t*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<const uint64_t*>(&a)), "l"(*reinterpret_cast<const uint64_t*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}

// 2^x for a pair of values on the FMA pipe, no MUFU: split x into its nearest
// integer n (magic-number rounding) and f in [-0.5, 0.5], evaluate a degree-3
// polynomial for 2^f (max relative error 7.5e-5, below f16 resolution) and add n
// to the exponent field.  Inputs below -126 (masked scores are -inf) give 2^-126.
// The MUFU unit delivers 16 ex2 per clock per SM, which is exactly the tensor
// core's appetite for a 128-wide head; moving part of the exponentials here
// takes the special-function unit off the critical path.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  constexpr float kMagic = 12582912.f;  // 1.5 * 2^23
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 xr = add2(x, make_float2(kMagic, kMagic));
  const float2 n = add2(xr, make_float2(-kMagic, -kMagic));
  const float2 f = fma2(n, make_float2(-1.f, -1.f), x);
  float2 r = fma2(make_float2(0.055171649903059006f, 0.055171649903059006f), f,
                  make_float2(0.2426111251115799f, 0.2426111251115799f));
  r = fma2(r, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
  r = fma2(r, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
  r.x = __int_as_float(__float_as_int(r.x) + (__float_as_int(xr.x) << 23));
  r.y = __int_as_float(__float_as_int(r.y) + (__float_as_int(xr.y) << 23));
  return r;
}
// Of every kPolyDen consecutive score pairs, kPolyNum take the polynomial path.
#ifndef RT_POLY_NUM
#define RT_POLY_NUM 0
#endif
constexpr int kPolyNum = RT_POLY_NUM, kPolyDen = 8;
__device__ __forceinline__ float2 exp2_pair(float2 t, int pairIndex) {
  if (pairIndex % kPolyDen < kPolyNum) return exp2_poly2(t);
  return make_float2(sm100::fast_exp2(t.x), sm100::fast_exp2(t.y));
}

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version bit set.
// Offsets are in bytes; the hardware fields drop the 4 low bits.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lboBytes, uint32_t sboBytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3fff);
  d |= (uint64_t)((lboBytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sboBytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor, kind::f16: f16 A and B, f32 D, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool bMnMajor) {
  return (1u << 4)                       // D format f32
         | (0u << 7) | (0u << 10)        // A, B format f16
         | (0u << 15)                    // A K-major
         | ((bMnMajor ? 1u : 0u) << 16)  // B major
         | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ---- host side: TMA tensor maps -------------------------------------------------

inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// [rows, cols] f16 row-major with `strideElems` between rows; box = 64 columns x boxRows.
inline bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t strideElems,
              int boxRows, std::string* err) {
  auto fn = encode_fn();
  if (!fn) {
    *err = "cuTensorMapEncodeTiled is not available from the driver";
    return false;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)strideElems * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)boxRows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *err = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r);
    return false;
  }
  return true;
}

}  // namespace tc
}  // namespace rt
