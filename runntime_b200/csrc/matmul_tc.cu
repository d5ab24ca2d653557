// Tensor-core matmul for the projections of a prefill (f16, more than 16 rows):
// out [M, N] = act(a [M, K] * b [K, N] + bias) + addend, f32 accumulation in tensor
// memory.  Same op as matmul.cu (packages/runntime/src/core/graph/ops/matmul.ts:28-99).
//
// One 128 x 128 output tile per CTA.  Warp 4 (one elected lane) streams K in steps of
// 64 through a three-stage ring of TMA loads: a 128 x 64 piece of a (K-major, 128-byte
// swizzle) and a 64 x 128 piece of b as two 64-column boxes (b is [K, N] row-major, that
// is MN-major for the MMA, the layout the V tiles of the attention kernels use).  Warp 5
// (one elected lane) issues four tcgen05.mma (M = 128, N = 128, K = 16) per stage into a
// 128-column accumulator and frees the stage by tcgen05.commit.  Warps 0-3 read the
// accumulator (one row per thread), apply bias, activation and addend, and store.
// Rows, columns and K past the matrices are zero-filled by TMA and never stored.
// Every wait is bounded (sm100.cuh).  Two CTAs share an SM (97 KB of shared memory and
// 128 tensor-memory columns each), so that one's start-up and read-out overlap the
// other's K loop.
#include "common.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace rt {
namespace {

using namespace sm100;
using namespace tc;

constexpr int GBM = 128, GBN = 128, GBK = 64, GSTAGES = 3;   // 97 KB of shared memory: two CTAs per SM
constexpr int kABytes = GBM * GBK * 2, kBBytes = GBK * GBN * 2, kStageBytes = kABytes + kBBytes;
constexpr int kGemmSmem = GSTAGES * kStageBytes + 1024;
constexpr int kGemmThreads = 192;

__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
               const __half* __restrict__ bias, const __half* __restrict__ addend,
               __half* __restrict__ out, int64_t M, int64_t K, int64_t N, int act, int* status) {
  extern __shared__ unsigned char smemRaw[];
  __shared__ __align__(8) uint64_t sFull[GSTAGES], sEmpty[GSTAGES], sAcc;
  __shared__ uint32_t sTmemBase;
  __shared__ int sAbort;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  TC_TRACE_DECL
  TC_TRACE(0, 0);
  const uint32_t smemBase = (smem_u32(smemRaw) + 1023u) & ~1023u;
  const int64_t row0 = (int64_t)blockIdx.y * GBM, col0 = (int64_t)blockIdx.x * GBN;
  const int nk = (int)((K + GBK - 1) / GBK);

  if (tid == 0) {
    sAbort = 0;
    for (int s = 0; s < GSTAGES; s++) {
      mbar_init(smem_u32(&sFull[s]), 1);
      mbar_init(smem_u32(&sEmpty[s]), 1);
    }
    mbar_init(smem_u32(&sAcc), 1);
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sTmemBase), GBN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sTmemBase;
  TC_TRACE(1, 0);

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      prefetch_tensormap(&mapA);
      prefetch_tensormap(&mapB);
      for (int it = 0; it < nk; it++) {
        const int s = it % GSTAGES;
        if (it >= GSTAGES && !mbar_wait(smem_u32(&sEmpty[s]), ((it / GSTAGES) - 1) & 1, &sAbort))
          break;
        const uint32_t bar = smem_u32(&sFull[s]);
        const uint32_t dA = smemBase + s * kStageBytes, dB = dA + kABytes;
        mbar_expect_tx(bar, kStageBytes);
        tma_load_2d(dA, &mapA, it * GBK, (int)row0, bar);                  // 64 k x 128 rows
        tma_load_2d(dB, &mapB, (int)col0, it * GBK, bar);                  // 64 cols x 64 k
        tma_load_2d(dB + GBK * 128, &mapB, (int)col0 + 64, it * GBK, bar);
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer --------------------------------
    constexpr uint32_t idesc = instr_desc(GBN, true);
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version, SW128
    constexpr uint32_t kLboA = (16u >> 4) << 16;                          // K-major operand
    constexpr uint32_t kLboB = ((uint32_t)(GBK * 128) >> 4) << 16;        // MN-major: next 64 columns
    bool ok = true;
    for (int it = 0; it < nk && ok; it++) {
      const int s = it % GSTAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sFull[s]), (it / GSTAGES) & 1, &sAbort)) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      TC_TRACE(2, it);
      if (elect_one()) {
        const uint32_t aLo = ((smemBase + s * kStageBytes) >> 4) | kLboA;
        const uint32_t bLo = ((smemBase + s * kStageBytes + kABytes) >> 4) | kLboB;
#pragma unroll
        for (int kk = 0; kk < GBK / 16; kk++) {
          const uint64_t aDesc = ((uint64_t)kDescHi << 32) | (aLo + kk * 2);
          const uint64_t bDesc = ((uint64_t)kDescHi << 32) | (bLo + kk * (2048 >> 4));
          mma_f16_ss(tmem, aDesc, bDesc, idesc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&sEmpty[s]));
        if (it == nk - 1) tc_commit(smem_u32(&sAcc));
      }
      __syncwarp();
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sAcc), 0, &sAbort)) != 0;
    TC_TRACE(4, 0);
    if (ok) {
      tc_fence_after_sync();
      const int64_t row = row0 + tid;  // thread = accumulator lane = output row
      const uint32_t laneBase = (uint32_t)(warp * 32) << 16;
#pragma unroll
      for (int c = 0; c < GBN; c += 32) {
        uint32_t acc[32];
        tmem_ld32(tmem + laneBase + c, acc);
        tmem_wait_ld();
        if (row < M) {
          const int64_t nc = col0 + c;             // first column of this 32-column piece
          uint4 pk[4];
          __half* h = reinterpret_cast<__half*>(pk);
          act_dispatch(act, [&](auto code) {
#pragma unroll
            for (int x = 0; x < 32; x++) {
              float y = __uint_as_float(acc[x]);
              const int64_t n = nc + x;
              if (bias && n < N) y += __half2float(bias[n]);
              y = act_apply<decltype(code)::value>(y);
              if (addend && n < N) y += __half2float(addend[row * N + n]);
              h[x] = __float2half_rn(y);
            }
          });
          __half* dst = out + row * N + nc;
          if (nc + 32 <= N) {
#pragma unroll
            for (int v = 0; v < 4; v++) reinterpret_cast<uint4*>(dst)[v] = pk[v];
          } else {
            for (int x = 0; x < 32 && nc + x < N; x++) dst[x] = h[x];
          }
        }
      }
    }
  }

  TC_TRACE(5, 0);
  tc_fence_before_sync();
  __syncthreads();
  TC_TRACE(6, 0);
  if (tid == 0 && sAbort) atomicOr(status, kStatusWaitTimeout);
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, GBN);
  }
  TC_TRACE(7, 0);
}

}  // namespace

// f16, more rows than the skinny kernel takes, whole 16-byte row pitches, at least one
// box of every operand.
bool matmul_tc_supported(const void* a, const void* b, const void* out, int64_t M, int64_t K,
                         int64_t N, int dtype) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  return dtype == RT_F16 && M > 16 && K >= 64 && N >= 64 && K % 8 == 0 && N % 8 == 0 && al(a) &&
         al(b) && al(out) && M < (1ll << 31) - 256 && N < (1ll << 31) - 256 &&
         K < (1ll << 31) - 256 && (M + GBM - 1) / GBM <= 65535 && encode_fn() != nullptr;
}

cudaError_t launch_matmul_tc(const void* a, const void* b, const void* bias, const void* addend,
                             void* out, int64_t M, int64_t K, int64_t N, int act, int* status,
                             cudaStream_t s, std::string* err) {
  CUtensorMap ma, mb;
  if (!make_map(&ma, a, M, K, K, GBM, err) || !make_map(&mb, b, K, N, N, GBK, err))
    return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kGemmSmem);
  if (e != cudaSuccess) return e;
  const dim3 grid((unsigned)((N + GBN - 1) / GBN), (unsigned)((M + GBM - 1) / GBM));
  gemm_tc_kernel<<<grid, kGemmThreads, kGemmSmem, s>>>(
      ma, mb, static_cast<const __half*>(bias), static_cast<const __half*>(addend),
      static_cast<__half*>(out), M, K, N, act, status);
  return cudaGetLastError();
}

}  // namespace rt
