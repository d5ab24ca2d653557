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
  const int tid = threadIdx.x, warp = tid >> 5;
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
        const uint32_t aLo = (((smemBase + s * kStageBytes) >> 4) & 0x3fffu) | kLboA;
        const uint32_t bLo = (((smemBase + s * kStageBytes + kABytes) >> 4) & 0x3fffu) | kLboB;
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

// ---- up to 16 rows (the projections of a decode step) -------------------------------
// HBM-bound: the weights are read once, 2 K N bytes.  The product is computed
// transposed, out^T [N, M] = b^T [N, K] * a^T [K, M], so that 128 columns of the weights
// fill the 128 rows of one tcgen05.mma (A operand MN-major, exactly as TMA lays a
// [64 k, 64 columns] box of b down) and the few rows of a are its N = 16 side.  The
// tensor core is far from busy; it is here because it takes the weights straight from
// shared memory, where a SIMT kernel spends 64 FMAs per 16-byte load.
//
// One CTA owns 128 output columns and one slice of K; the slices of a column tile form
// a thread-block cluster (1, 2, 4 or 8 CTAs).  Each CTA streams its slice through a
// three-stage TMA ring into a 16-column accumulator; the CTAs of rank > 0 then write
// their accumulators into the shared memory of rank 0 (distributed shared memory),
// one hardware cluster barrier orders that, and rank 0 adds them, applies bias,
// activation and addend and stores.  One launch, no atomics, no scratch.
#ifndef RT_SK_STAGES
#define RT_SK_STAGES 3
#endif
#ifndef RT_SK_CTAS_PER_SM
#define RT_SK_CTAS_PER_SM 2
#endif
#ifndef RT_SK_MIN_CTAS
#define RT_SK_MIN_CTAS 3
#endif
constexpr int SKN = 128, SKM = 16, SKK = 64, SKSTAGES = RT_SK_STAGES;
constexpr int kSkB = SKK * SKN * 2, kSkA = SKM * SKK * 2, kSkStage = kSkB + kSkA;   // 16 KB + 2 KB
constexpr int kSkThreads = 192;
constexpr int kSkMaxCluster = 8;

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
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of `addr` in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Programmatic dependent launch: a grid launched with the stream-serialization attribute
// may start while the grid before it in the stream drains; grid_dependency_wait() returns
// once that grid has completed and its writes are visible (at once if there is none);
// grid_launch_dependents() lets the next such grid start its prologue.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// The hardware barrier over all threads of the cluster, in its two halves.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Optional per-CTA timeline for kernel development (off unless the translation unit is
// compiled with RT_SK_TRACE): thread 0 of every CTA stores the GPU-wide nanosecond timer at
// eight points of the kernel.
#ifdef RT_SK_TRACE
__device__ unsigned long long gSkTrace[4096 * 8];
#define SK_MARK(i)                                                                        \
  do {                                                                                    \
    if (threadIdx.x == (i == 2 ? 160 : 0)) {                                              \
      unsigned long long t_;                                                              \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                              \
      gSkTrace[((blockIdx.y * gridDim.x + blockIdx.x) & 4095) * 8 + (i)] = t_;            \
    }                                                                                     \
  } while (0)
#else
#define SK_MARK(i) \
  do {             \
  } while (0)
#endif

// rowsPad: 8 or 16, the rows of a that are exchanged and stored (M <= rowsPad).
__global__ void __launch_bounds__(kSkThreads, RT_SK_MIN_CTAS)
gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                      const __half* __restrict__ bias, const __half* __restrict__ addend,
                      __half* __restrict__ out, int M, int64_t K, int64_t N, int stepsPerRank,
                      int rowsPad, int act, int* status) {
  extern __shared__ unsigned char smemRaw[];
  __shared__ __align__(8) uint64_t sFull[SKSTAGES], sEmpty[SKSTAGES], sAcc;
  __shared__ uint32_t sTmemBase;
  __shared__ int sAbort;
  const int tid = threadIdx.x, warp = tid >> 5;
  SK_MARK(0);
  const uint32_t smemBase = (smem_u32(smemRaw) + 1023u) & ~1023u;
  const uint32_t redBase = smemBase + SKSTAGES * kSkStage;   // [rank - 1][rowsPad][128] f32, rank 0 only
  const uint32_t rank = cluster_rank(), ranks = cluster_size();
  const int64_t col0 = (int64_t)blockIdx.x * SKN;
  const int nkAll = (int)((K + SKK - 1) / SKK);
  const int it0 = (int)rank * stepsPerRank;
  const int nk = max(0, min(stepsPerRank, nkAll - it0));     // K steps of this CTA; may be none

  if (tid == 0) {
    sAbort = 0;
    for (int s = 0; s < SKSTAGES; s++) {
      mbar_init(smem_u32(&sFull[s]), 1);
      mbar_init(smem_u32(&sEmpty[s]), 1);
    }
    mbar_init(smem_u32(&sAcc), 1);
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sTmemBase), 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sTmemBase;
  SK_MARK(1);
  // Everything above touched no global memory; what follows reads tensors the grid before
  // this one may have written (a, addend) and overwrites out, which it may still read.
  grid_dependency_wait();
  cluster_arrive();   // first barrier: every CTA of the cluster is running (waited on below)

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      prefetch_tensormap(&mapA);
      prefetch_tensormap(&mapB);
      for (int it = 0; it < nk; it++) {
        const int s = it % SKSTAGES;
        if (it >= SKSTAGES && !mbar_wait(smem_u32(&sEmpty[s]), ((it / SKSTAGES) - 1) & 1, &sAbort))
          break;
        const uint32_t bar = smem_u32(&sFull[s]);
        const uint32_t dB = smemBase + s * kSkStage, dA = dB + kSkB;
        const int k0 = (it0 + it) * SKK;
        mbar_expect_tx(bar, kSkStage);
        tma_load_2d(dB, &mapB, (int)col0, k0, bar);                  // 64 columns x 64 k
        tma_load_2d(dB + SKK * 128, &mapB, (int)col0 + 64, k0, bar);
        tma_load_2d(dA, &mapA, k0, 0, bar);                          // 64 k x 16 rows of a
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer --------------------------------
    // D [128 columns of b, 16 rows of a]: A = b^T (MN-major), B = a (K-major), f32 D.
    constexpr uint32_t idesc = (1u << 4) | (1u << 15) | ((uint32_t)(SKM >> 3) << 17) |
                               ((uint32_t)(SKN >> 4) << 24);
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version, SW128
    constexpr uint32_t kLboMn = ((uint32_t)(SKK * 128) >> 4) << 16;       // next 64 columns of b
    constexpr uint32_t kLboK = (16u >> 4) << 16;
    bool ok = true;
    for (int it = 0; it < nk && ok; it++) {
      const int s = it % SKSTAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sFull[s]), (it / SKSTAGES) & 1, &sAbort)) != 0;
      if (!ok) break;
      tc_fence_after_sync();
      if (it == 0) SK_MARK(2);
      if (elect_one()) {
        // In a cluster the shared-window address of a CTA carries its rank above the
        // offset; the descriptor's address field takes the 14 offset bits only (left
        // in, the rank lands in the leading-dimension field beside it).
        const uint32_t wLo = (((smemBase + s * kSkStage) >> 4) & 0x3fffu) | kLboMn;
        const uint32_t xLo = (((smemBase + s * kSkStage + kSkB) >> 4) & 0x3fffu) | kLboK;
#pragma unroll
        for (int kk = 0; kk < SKK / 16; kk++) {
          const uint64_t wDesc = ((uint64_t)kDescHi << 32) | (wLo + kk * (2048 >> 4));
          const uint64_t xDesc = ((uint64_t)kDescHi << 32) | (xLo + kk * 2);
          mma_f16_ss(tmem, wDesc, xDesc, idesc, (it > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&sEmpty[s]));
        if (it == nk - 1) tc_commit(smem_u32(&sAcc));
      }
      __syncwarp();
    }
  }

  // Accumulator of this CTA: thread = column, 16 values = rows of a.
  float acc[SKM];
#pragma unroll
  for (int m = 0; m < SKM; m++) acc[m] = 0.f;
  if (warp < 4 && nk > 0) {
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sAcc), 0, &sAbort)) != 0;
    if (ok) {
      tc_fence_after_sync();
      uint32_t raw[SKM];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16), raw);
      tmem_wait_ld();
#pragma unroll
      for (int m = 0; m < SKM; m++) acc[m] = __uint_as_float(raw[m]);
    }
  }
  SK_MARK(3);
  grid_launch_dependents();   // the weights of this CTA are in: the next grid may set itself up
  __syncwarp();
  cluster_wait();
  if (warp < 4 && rank > 0) {
    const uint32_t dst = map_to_rank(redBase, 0) + (((rank - 1) * rowsPad) * SKN + tid) * 4;
#pragma unroll
    for (int m = 0; m < SKM; m++)
      if (m < rowsPad) st_cluster_f32(dst + m * SKN * 4, acc[m]);
  }
  // Second barrier: the partial sums are in rank 0's shared memory.  Every thread of every
  // CTA of the cluster reaches both barriers whatever happened above.
  __syncwarp();
  cluster_arrive();
  cluster_wait();
  SK_MARK(4);

  if (warp < 4 && rank == 0) {
    const float* red = reinterpret_cast<const float*>(smemRaw + (redBase - smem_u32(smemRaw)));
    for (uint32_t r = 1; r < ranks; r++)
#pragma unroll
      for (int m = 0; m < SKM; m++)
        if (m < rowsPad) acc[m] += red[((r - 1) * rowsPad + m) * SKN + tid];
    const int64_t n = col0 + tid;
    if (n < N) {
      const float bv = bias ? __half2float(bias[n]) : 0.f;
      act_dispatch(act, [&](auto code) {
#pragma unroll
        for (int m = 0; m < SKM; m++) {
          if (m < M) {
            float y = act_apply<decltype(code)::value>(acc[m] + bv);
            if (addend) y += __half2float(addend[(int64_t)m * N + n]);
            out[(int64_t)m * N + n] = __float2half_rn(y);
          }
        }
      });
    }
  }

  SK_MARK(5);
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && sAbort) atomicOr(status, kStatusWaitTimeout);
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 32);
  }
  SK_MARK(6);
}

}  // namespace

// f16, whole 16-byte row pitches, at least one box of every operand.  Up to 16 rows go
// to the cluster kernel (which wants a full tile of columns), more to the tiled one.
bool matmul_tc_supported(const void* a, const void* b, const void* out, int64_t M, int64_t K,
                         int64_t N, int dtype) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  return dtype == RT_F16 && M >= 1 && K >= 64 && N >= (M <= SKM ? SKN : 64) && K % 8 == 0 &&
         N % 8 == 0 && al(a) && al(b) && al(out) && M < (1ll << 31) - 256 && N < (1ll << 31) - 256 &&
         K < (1ll << 31) - 256 && (M + GBM - 1) / GBM <= 65535 && encode_fn() != nullptr;
}

namespace {
cudaError_t launch_skinny(const void* a, const void* b, const void* bias, const void* addend,
                          void* out, int64_t M, int64_t K, int64_t N, int act, int* status,
                          cudaStream_t s, std::string* err) {
  CUtensorMap ma, mb;
  if (!make_map(&ma, a, M, K, K, SKM, err) || !make_map(&mb, b, K, N, N, SKK, err))
    return cudaErrorInvalidValue;
  // Slices of K: enough CTAs for two per SM, at least two K steps each.
  const int64_t tiles = (N + SKN - 1) / SKN;
  const int nkAll = (int)((K + SKK - 1) / SKK);
  int cluster = 1;
  while (cluster < kSkMaxCluster && tiles * cluster < RT_SK_CTAS_PER_SM * 148 && nkAll / (cluster * 2) >= 2) cluster *= 2;
  const int stepsPerRank = (nkAll + cluster - 1) / cluster;
  const int rowsPad = M <= 8 ? 8 : 16;
  const int smem = SKSTAGES * kSkStage + 1024 + (cluster - 1) * rowsPad * SKN * 4;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_skinny_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)tiles, (unsigned)cluster);
  cfg.blockDim = dim3(kSkThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = (unsigned)cluster;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, gemm_tc_skinny_kernel, ma, mb, static_cast<const __half*>(bias),
                            static_cast<const __half*>(addend), static_cast<__half*>(out), (int)M,
                            K, N, stepsPerRank, rowsPad, act, status);
}
}  // namespace

cudaError_t launch_matmul_tc(const void* a, const void* b, const void* bias, const void* addend,
                             void* out, int64_t M, int64_t K, int64_t N, int act, int* status,
                             cudaStream_t s, std::string* err) {
  if (M <= SKM) return launch_skinny(a, b, bias, addend, out, M, K, N, act, status, s, err);
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
