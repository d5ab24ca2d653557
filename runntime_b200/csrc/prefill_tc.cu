// Tensor-core prefill attention for f16 storage: a flash-style fused kernel on
// the 5th-generation tensor cores (tcgen05) with accumulators in tensor memory.
//
// One CTA owns 128 query rows of one query head.  Roles:
//   warps 0-3  softmax: one thread per query row (= one TMEM lane).  Reads the
//              scores S from TMEM, applies the band/segment mask, keeps the
//              online-softmax state in fp32, writes the probabilities P back to
//              TMEM as f16 (over the S columns it has just read), rescales the
//              output accumulator only when a row's max has grown by more than
//              2^8, and runs the epilogue (O / l -> f16 -> global).
//   warp 4     TMA producer: Q once, then K and V tiles of BK keys into a
//              shared-memory ring (128-byte swizzle), one mbarrier per tile.
//   warp 5     MMA issuer: S = Q K^T (A, B from shared memory) into one of two
//              S buffers, and O += P V (A = P from TMEM, B = V tile, MN-major).
//              S of tile j+1 is issued before P V of tile j so that the tensor
//              pipe works while the softmax warps are busy.
//
// Semantics are the 'attn' op's (window, segments / per-sequence lengths, GQA,
// sinks, key bias, no score scale, empty rows -> zeros); see rt_attn.h.  It
// replaces attnFlash (packages/runntime/src/core/kernels/attention/
// attnFlash.ts:93-276), which has no tensor-core path.
//
// Every wait is bounded (sm100.cuh); a wait that runs out sets the status word
// and the CTA winds down through the common exit that frees its tensor memory.
#include "common.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace rt {
namespace {

using namespace sm100;
using namespace tc;

constexpr int kSoftmaxThreads = 128;
constexpr int kThreads = 192;

template <int HD, bool PSMEM>
struct Cfg {
  static constexpr int BK = HD <= 128 ? 128 : 64;          // keys per tile
  static constexpr int CHUNKS = HD / 64;                   // 64-column (128-byte) chunks of a row
  static constexpr int Q_BYTES = BM * HD * 2;
  static constexpr int KV_BYTES = BK * HD * 2;             // one K (or V) tile
  // Where P lives.  In tensor memory (over the S columns) P V is a TS MMA; in
  // shared memory (two buffers of 128 x BK f16) it is an SS MMA.  Measured rates
  // per K = 16 step at M = 128: SS 64 cycles at N = 128; TS 113 cycles at
  // N = 128 and 137 at N = 256.
  static constexpr bool P_SMEM = PSMEM;
  static constexpr int P_BYTES = P_SMEM ? BM * BK * 2 : 0;  // one P buffer
  // K and V tiles sit in separate rings: a K slot is free as soon as S(j) has been
  // computed, a V slot only after P V(j), so K can be fetched further ahead.
  static constexpr int TILE_SLOTS = (226 * 1024 - Q_BYTES - 2 * P_BYTES) / KV_BYTES;
  static constexpr int K_SLOTS = (TILE_SLOTS + 1) / 2 > 4 ? 4 : (TILE_SLOTS + 1) / 2;
  static constexpr int V_SLOTS = TILE_SLOTS / 2 > 4 ? 4 : TILE_SLOTS / 2;
  static constexpr int SMEM = Q_BYTES + 2 * P_BYTES + (K_SLOTS + V_SLOTS) * KV_BYTES + 1024;
  static constexpr int S_COLS = BK;                        // f32 score columns per buffer
  static constexpr int O_COL = 2 * S_COLS;                 // O accumulator after the two S buffers
  static constexpr int TMEM_COLS = 512;
  static_assert(O_COL + HD <= TMEM_COLS, "tensor memory budget");
  static_assert(K_SLOTS >= 2 && V_SLOTS >= 2, "need double-buffered rings");
};

struct Barriers {
  uint64_t fullQ;
  uint64_t fullK[4], fullV[4], emptyK[4], emptyV[4];
  uint64_t sFull[2], pReady[2], pvDone[2];
};

template <int HD, bool PSMEM>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const AttnParams p, int* status) {
  using C = Cfg<HD, PSMEM>;
  constexpr int BK = C::BK;
  extern __shared__ unsigned char smemRaw[];
  __shared__ Barriers bars;
  __shared__ uint32_t sTmemBase;
  __shared__ int sAbort;
  __shared__ int sLoMin[4], sEndMax[4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  TC_TRACE_DECL
  // Long rows first: under a causal mask the last row tile has the most keys.
  const int qTile = (int)gridDim.x - 1 - (int)blockIdx.x;
  const int h = blockIdx.y;
  const int kvh = h / (p.qHeads / p.kvHeads);
  const int64_t row0 = (int64_t)qTile * BM;

  // 1024-byte aligned carve-up: swizzle atoms must start on 1024-byte lines.
  const uint32_t smemBase = (smem_u32(smemRaw) + 1023u) & ~1023u;
  const uint32_t sQ = smemBase;
  const uint32_t sP = sQ + C::Q_BYTES;            // two P buffers (head sizes up to 128)
  const uint32_t sK = sP + 2 * C::P_BYTES;        // K ring
  const uint32_t sV = sK + C::K_SLOTS * C::KV_BYTES;  // V ring

  if (tid == 0) {
    sAbort = 0;
    mbar_init(smem_u32(&bars.fullQ), 1);
    for (int s = 0; s < 4; s++) {
      mbar_init(smem_u32(&bars.fullK[s]), 1);
      mbar_init(smem_u32(&bars.fullV[s]), 1);
      mbar_init(smem_u32(&bars.emptyK[s]), 1);
      mbar_init(smem_u32(&bars.emptyV[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&bars.sFull[b]), 1);
      mbar_init(smem_u32(&bars.pReady[b]), kSoftmaxThreads);
      mbar_init(smem_u32(&bars.pvDone[b]), 1);
    }
    fence_barrier_init();
  }
  if (warp == 5) {
    tmem_alloc(smem_u32(&sTmemBase), C::TMEM_COLS);
    tmem_relinquish();
  }

  // Band of this thread's row (softmax threads) and of the whole row tile.
  int lo = 1, end = 0;  // empty
  if (tid < kSoftmaxThreads) {
    const int64_t row = row0 + tid;
    if (row < p.qLen) {
      int64_t l64, e64;
      row_band(p, row, l64, e64);
      if (l64 <= e64) {
        lo = (int)l64;
        end = (int)e64;
      }
    }
    int wl = lo <= end ? lo : INT_MAX, we = lo <= end ? end : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      wl = min(wl, __shfl_xor_sync(0xffffffffu, wl, o));
      we = max(we, __shfl_xor_sync(0xffffffffu, we, o));
    }
    if (lane == 0) {
      sLoMin[warp] = wl;
      sEndMax[warp] = we;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sTmemBase;
  const int tileLo = min(min(sLoMin[0], sLoMin[1]), min(sLoMin[2], sLoMin[3]));
  const int tileEnd = max(max(sEndMax[0], sEndMax[1]), max(sEndMax[2], sEndMax[3]));
  const int kt0 = tileEnd >= 0 ? tileLo / BK : 0;
  const int nTiles = tileEnd >= 0 ? tileEnd / BK - kt0 + 1 : 0;

  if (warp == 4) {
    // ------------------------------ TMA producer ------------------------------
    // lane 0: Q, then the K ring; lane 1: the V ring (each runs ahead on its own).
    if (lane == 0 && nTiles > 0) {
      prefetch_tensormap(&mapQ);
      prefetch_tensormap(&mapK);
      mbar_expect_tx(smem_u32(&bars.fullQ), C::Q_BYTES);
      for (int c = 0; c < C::CHUNKS; c++)
        tma_load_2d(sQ + c * (BM * 128), &mapQ, h * HD + c * 64, (int)row0, smem_u32(&bars.fullQ));
      for (int j = 0; j < nTiles; j++) {
        const int s = j % C::K_SLOTS;
        if (j >= C::K_SLOTS &&
            !mbar_wait(smem_u32(&bars.emptyK[s]), ((j / C::K_SLOTS) - 1) & 1, &sAbort))
          break;
        mbar_expect_tx(smem_u32(&bars.fullK[s]), C::KV_BYTES);
        for (int c = 0; c < C::CHUNKS; c++)
          tma_load_2d(sK + s * C::KV_BYTES + c * (BK * 128), &mapK, kvh * HD + c * 64,
                      (kt0 + j) * BK, smem_u32(&bars.fullK[s]));
      }
    } else if (lane == 1 && nTiles > 0) {
      prefetch_tensormap(&mapV);
      for (int j = 0; j < nTiles; j++) {
        const int s = j % C::V_SLOTS;
        if (j >= C::V_SLOTS &&
            !mbar_wait(smem_u32(&bars.emptyV[s]), ((j / C::V_SLOTS) - 1) & 1, &sAbort))
          break;
        mbar_expect_tx(smem_u32(&bars.fullV[s]), C::KV_BYTES);
        for (int c = 0; c < C::CHUNKS; c++)
          tma_load_2d(sV + s * C::KV_BYTES + c * (BK * 128), &mapV, kvh * HD + c * 64,
                      (kt0 + j) * BK, smem_u32(&bars.fullV[s]));
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && nTiles > 0) {
      constexpr uint32_t idescS = instr_desc(BK, false);
      constexpr uint32_t idescO = instr_desc(HD, true);
      bool ok = mbar_wait(smem_u32(&bars.fullQ), 0, &sAbort);
      for (int j = 0; ok && j <= nTiles; j++) {
        if (j < nTiles) {
          const int s = j % C::K_SLOTS, b = j & 1;
          ok = mbar_wait(smem_u32(&bars.fullK[s]), (j / C::K_SLOTS) & 1, &sAbort);
          // With P in tensor memory over the S columns, S(j) must not land before
          // P V(j-2) has read them.  With P in shared memory the S buffer is free as
          // soon as the softmax warps have loaded it, which P-ready(j-2) implies.
          if (!C::P_SMEM && ok && j >= 2)
            ok = mbar_wait(smem_u32(&bars.pvDone[b]), ((j - 2) >> 1) & 1, &sAbort);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t dK = sK + s * C::KV_BYTES;
#pragma unroll
          for (int kk = 0; kk < HD / 16; kk++) {
            // K-major operands: 16 elements (32 bytes) further along the swizzled row per step
            const uint64_t aDesc = smem_desc(sQ + (kk >> 2) * (BM * 128) + (kk & 3) * 32, 16, 1024);
            const uint64_t bDesc = smem_desc(dK + (kk >> 2) * (BK * 128) + (kk & 3) * 32, 16, 1024);
            mma_f16_ss(tmem + b * C::S_COLS, aDesc, bDesc, idescS, kk > 0);
          }
          tc_commit(smem_u32(&bars.sFull[b]));
          tc_commit(smem_u32(&bars.emptyK[s]));
        }
        if (j >= 1) {
          const int t = j - 1, s = t % C::V_SLOTS, b = t & 1;
          ok = mbar_wait(smem_u32(&bars.pReady[b]), (t >> 1) & 1, &sAbort);
          if (ok) ok = mbar_wait(smem_u32(&bars.fullV[s]), (t / C::V_SLOTS) & 1, &sAbort);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t dV = sV + s * C::KV_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; kk++) {
            // V is [keys][hd] (MN-major B): 16 keys = 2048 bytes further per step;
            // LBO = next 64 columns of hd, SBO = next 8 keys.
            const uint64_t bDesc = smem_desc(dV + kk * 2048, BK * 128, 1024);
            // P: f16 pairs, 8 columns of TMEM per 16 keys
            if (C::P_SMEM) {
              // P: [128 rows][BK keys] f16, K-major, 64-key chunks of 128-byte rows
              const uint64_t aDesc =
                  smem_desc(sP + b * C::P_BYTES + (kk >> 2) * (BM * 128) + (kk & 3) * 32, 16, 1024);
              mma_f16_ss(tmem + C::O_COL, aDesc, bDesc, idescO, (t > 0 || kk > 0) ? 1u : 0u);
            } else {
              mma_f16_ts(tmem + C::O_COL, tmem + b * C::S_COLS + kk * 8, bDesc, idescO,
                         (t > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(smem_u32(&bars.emptyV[s]));
          tc_commit(smem_u32(&bars.pvDone[b]));
        }
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    const uint32_t laneBase = (uint32_t)(warp * 32) << 16;
    float mref = kNegSeed, l = 0.f;
    if (p.sinks) {
      mref = p.sinks[h];  // log2 domain: sink * ln2 * log2e
      l = 1.f;
    }
    bool ok = true;
    for (int j = 0; j < nTiles && ok; j++) {
      const int b = j & 1;
      const int key0 = (kt0 + j) * BK;
      TC_TRACE(0, j);
      ok = mbar_wait(smem_u32(&bars.sFull[b]), (j >> 1) & 1, &sAbort);
      if (!ok) break;
      tc_fence_after_sync();
      TC_TRACE(1, j);
      uint32_t sv[BK];
#pragma unroll
      for (int c = 0; c < BK; c += 32)
        tmem_ld32(tmem + laneBase + b * C::S_COLS + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_wait_ld();
      TC_TRACE(2, j);
      const bool fullTile = lo <= key0 && end >= key0 + BK - 1;
      if (!fullTile || p.hasKeyBias) {
#pragma unroll
        for (int c = 0; c < BK; c++) {
          const int jj = key0 + c;
          float s = __uint_as_float(sv[c]);
          if (p.hasKeyBias && jj >= p.biasStart && jj < p.biasEnd) s += p.biasValue;
          sv[c] = __float_as_uint((jj >= lo && jj <= end) ? s : -INFINITY);
        }
      }
      // Row max with four independent chains of 3-input max.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BK; c += 8) {
#pragma unroll
        for (int u = 0; u < 4; u++)
          mx4[u] = max3(mx4[u], __uint_as_float(sv[c + 2 * u]), __uint_as_float(sv[c + 2 * u + 1]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * kLog2e;
      // Lazy rescale: only when some row's max grew by more than 2^8 (whole warp
      // together, because TMEM loads/stores are warp-collective).
      const bool grow = mx > mref + kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float mnew = fmaxf(mref, mx);
        const float f = fast_exp2(mref - mnew);
        mref = mnew;
        l *= f;
        if (j > 0) {
          // O holds the tiles up to j-1: wait for the last P V to land, then scale.
          ok = mbar_wait(smem_u32(&bars.pvDone[(j - 1) & 1]), ((j - 1) >> 1) & 1, &sAbort);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < HD; c += 32) {
            uint32_t o[32];
            tmem_ld32(tmem + laneBase + C::O_COL + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
            tmem_st32(tmem + laneBase + C::O_COL + c, o);
          }
        }
      }
      // p = 2^(s*log2e - mref): one packed FFMA per two scores, one MUFU each, four
      // independent packed sums; packed to f16 pairs over the S columns just read.
      TC_TRACE(3, j);
      const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-mref, -mref);
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f),
                        make_float2(0.f, 0.f)};
      uint32_t pk[BK / 2];
#pragma unroll
      for (int c = 0; c < BK; c += 2) {
        const float2 t = fma2(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])),
                              scale2, shift2);
        const float2 pe = exp2_pair(t, c >> 1);
        sum2[(c >> 1) & 3] = add2(sum2[(c >> 1) & 3], pe);
        const __half2 hp = __floats2half2_rn(pe.x, pe.y);
        pk[c / 2] = *reinterpret_cast<const uint32_t*>(&hp);
      }
      const float2 s01 = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
      l += s01.x + s01.y;
      if (C::P_SMEM) {
        // The buffer was last read by P V(j-2).
        if (j >= 2) {
          ok = mbar_wait(smem_u32(&bars.pvDone[b]), ((j - 2) >> 1) & 1, &sAbort);
          if (!ok) break;
        }
        // Row `tid` of the A operand: 16-byte units (8 keys) swizzled by row & 7.
        const uint32_t rowBase = sP + b * C::P_BYTES + tid * 128;
#pragma unroll
        for (int u = 0; u < BK / 8; u++) {
          const uint32_t addr = rowBase + (u >> 3) * (BM * 128) + (((u & 7) ^ (tid & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * u]),
                       "r"(pk[4 * u + 1]), "r"(pk[4 * u + 2]), "r"(pk[4 * u + 3])
                       : "memory");
        }
        fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
      } else {
#pragma unroll
        for (int c = 0; c < BK / 2; c += 32)
          tmem_st32(tmem + laneBase + b * C::S_COLS + c, *reinterpret_cast<uint32_t(*)[32]>(&pk[c]));
      }
      TC_TRACE(4, j);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars.pReady[b]));
      TC_TRACE(5, j);
    }

    // Epilogue: O / l -> f16 -> global.  Rows that saw no key are zeros.
    const int64_t row = row0 + tid;
    __half* out = static_cast<__half*>(p.out) + row * ((int64_t)p.qHeads * HD) + (int64_t)h * HD;
    if (nTiles > 0 && ok) {
      ok = mbar_wait(smem_u32(&bars.pvDone[(nTiles - 1) & 1]), ((nTiles - 1) >> 1) & 1, &sAbort);
      if (ok) {
        tc_fence_after_sync();
        const float invL = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t o[32];
          tmem_ld32(tmem + laneBase + C::O_COL + c, o);
          tmem_wait_ld();
          if (row < p.qLen) {
            uint4 pkd[4];
            uint32_t* w = reinterpret_cast<uint32_t*>(pkd);
#pragma unroll
            for (int x = 0; x < 32; x += 2) {
              // a row with an empty band has l = 0 (or only the sink): force zeros
              const float a = lo <= end ? __uint_as_float(o[x]) * invL : 0.f;
              const float bb = lo <= end ? __uint_as_float(o[x + 1]) * invL : 0.f;
              const __half2 hp = __floats2half2_rn(a, bb);
              w[x / 2] = *reinterpret_cast<const uint32_t*>(&hp);
            }
#pragma unroll
            for (int v = 0; v < 4; v++) reinterpret_cast<uint4*>(out + c)[v] = pkd[v];
          }
        }
      }
    } else if (nTiles == 0 && row < p.qLen) {
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int c = 0; c < HD; c += 8) *reinterpret_cast<uint4*>(out + c) = z;
    }
  }

  // Common exit: every role arrives here, then the allocating warp frees TMEM.
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && sAbort) atomicOr(status, kStatusWaitTimeout);
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------

template <int HD, bool PSMEM>
cudaError_t launch(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  using C = Cfg<HD, PSMEM>;
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, p.q, p.qLen, (int64_t)p.qHeads * HD, p.qStride, BM, err) ||
      !make_map(&mk, p.k, p.kvLen, (int64_t)p.kvHeads * HD, p.kvStride, C::BK, err) ||
      !make_map(&mv, p.v, p.kvLen, (int64_t)p.kvHeads * HD, p.kvStride, C::BK, err))
    return cudaErrorInvalidValue;
  auto kern = prefill_tc_kernel<HD, PSMEM>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)((p.qLen + BM - 1) / BM), (unsigned)p.qHeads);
  kern<<<grid, kThreads, C::SMEM, s>>>(mq, mk, mv, p, status);
  return cudaGetLastError();
}

}  // namespace

bool prefill_tc_supported(const AttnParams& p, int dtype) {
  if (dtype != RT_F16) return false;
  if (p.hd != 64 && p.hd != 128 && p.hd != 256) return false;
  if (p.qLen < 2 || p.qLen >= (1ll << 31) - BM || p.kvLen >= (1ll << 31) - 256) return false;
  // TMA: 16-byte aligned bases and row pitches
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  if (!al(p.q) || !al(p.k) || !al(p.v) || !al(p.out)) return false;
  if ((p.qStride * 2) % 16 || (p.kvStride * 2) % 16) return false;
  if (!encode_fn()) return false;
  return true;
}

cudaError_t launch_prefill_tc(const AttnParams& p, int dtype, int* status, cudaStream_t s,
                              std::string* err) {
  (void)dtype;
  if (p.tcMode == 3 && prefill_tc2_supported(p)) return launch_prefill_tc2(p, status, s, err);
  switch (p.hd) {
    case 64: return p.tcMode == 4 ? launch<64, true>(p, status, s, err)
                                  : launch<64, false>(p, status, s, err);
    case 128: return p.tcMode == 4 ? launch<128, true>(p, status, s, err)
                                   : launch<128, false>(p, status, s, err);
    case 256: return launch<256, false>(p, status, s, err);
  }
  *err = "unsupported head size";
  return cudaErrorInvalidValue;
}

}  // namespace rt
