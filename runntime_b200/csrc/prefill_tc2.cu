// Tensor-core prefill attention, two query tiles per CTA (head sizes 64 and 128).
//
// Same math and operand layouts as prefill_tc.cu, arranged so that the tensor
// pipe and the softmax warps of one SM keep each other busy: a CTA owns 256
// query rows of one head as two 128-row tiles, each with its own softmax
// warpgroup (warps 0-3 and 4-7), its own S/P columns and its own O accumulator
// in tensor memory (2 x 128 S + 2 x HD O <= 512 columns).  The K and V tiles in
// shared memory are shared by both query tiles.  The MMA warp interleaves the
// two tiles half a period apart,
//     S0(j) | PV1(j-1) | S1(j) | PV0(j) | S0(j+1) | ...
// so that while one warpgroup computes its softmax the tensor core runs the
// other tile's two products.  P overwrites the S columns it came from; the next
// S into those columns is issued after the PV that reads them, from the same
// thread, and tcgen05.mma operations issued by one thread execute in order.
//
// warp 8 = TMA producer (Q tiles once; K ring and V ring, separately released),
// warp 9 = MMA issuer and TMEM owner.
#include "common.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace rt {
namespace {

using namespace sm100;
using namespace tc;

constexpr int kThreads2 = 320;
constexpr int BK2 = 128;

template <int HD>
struct Cfg2 {
  static constexpr int CHUNKS = HD / 64;
  static constexpr int QT_BYTES = BM * HD * 2;        // one query tile
  static constexpr int KV_BYTES = BK2 * HD * 2;       // one K (or V) tile
  static constexpr int TOTAL_SLOTS = (226 * 1024 - 2 * QT_BYTES) / KV_BYTES;
  static constexpr int K_SLOTS = TOTAL_SLOTS >= 8 ? 4 : (TOTAL_SLOTS + 1) / 2;
  static constexpr int V_SLOTS = TOTAL_SLOTS >= 8 ? 4 : TOTAL_SLOTS / 2;
  static constexpr int SMEM = 2 * QT_BYTES + (K_SLOTS + V_SLOTS) * KV_BYTES + 1024;
  static constexpr int S_COLS = BK2;
  static constexpr int O_COL0 = 2 * S_COLS;
  static constexpr int TMEM_COLS = 512;
  static_assert(O_COL0 + 2 * HD <= TMEM_COLS, "tensor memory budget");
  static_assert(K_SLOTS >= 2 && V_SLOTS >= 2 && K_SLOTS <= 4 && V_SLOTS <= 4, "ring sizes");
};

struct Barriers2 {
  uint64_t fullQ;
  uint64_t fullK[4], emptyK[4], fullV[4], emptyV[4];
  uint64_t sFull[2], pReady[2], pvDone[2];
};

template <int HD>
__global__ void __launch_bounds__(kThreads2, 1)
prefill_tc2_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, const AttnParams p, int* status) {
  using C = Cfg2<HD>;
  constexpr int BK = BK2;
  extern __shared__ unsigned char smemRaw[];
  __shared__ Barriers2 bars;
  __shared__ uint32_t sTmemBase;
  __shared__ int sAbort;
  __shared__ int sLoMin[8], sEndMax[8];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  TC_TRACE_DECL
  const int pairTile = (int)gridDim.x - 1 - (int)blockIdx.x;  // longest rows first under a causal mask
  const int h = blockIdx.y;
  const int kvh = h / (p.qHeads / p.kvHeads);
  const int64_t row0 = (int64_t)pairTile * (2 * BM);

  const uint32_t smemBase = (smem_u32(smemRaw) + 1023u) & ~1023u;
  const uint32_t sQ = smemBase;                               // two query tiles back to back
  const uint32_t sK = sQ + 2 * C::QT_BYTES;                   // K ring
  const uint32_t sV = sK + C::K_SLOTS * C::KV_BYTES;          // V ring

  if (tid == 0) {
    sAbort = 0;
    mbar_init(smem_u32(&bars.fullQ), 1);
    for (int s = 0; s < 4; s++) {
      mbar_init(smem_u32(&bars.fullK[s]), 1);
      mbar_init(smem_u32(&bars.emptyK[s]), 1);
      mbar_init(smem_u32(&bars.fullV[s]), 1);
      mbar_init(smem_u32(&bars.emptyV[s]), 1);
    }
    for (int q = 0; q < 2; q++) {
      mbar_init(smem_u32(&bars.sFull[q]), 1);
      mbar_init(smem_u32(&bars.pReady[q]), BM);
      mbar_init(smem_u32(&bars.pvDone[q]), 1);
    }
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sTmemBase), C::TMEM_COLS);
    tmem_relinquish();
  }

  // Band of this thread's row, then of each 128-row tile.
  int lo = 1, end = 0;
  if (warp < 8) {
    const int64_t row = row0 + tid;  // tid 0..255 = tile q * 128 + row in tile
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

  // Per query tile: first and last key tile it touches; the CTA walks their union.
  int ktLo[2], ktHi[2], nq[2];
#pragma unroll
  for (int q = 0; q < 2; q++) {
    const int l4 = min(min(sLoMin[4 * q], sLoMin[4 * q + 1]), min(sLoMin[4 * q + 2], sLoMin[4 * q + 3]));
    const int e4 = max(max(sEndMax[4 * q], sEndMax[4 * q + 1]), max(sEndMax[4 * q + 2], sEndMax[4 * q + 3]));
    if (e4 >= 0) {
      ktLo[q] = l4 / BK;
      ktHi[q] = e4 / BK;
      nq[q] = ktHi[q] - ktLo[q] + 1;
    } else {
      ktLo[q] = INT_MAX;
      ktHi[q] = -1;
      nq[q] = 0;
    }
  }
  const int kt0 = min(ktLo[0], ktLo[1]);
  const int nU = (nq[0] | nq[1]) ? max(ktHi[0], ktHi[1]) - kt0 + 1 : 0;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && nU > 0) {
      prefetch_tensormap(&mapQ);
      prefetch_tensormap(&mapK);
      prefetch_tensormap(&mapV);
      mbar_expect_tx(smem_u32(&bars.fullQ), 2 * C::QT_BYTES);
      for (int q = 0; q < 2; q++)
        for (int c = 0; c < C::CHUNKS; c++)
          tma_load_2d(sQ + q * C::QT_BYTES + c * (BM * 128), &mapQ, h * HD + c * 64,
                      (int)row0 + q * BM, smem_u32(&bars.fullQ));
      for (int j = 0; j < nU; j++) {
        const int key0 = (kt0 + j) * BK;
        const int ks = j % C::K_SLOTS, vs = j % C::V_SLOTS;
        if (j >= C::K_SLOTS &&
            !mbar_wait(smem_u32(&bars.emptyK[ks]), ((j / C::K_SLOTS) - 1) & 1, &sAbort))
          break;
        mbar_expect_tx(smem_u32(&bars.fullK[ks]), C::KV_BYTES);
        for (int c = 0; c < C::CHUNKS; c++)
          tma_load_2d(sK + ks * C::KV_BYTES + c * (BK * 128), &mapK, kvh * HD + c * 64, key0,
                      smem_u32(&bars.fullK[ks]));
        if (j >= C::V_SLOTS &&
            !mbar_wait(smem_u32(&bars.emptyV[vs]), ((j / C::V_SLOTS) - 1) & 1, &sAbort))
          break;
        mbar_expect_tx(smem_u32(&bars.fullV[vs]), C::KV_BYTES);
        for (int c = 0; c < C::CHUNKS; c++)
          tma_load_2d(sV + vs * C::KV_BYTES + c * (BK * 128), &mapV, kvh * HD + c * 64, key0,
                      smem_u32(&bars.fullV[vs]));
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0 && nU > 0) {
      constexpr uint32_t idescS = instr_desc(BK, false);
      constexpr uint32_t idescO = instr_desc(HD, true);
      bool ok = mbar_wait(smem_u32(&bars.fullQ), 0, &sAbort);
      auto active = [&](int q, int j) {
        return nq[q] > 0 && kt0 + j >= ktLo[q] && kt0 + j <= ktHi[q];
      };
      // S_q(j) = Q_q K_j^T
      auto issueS = [&](int q, int j) {
        if (!ok || !active(q, j)) return;
        const int ks = j % C::K_SLOTS;
        ok = mbar_wait(smem_u32(&bars.fullK[ks]), (j / C::K_SLOTS) & 1, &sAbort);
        if (!ok) return;
        tc_fence_after_sync();
        TC_TRACE(10 + q, j);
        const uint32_t aBase = sQ + q * C::QT_BYTES, bBase = sK + ks * C::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) {
          const uint64_t aDesc = smem_desc(aBase + (kk >> 2) * (BM * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bDesc = smem_desc(bBase + (kk >> 2) * (BK * 128) + (kk & 3) * 32, 16, 1024);
          mma_f16_ss(tmem + q * C::S_COLS, aDesc, bDesc, idescS, kk > 0);
        }
        tc_commit(smem_u32(&bars.sFull[q]));
      };
      // O_q += P_q(j) V_j
      auto issuePV = [&](int q, int j) {
        if (!ok || !active(q, j)) return;
        const int i = kt0 + j - ktLo[q];  // index among this query tile's key tiles
        const int vs = j % C::V_SLOTS;
        TC_TRACE(20 + q, j);
        ok = mbar_wait(smem_u32(&bars.pReady[q]), i & 1, &sAbort);
        TC_TRACE(22 + q, j);
        if (ok) ok = mbar_wait(smem_u32(&bars.fullV[vs]), (j / C::V_SLOTS) & 1, &sAbort);
        if (!ok) return;
        tc_fence_after_sync();
        TC_TRACE(24 + q, j);
        const uint32_t bBase = sV + vs * C::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; kk++) {
          const uint64_t bDesc = smem_desc(bBase + kk * 2048, BK * 128, 1024);
          mma_f16_ts(tmem + C::O_COL0 + q * HD, tmem + q * C::S_COLS + kk * 8, bDesc, idescO,
                     (i > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&bars.pvDone[q]));
      };
      issueS(0, 0);
      for (int j = 0; j < nU && ok; j++) {
        if (j > 0) {
          issuePV(1, j - 1);
          if (ok) tc_commit(smem_u32(&bars.emptyV[(j - 1) % C::V_SLOTS]));
        }
        issueS(1, j);
        if (ok) tc_commit(smem_u32(&bars.emptyK[j % C::K_SLOTS]));
        issuePV(0, j);
        if (j + 1 < nU) issueS(0, j + 1);
      }
      issuePV(1, nU - 1);
      if (ok) tc_commit(smem_u32(&bars.emptyV[(nU - 1) % C::V_SLOTS]));
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    const int q = warp >> 2;
    const uint32_t laneBase = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t sCol = tmem + laneBase + q * C::S_COLS;
    const uint32_t oCol = tmem + laneBase + C::O_COL0 + q * HD;
    float mref = kNegSeed, l = 0.f;
    if (p.sinks) {
      mref = p.sinks[h];  // log2 domain: sink * ln2 * log2e
      l = 1.f;
    }
    bool ok = true;
    const int n = nq[q];
    for (int i = 0; i < n && ok; i++) {
      const int key0 = (ktLo[q] + i) * BK;
      TC_TRACE(0, i);
      ok = mbar_wait(smem_u32(&bars.sFull[q]), i & 1, &sAbort);
      if (!ok) break;
      tc_fence_after_sync();
      TC_TRACE(1, i);
      uint32_t sv[BK];
#pragma unroll
      for (int c = 0; c < BK; c += 32)
        tmem_ld32(sCol + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_wait_ld();
      TC_TRACE(2, i);
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
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BK; c += 8) {
#pragma unroll
        for (int u = 0; u < 4; u++)
          mx4[u] = max3(mx4[u], __uint_as_float(sv[c + 2 * u]), __uint_as_float(sv[c + 2 * u + 1]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * kLog2e;
      const bool grow = mx > mref + kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        const float mnew = fmaxf(mref, mx);
        const float f = fast_exp2(mref - mnew);
        mref = mnew;
        l *= f;
        if (i > 0) {
          ok = mbar_wait(smem_u32(&bars.pvDone[q]), (i - 1) & 1, &sAbort);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < HD; c += 32) {
            uint32_t o[32];
            tmem_ld32(oCol + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
            tmem_st32(oCol + c, o);
          }
        }
      }
      TC_TRACE(3, i);
      const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-mref, -mref);
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f),
                        make_float2(0.f, 0.f)};
      // Two halves of 64 scores: the packed P of a half goes to TMEM before the
      // next half is computed, which keeps the live registers under the budget.
#pragma unroll
      for (int half = 0; half < 2; half++) {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const int cc = half * 64 + c;
          const float2 t = fma2(make_float2(__uint_as_float(sv[cc]), __uint_as_float(sv[cc + 1])),
                                scale2, shift2);
          const float2 pe = exp2_pair(t, c >> 1);
          sum2[(c >> 1) & 3] = add2(sum2[(c >> 1) & 3], pe);
          const __half2 hp = __floats2half2_rn(pe.x, pe.y);
          pk[c / 2] = *reinterpret_cast<const uint32_t*>(&hp);
        }
        tmem_st32(sCol + half * 32, pk);
      }
      const float2 s01 = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
      l += s01.x + s01.y;
      TC_TRACE(4, i);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bars.pReady[q]));
      TC_TRACE(5, i);
    }

    // Epilogue: O / l -> f16 -> global.  Rows that saw no key are zeros.
    const int64_t row = row0 + tid;
    __half* out = static_cast<__half*>(p.out) + row * ((int64_t)p.qHeads * HD) + (int64_t)h * HD;
    if (n > 0 && ok) {
      ok = mbar_wait(smem_u32(&bars.pvDone[q]), (n - 1) & 1, &sAbort);
      if (ok) {
        tc_fence_after_sync();
        const float invL = (l > 0.f && lo <= end) ? 1.f / l : 0.f;
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t o[32];
          tmem_ld32(oCol + c, o);
          tmem_wait_ld();
          if (row < p.qLen) {
            uint4 pkd[4];
            uint32_t* w = reinterpret_cast<uint32_t*>(pkd);
#pragma unroll
            for (int x = 0; x < 32; x += 2) {
              const __half2 hp = __floats2half2_rn(__uint_as_float(o[x]) * invL,
                                                   __uint_as_float(o[x + 1]) * invL);
              w[x / 2] = *reinterpret_cast<const uint32_t*>(&hp);
            }
#pragma unroll
            for (int v = 0; v < 4; v++) reinterpret_cast<uint4*>(out + c)[v] = pkd[v];
          }
        }
      }
    } else if (n == 0 && row < p.qLen) {
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int c = 0; c < HD; c += 8) *reinterpret_cast<uint4*>(out + c) = z;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && sAbort) atomicOr(status, kStatusWaitTimeout);
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

template <int HD>
cudaError_t launch2(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  using C = Cfg2<HD>;
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, p.q, p.qLen, (int64_t)p.qHeads * HD, p.qStride, BM, err) ||
      !make_map(&mk, p.k, p.kvLen, (int64_t)p.kvHeads * HD, p.kvStride, BK2, err) ||
      !make_map(&mv, p.v, p.kvLen, (int64_t)p.kvHeads * HD, p.kvStride, BK2, err))
    return cudaErrorInvalidValue;
  auto kern = prefill_tc2_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)((p.qLen + 2 * BM - 1) / (2 * BM)), (unsigned)p.qHeads);
  kern<<<grid, kThreads2, C::SMEM, s>>>(mq, mk, mv, p, status);
  return cudaGetLastError();
}

}  // namespace

bool prefill_tc2_supported(const AttnParams& p) {
  return (p.hd == 64 || p.hd == 128) && p.qLen > BM;
}

cudaError_t launch_prefill_tc2(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  return p.hd == 64 ? launch2<64>(p, status, s, err) : launch2<128>(p, status, s, err);
}

}  // namespace rt
