// Tensor-core prefill attention, two query tiles per CTA (head sizes 64 and 128).
//
// Same math and operand layouts as prefill_tc.cu, arranged so that the tensor
// pipe and the softmax warps of one SM keep each other busy: a CTA owns 256
// query rows of one head as two 128-row tiles, each with its own softmax
// warpgroup (warps 0-3 and 4-7), its own S/P columns and its own O accumulator
// in tensor memory (2 x 128 S + 2 x HD O <= 512 columns).  The K and V tiles in
// shared memory are shared by both query tiles.  Each tile is a chain
//     S(j) -> softmax -> P V(j) -> S(j+1) -> ...
// and the two chains run half a period apart, so that while one warpgroup
// computes its softmax the tensor core runs the other tile's two products.  P overwrites the S columns it came from; the next
// S into those columns is issued after the PV that reads them, from the same
// thread, and tcgen05.mma operations issued by one thread execute in order.
//
// Warps 0-3 and 4-7 are the two softmax warpgroups; the third warpgroup holds
// the TMA producer (warp 8: Q tiles once; K ring and V ring, separately
// released), one MMA issuing warp per query tile (warps 9 and 10; warp 9 also
// owns the TMEM allocation) and a padding warp.  A softmax thread keeps a whole row of 128 scores in registers, so
// the register file is re-split at run time (setmaxnreg): the third warpgroup
// gives up what it does not need and the softmax warpgroups take it.
#include "common.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace rt {
namespace {

using namespace sm100;
using namespace tc;

#ifndef RT_TC2_STAGGER_NS
#define RT_TC2_STAGGER_NS 1000
#endif
constexpr int kThreads2 = 384;
#ifndef RT_TC2_REGS_SOFTMAX
#define RT_TC2_REGS_SOFTMAX 216
#define RT_TC2_REGS_OTHER 64
#endif
constexpr int kRegsSoftmax = RT_TC2_REGS_SOFTMAX, kRegsOther = RT_TC2_REGS_OTHER;  // 2*128*216 + 128*64 <= 384*168
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
  uint64_t sFull[2], pReady[2][2], pvDone[2];   // pReady[q][half of the key tile]
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
      mbar_init(smem_u32(&bars.emptyK[s]), 2);   // one arrival per chain
      mbar_init(smem_u32(&bars.fullV[s]), 1);
      mbar_init(smem_u32(&bars.emptyV[s]), 2);
    }
    for (int q = 0; q < 2; q++) {
      mbar_init(smem_u32(&bars.sFull[q]), 1);
      mbar_init(smem_u32(&bars.pReady[q][0]), 4);   // one arrival per softmax warp
      mbar_init(smem_u32(&bars.pReady[q][1]), 4);
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

  if (warp >= 8) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
   // warps 10 and 11 only pad the warpgroup
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
   } else if (warp == 9 || warp == 10) {
    // ------------------------------ MMA issuers -------------------------------
    // One issuing warp per query tile: S_q(j) = Q_q K_j^T, then (once the softmax
    // warpgroup has turned S into P in place) O_q += P_q(j) V_j, then S_q(j+1) into the
    // same columns.  tcgen05.mma operations issued by one thread execute in order,
    // which is all the ordering a chain needs; the two chains share nothing but the
    // read-only K and V tiles, so each tile is released by two arrivals.  The whole
    // warp walks the loop (waits included); only the tensor-core instructions run in
    // one elected lane.  A single thread spends 150-300 cycles on every wait-fence-
    // issue-commit round, far more than the eight MMAs of a product take to issue, so
    // one warp for both chains serialises them.
    const int q = warp - 9;
    if (nU > 0) {
      constexpr uint32_t idescS = instr_desc(BK, false);
      constexpr uint32_t idescO = instr_desc(HD, true);
      // Shared-memory descriptors: the high word is constant, the low word is
      // (address >> 4) | leading-offset field, so stepping to the next K slice or
      // ring slot is one 32-bit add.
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version, SW128
      constexpr uint32_t kLboK = (16u >> 4) << 16;                   // K-major operands (Q, K)
      constexpr uint32_t kLboV = ((uint32_t)(BK * 128) >> 4) << 16;  // MN-major operand (V)
      auto desc = [](uint32_t lo) { return ((uint64_t)kDescHi << 32) | lo; };
      const uint32_t aLo = ((sQ + q * C::QT_BYTES) >> 4) | kLboK;
      const uint32_t kLo = (sK >> 4) | kLboK, vLo = (sV >> 4) | kLboV;
      const uint32_t dS = tmem + q * C::S_COLS, dO = tmem + C::O_COL0 + q * HD;
      auto wait = [&](uint64_t* bar, int parity) {  // the warp agrees on the outcome
        return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), (uint32_t)parity, &sAbort)) != 0;
      };
      bool ok = wait(&bars.fullQ, 0);
      const int jLo = nq[q] > 0 ? ktLo[q] - kt0 : nU, jHi = nq[q] > 0 ? ktHi[q] - kt0 : -1;
      // Start the second chain about half a period late.  Left alone the chains fall
      // into step: both softmax warpgroups then want the special-function unit at the
      // same time and both want the tensor pipe at the same time.
      if (q == 1) __nanosleep(RT_TC2_STAGGER_NS);
      int kSeen = -1;  // last K tile this warp has waited for
#pragma unroll 1
      for (int j = 0; j < nU && ok; j++) {
        const int ks = j % C::K_SLOTS, vs = j % C::V_SLOTS;
        const bool mine = j >= jLo && j <= jHi;
        if (mine) {
          if (kSeen < j) {
            ok = wait(&bars.fullK[ks], (j / C::K_SLOTS) & 1);
            if (!ok) break;
            tc_fence_after_sync();
          }
          TC_TRACE(10 + q, j);
          if (elect_one()) {
            const uint32_t bLo = kLo + ks * (C::KV_BYTES >> 4);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) {
              constexpr int kChunk = (BM * 128) >> 4;  // BM == BK: same step for Q and K
              const uint32_t off = (kk >> 2) * kChunk + (kk & 3) * 2;
              mma_f16_ss(dS, desc(aLo + off), desc(bLo + off), idescS, kk > 0);
            }
            tc_commit(smem_u32(&bars.sFull[q]));
            tc_commit(smem_u32(&bars.emptyK[ks]));
          }
          __syncwarp();
          // While the softmax runs: make sure V(j) and the next K tile have landed, so
          // that nothing but P stands between its arrival and the next two products.
          ok = wait(&bars.fullV[vs], (j / C::V_SLOTS) & 1);
          if (ok && j + 1 < nU) {
            ok = wait(&bars.fullK[(j + 1) % C::K_SLOTS], ((j + 1) / C::K_SLOTS) & 1);
            kSeen = j + 1;
          }
          if (!ok) break;
          TC_TRACE(20 + q, j);
          const uint32_t bLo = vLo + vs * (C::KV_BYTES >> 4);
          // P arrives in two halves of 64 keys; the first half's products run while the
          // softmax warps still work on the second.
#pragma unroll
          for (int half = 0; half < 2; half++) {
            ok = wait(&bars.pReady[q][half], (j - jLo) & 1);
            if (!ok) break;
            tc_fence_after_sync();
            TC_TRACE(22 + 2 * half + q, j);
            if (elect_one()) {
#pragma unroll
              for (int kk = 4 * half; kk < 4 * half + 4; kk++)
                mma_f16_ts(dO, dS + kk * 8, desc(bLo + kk * (2048 >> 4)), idescO,
                           (j > jLo || kk > 0) ? 1u : 0u);
              if (half == 1) {
                tc_commit(smem_u32(&bars.emptyV[vs]));
                if (j == jHi) tc_commit(smem_u32(&bars.pvDone[q]));  // the epilogue waits for this one
              }
            }
            __syncwarp();
          }
          if (!ok) break;
        } else {
          // Not a tile of this chain: only hand the K and V slots back — after they
          // were filled, so that the arrival cannot land in the slot's previous round.
          ok = wait(&bars.fullK[ks], (j / C::K_SLOTS) & 1) && wait(&bars.fullV[vs], (j / C::V_SLOTS) & 1);
          if (!ok) break;
          if (elect_one()) {
            mbar_arrive(smem_u32(&bars.emptyK[ks]));
            mbar_arrive(smem_u32(&bars.emptyV[vs]));
          }
          __syncwarp();
        }
      }
    }
   }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
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
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.sFull[q]), i & 1, &sAbort));
      if (!ok) break;  // the whole warp leaves together
      tc_fence_after_sync();
      TC_TRACE(1, i);
      uint32_t sv[BK];
#pragma unroll
      for (int c = 0; c < BK; c += 32)
        tmem_ld32(sCol + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_wait_ld();
      TC_TRACE(2, i);
      const bool fullTile = lo <= key0 && end >= key0 + BK - 1;
      if (p.hasKeyBias) {
        // columns [b0, b1) of this tile get the bias (select, no branch per element)
        const int b0 = p.biasStart - key0, b1 = p.biasEnd - key0;
#pragma unroll
        for (int c = 0; c < BK; c++) {
          const float s = __uint_as_float(sv[c]);
          sv[c] = __float_as_uint((c >= b0 && c < b1) ? s + p.biasValue : s);
        }
      }
      if (!fullTile) {
        // visible columns of this row are the interval [c0, c0 + span]; one unsigned
        // compare and one select per score
        const int c0 = lo <= end ? lo - key0 : (1 << 30);  // a row that sees nothing: no column passes
        const unsigned span = lo <= end ? (unsigned)(end - lo) : 0u;
#pragma unroll
        for (int c = 0; c < BK; c++)
          sv[c] = ((unsigned)(c - c0) <= span) ? sv[c] : 0xff800000u;  // -inf
      }
      TC_TRACE(6, i);
      // Row maximum (four independent chains of 3-input max), folded into whichever
      // loop runs first.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      auto foldMax = [&](int c) {  // columns c .. c+7
#pragma unroll
        for (int u = 0; u < 4; u++)
          mx4[u] = max3(mx4[u], __uint_as_float(sv[c + 2 * u]), __uint_as_float(sv[c + 2 * u + 1]));
      };
      // Lazy rescale: the reference point mref moves only when some row's maximum
      // grew by more than 2^8 (whole warp together, because TMEM loads and stores are
      // warp-collective).  O holds the tiles up to i-1; their P V products were issued,
      // by the same thread, before S(i), whose completion this warp has already seen:
      // they are done, and the accumulator can be scaled in place.
      auto rescale = [&]() {
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * kLog2e;
        if (!__any_sync(0xffffffffu, mx > mref + kRescaleThreshold)) return false;
        const float mnew = fmaxf(mref, mx);
        const float f = fast_exp2(mref - mnew);
        mref = mnew;
        l *= f;
        if (i > 0) {
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
        return true;
      };
      float2 sum2[4];
      uint32_t pk[32];
      // p = 2^(s*log2e - mref) for 64 scores: one packed FFMA per two scores, MUFU,
      // four independent packed sums, packed to f16 pairs.  With `withMax` the row
      // maximum over all 128 scores is gathered in the same loop, where its
      // instructions hide under the special-function unit's.
      auto expHalf = [&](int half, bool withMax) {
        const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-mref, -mref);
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const int cc = half * 64 + c;
          const float2 t = fma2(make_float2(__uint_as_float(sv[cc]), __uint_as_float(sv[cc + 1])),
                                scale2, shift2);
          const float2 pe = exp2_pair(t, c >> 1);
          sum2[(c >> 1) & 3] = add2(sum2[(c >> 1) & 3], pe);
          const __half2 hp = __floats2half2_rn(pe.x, pe.y);
          pk[c / 2] = *reinterpret_cast<const uint32_t*>(&hp);
          if (withMax && (c & 3) == 0) foldMax(2 * c);  // 16 steps x 8 columns = all 128
        }
      };
      auto publish = [&](int half) {
        tmem_st32(sCol + half * 32, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.pReady[q][half]));
        TC_TRACE(4 + half, i);
      };
      auto clearSums = [&]() {
#pragma unroll
        for (int u = 0; u < 4; u++) sum2[u] = make_float2(0.f, 0.f);
      };
      clearSums();
      if (i == 0) {
        // First tile: there is no reference point yet, the maximum comes first.
#pragma unroll
        for (int c = 0; c < BK; c += 8) foldMax(c);
        rescale();
        TC_TRACE(3, i);
        expHalf(0, false);
      } else {
        // Later tiles: start the exponentials against the current reference point
        // at once; the maximum is rarely 2^8 above it, and when it is the half is
        // simply computed again.
        TC_TRACE(3, i);
        expHalf(0, true);
        if (rescale()) {
          clearSums();
          expHalf(0, false);
        }
      }
      publish(0);
      expHalf(1, false);
      publish(1);
      const float2 s01 = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
      l += s01.x + s01.y;
    }

    // Epilogue: O / l -> f16 -> global.  Rows that saw no key are zeros.
    const int64_t row = row0 + tid;
    __half* out = static_cast<__half*>(p.out) + row * ((int64_t)p.qHeads * HD) + (int64_t)h * HD;
    if (n > 0 && ok) {
      ok = mbar_wait(smem_u32(&bars.pvDone[q]), 0, &sAbort);  // committed once, after the last P V
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

bool prefill_tc2_supported(const AttnParams& p, int dtype) {
  return prefill_tc_supported(p, dtype) && (p.hd == 64 || p.hd == 128) && p.qLen > BM;
}

cudaError_t launch_prefill_tc2(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  return p.hd == 64 ? launch2<64>(p, status, s, err) : launch2<128>(p, status, s, err);
}

}  // namespace rt
