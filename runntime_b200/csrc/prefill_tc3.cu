// Tensor-core prefill attention with two softmax warpgroups taking alternate
// key tiles of one 128-row query tile.
//
// In the other two tensor-core kernels a query tile is one serial chain
// S(j) -> softmax -> P V(j) -> S(j+1): the tensor pipe idles while a tile's
// softmax runs, and a second chain on the same SM only fills part of that gap.
// Here S has two buffers in tensor memory and P has columns of its own, so
//   - the S issuer runs ahead: S(j+1) is computed while tile j is in the softmax,
//   - warpgroup g (warps 4g..4g+3) owns tiles j = g, g+2, ...: each tile still gets a
//     whole warpgroup (one thread per query row, 128 scores in registers), but two
//     tiles are in flight, which doubles the softmax rate the tensor pipe can be fed
//     from,
//   - the P V issuer accumulates O += P(j) V(j) in tile order as the halves of P arrive.
// The running maximum is shared by the two warpgroups through shared memory: the
// reference point of a row moves only when its maximum has grown by more than 2^8
// (rare after the first tile), and the "max phases" of consecutive tiles are
// ordered by a per-warp counter, so both warpgroups always exponentiate against
// the same reference point and the accumulator is rescaled by exactly one of them.
//
// Head sizes: 64 and 128 (P in its own columns), 256 (the accumulator takes half of
// tensor memory, P overwrites the S columns it came from; K arrives as two
// 128-column halves and V as two 64-key halves so that every ring slot is 32 KB and
// S keeps the full-rate 128-key tile), and the narrow heads 32, 36, 52, ... (any
// multiple of 4 up to 60) padded to 64 inside the tile: K and V tiles are fetched
// with a 64-column box that starts on the 16-byte boundary at or below the head
// (the columns beside the head belong to its neighbours), Q is staged by the
// softmax threads with zeros in those columns, so the neighbours' columns add
// nothing to the scores, and the output columns they produce are dropped.
//
// Semantics are the 'attn' op's (see rt_attn.h); replaces attnFlash
// (packages/runntime/src/core/kernels/attention/attnFlash.ts:93-276).  Every wait is
// bounded; a wait that runs out sets the status word and the CTA winds down through
// the common exit that frees its tensor memory.
#include "common.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace rt {
namespace {

using namespace sm100;
using namespace tc;

constexpr int kThreads3 = 384;
constexpr int kRegsSoftmax3 = 216, kRegsOther3 = 64;  // 2*128*216 + 128*64 <= 384*168
constexpr int BK3 = 128;
constexpr int kMaxSlots = 8;

template <int HD>
struct Cfg3 {
  static constexpr int CHUNKS = HD / 64;                       // 64-column chunks of a row
  static constexpr int Q_BYTES = BM * HD * 2;
  static constexpr bool SPLIT = HD == 256;                      // K and V tiles arrive in two parts
  static constexpr int KP = SPLIT ? 2 : 1, VP = SPLIT ? 2 : 1;  // parts per key tile
  static constexpr int SLOT_BYTES = SPLIT ? 32 * 1024 : BK3 * HD * 2;
  static constexpr int SLOTS_FIT = (226 * 1024 - Q_BYTES) / SLOT_BYTES;
  static constexpr int SLOTS = SLOTS_FIT > kMaxSlots ? kMaxSlots : SLOTS_FIT;
  static constexpr int SMEM = Q_BYTES + SLOTS * SLOT_BYTES + 1024;
  static constexpr int K_CHUNKS = SPLIT ? 2 : CHUNKS;           // 64-column chunks in one K part
  static constexpr int V_ROWS = SPLIT ? 64 : BK3;               // keys in one V part
  static constexpr int O_COL = 2 * BK3;
  static constexpr bool P_OWN = HD <= 128;                      // P has columns of its own
  static constexpr int P_COL = O_COL + 128;
  static constexpr int TMEM_COLS = 512;
  static_assert(SLOTS >= KP + VP + 1, "ring too small");
  static_assert(O_COL + HD <= TMEM_COLS, "tensor memory budget");
};

struct Barriers3 {
  uint64_t fullQ;
  uint64_t full[kMaxSlots], empty[kMaxSlots];
  uint64_t sFull[2], sFree[2], pReady[2][2], pvDone[2];
};

// Ring sequence numbers.  The producer issues K(0); then, for every tile j, K(j+1)
// (if there is one) and V(j): K runs one tile ahead of V.
template <int KP, int VP>
__device__ __forceinline__ int seq_k(int j) { return j == 0 ? 0 : KP + (j - 1) * (KP + VP); }
template <int KP, int VP>
__device__ __forceinline__ int seq_v(int j, int n) {
  return KP + j * (KP + VP) + (j + 1 < n ? KP : 0);
}

// PADDED: the head is narrower than the 64 columns the tile holds (see the file header);
// p.hd is the real size, `shift` = (kvh * hd) & 7 the head's first column inside the box.
template <int HD, bool PADDED>
__global__ void __launch_bounds__(kThreads3, 1)
prefill_tc3_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, const AttnParams p, int* status) {
  using C = Cfg3<HD>;
  constexpr int BK = BK3, KP = C::KP, VP = C::VP, NS = C::SLOTS;
  static_assert(!PADDED || HD == 64, "narrow heads are padded to 64 columns");
  extern __shared__ unsigned char smemRaw[];
  __shared__ Barriers3 bars;
  __shared__ uint32_t sTmemBase;
  __shared__ int sAbort;
  __shared__ int sLoMin[4], sEndMax[4];
  __shared__ float sMref[BM];          // the rows' reference points (log2 domain)
  __shared__ float sL[2][BM];          // the warpgroups' row sums, for the epilogue
  __shared__ volatile int sMaxDone[4];  // per warp of a warpgroup: tiles whose max phase is over

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qTile = (int)gridDim.x - 1 - (int)blockIdx.x;  // long rows first under a causal mask
  const int h = blockIdx.y;
  const int kvh = h / (p.qHeads / p.kvHeads);
  const int64_t row0 = (int64_t)qTile * BM;
  const int hd = PADDED ? p.hd : HD;
  const int shift = PADDED ? ((kvh * hd) & 7) : 0;

  const uint32_t smemBase = (smem_u32(smemRaw) + 1023u) & ~1023u;
  const uint32_t sQ = smemBase;
  const uint32_t sRing = sQ + C::Q_BYTES;

  if (tid == 0) {
    sAbort = 0;
    mbar_init(smem_u32(&bars.fullQ), 1);
    for (int s = 0; s < kMaxSlots; s++) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&bars.sFull[b]), 1);
      mbar_init(smem_u32(&bars.sFree[b]), 4);        // one arrival per warp of the warpgroup
      mbar_init(smem_u32(&bars.pReady[b][0]), 4);
      mbar_init(smem_u32(&bars.pReady[b][1]), 4);
      mbar_init(smem_u32(&bars.pvDone[b]), 1);
    }
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sTmemBase), C::TMEM_COLS);
    tmem_relinquish();
  }

  // Band of this thread's row (warpgroup 0 computes it; warpgroup 1 gets the same row's
  // band from the same formula), then of the whole row tile.
  const int rowInTile = tid & 127;
  int lo = 1, end = 0;  // empty
  if (warp < 8) {
    const int64_t row = row0 + rowInTile;
    if (row < p.qLen) {
      int64_t l64, e64;
      row_band(p, row, l64, e64);
      if (l64 <= e64) {
        lo = (int)l64;
        end = (int)e64;
      }
    }
    if (warp < 4) {
      int wl = lo <= end ? lo : INT_MAX, we = lo <= end ? end : -1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        wl = min(wl, __shfl_xor_sync(0xffffffffu, wl, o));
        we = max(we, __shfl_xor_sync(0xffffffffu, we, o));
      }
      if (lane == 0) {
        sLoMin[warp] = wl;
        sEndMax[warp] = we;
        sMaxDone[warp] = 0;
      }
      sMref[rowInTile] = p.sinks ? p.sinks[h] : kNegSeed;  // sinks arrive in the log2 domain
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

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther3));
    if (warp == 8) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0 && nTiles > 0) {
        prefetch_tensormap(&mapK);
        prefetch_tensormap(&mapV);
        if (!PADDED) {
          prefetch_tensormap(&mapQ);
          mbar_expect_tx(smem_u32(&bars.fullQ), C::Q_BYTES);
          for (int c = 0; c < C::CHUNKS; c++)
            tma_load_2d(sQ + c * (BM * 128), &mapQ, h * HD + c * 64, (int)row0, smem_u32(&bars.fullQ));
        }
        const int xKV = PADDED ? ((kvh * hd) & ~7) : kvh * HD;
        int seq = 0;
        bool ok = true;
        auto slot_for = [&](int& slot) {  // claims the next ring slot, waiting for its release
          slot = seq % NS;
          if (seq >= NS) ok = mbar_wait(smem_u32(&bars.empty[slot]), ((seq / NS) - 1) & 1, &sAbort);
          seq++;
          return ok;
        };
        auto load_k = [&](int j) {
          const int key0 = (kt0 + j) * BK;
          for (int part = 0; part < KP && ok; part++) {
            int slot;
            if (!slot_for(slot)) return;
            const uint32_t bar = smem_u32(&bars.full[slot]), dst = sRing + slot * C::SLOT_BYTES;
            mbar_expect_tx(bar, C::K_CHUNKS * BK * 128);
            for (int c = 0; c < C::K_CHUNKS; c++)
              tma_load_2d(dst + c * (BK * 128), &mapK, xKV + (part * C::K_CHUNKS + c) * 64, key0, bar);
          }
        };
        auto load_v = [&](int j) {
          const int key0 = (kt0 + j) * BK;
          for (int part = 0; part < VP && ok; part++) {
            int slot;
            if (!slot_for(slot)) return;
            const uint32_t bar = smem_u32(&bars.full[slot]), dst = sRing + slot * C::SLOT_BYTES;
            mbar_expect_tx(bar, C::CHUNKS * C::V_ROWS * 128);
            for (int c = 0; c < C::CHUNKS; c++)
              tma_load_2d(dst + c * (C::V_ROWS * 128), &mapV, xKV + c * 64, key0 + part * C::V_ROWS, bar);
          }
        };
        load_k(0);
        for (int j = 0; j < nTiles && ok; j++) {
          if (j + 1 < nTiles) load_k(j + 1);
          if (ok) load_v(j);
        }
      }
    } else if (warp == 9) {
      // ------------------------------ MMA issuer: S = Q K^T ----------------------
      // The whole warp walks the loop (waits included); the tensor-core instructions
      // run in one elected lane, which keeps their operands in uniform registers.
      if (nTiles > 0) {
        constexpr uint32_t idescS = instr_desc(BK, false);
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version, SW128
        constexpr uint32_t kLboK = (16u >> 4) << 16;
        auto desc = [](uint32_t lo32) { return ((uint64_t)kDescHi << 32) | lo32; };
        auto wait = [&](uint64_t* bar, int parity) {
          return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), (uint32_t)parity, &sAbort)) != 0;
        };
        const uint32_t aLo = (sQ >> 4) | kLboK;
        const int kSteps = PADDED ? (shift + hd + 15) / 16 : HD / 16;  // K = 16 per instruction
        bool ok = wait(&bars.fullQ, 0);
#pragma unroll 1
        for (int j = 0; j < nTiles && ok; j++) {
          const int b = j & 1;
          const int s0 = seq_k<KP, VP>(j);
#pragma unroll
          for (int part = 0; part < KP; part++) {
            const int slot = (s0 + part) % NS;
            ok = wait(&bars.full[slot], ((s0 + part) / NS) & 1);
            // The S buffer is free once its previous contents are dead: after the softmax
            // warpgroup has loaded S(j-2) into registers, or — where P overwrites S — after
            // P V(j-2) has read it.
            if (ok && part == 0 && j >= 2)
              ok = wait(C::P_OWN ? &bars.sFree[b] : &bars.pvDone[b], ((j >> 1) - 1) & 1);
            if (!ok) break;
            tc_fence_after_sync();
            if (elect_one()) {
              const uint32_t bLo = ((sRing + slot * C::SLOT_BYTES) >> 4) | kLboK;
              constexpr int kPerPart = C::K_CHUNKS * 4;  // K = 16 steps in one part
#pragma unroll
              for (int k2 = 0; k2 < kPerPart; k2++) {
                const int kk = part * kPerPart + k2;
                if (PADDED && k2 >= kSteps) break;
                const uint32_t aOff = (kk >> 2) * ((BM * 128) >> 4) + (kk & 3) * 2;
                const uint32_t bOff = (k2 >> 2) * ((BK * 128) >> 4) + (k2 & 3) * 2;
                mma_f16_ss(tmem + b * BK, desc(aLo + aOff), desc(bLo + bOff), idescS, kk > 0);
              }
              tc_commit(smem_u32(&bars.empty[slot]));
              if (part == KP - 1) tc_commit(smem_u32(&bars.sFull[b]));
            }
            __syncwarp();
          }
        }
      }
    } else if (warp == 10) {
      // ------------------------------ MMA issuer: O += P V ------------------------
      if (nTiles > 0) {
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
        constexpr uint32_t kLboV = ((uint32_t)(C::V_ROWS * 128) >> 4) << 16;  // next 64 columns of hd
        auto desc = [](uint32_t lo32) { return ((uint64_t)kDescHi << 32) | lo32; };
        auto wait = [&](uint64_t* bar, int parity) {
          return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), (uint32_t)parity, &sAbort)) != 0;
        };
        const uint32_t idescO = instr_desc(PADDED ? ((shift + hd + 15) & ~15) : HD, true);
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < nTiles && ok; j++) {
          const int b = j & 1;
          const int s0 = seq_v<KP, VP>(j, nTiles);
          const uint32_t pCol = tmem + (C::P_OWN ? C::P_COL + b * 64 : b * BK);
#pragma unroll
          for (int half = 0; half < 2; half++) {
            const int part = VP == 2 ? half : 0;
            const int slot = (s0 + part) % NS;
            if (VP == 2 || half == 0) ok = wait(&bars.full[slot], ((s0 + part) / NS) & 1);
            if (ok) ok = wait(&bars.pReady[b][half], (j >> 1) & 1);
            if (!ok) break;
            tc_fence_after_sync();
            if (elect_one()) {
              const uint32_t bLo = ((sRing + slot * C::SLOT_BYTES) >> 4) | kLboV;
#pragma unroll
              for (int k2 = 0; k2 < 4; k2++) {
                const int kk = half * 4 + k2;              // 16 keys per step
                const int kLocal = VP == 2 ? k2 : kk;       // within this part's rows
                mma_f16_ts(tmem + C::O_COL, pCol + kk * 8, desc(bLo + kLocal * (2048 >> 4)), idescO,
                           (j > 0 || kk > 0) ? 1u : 0u);
              }
              if (VP == 2 || half == 1) tc_commit(smem_u32(&bars.empty[slot]));
              if (half == 1) tc_commit(smem_u32(&bars.pvDone[b]));
            }
            __syncwarp();
          }
        }
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax3));
    const int g = warp >> 2, w = warp & 3;
    const uint32_t laneBase = (uint32_t)(w * 32) << 16;
    const uint32_t sCol = tmem + laneBase + g * BK;
    const uint32_t pCol = tmem + laneBase + (C::P_OWN ? C::P_COL + g * 64 : g * BK);
    const uint32_t oCol = tmem + laneBase + C::O_COL;
    bool ok = true;

    if (PADDED && nTiles > 0) {
      // Q tile by hand: 16-byte units of the swizzled K-major layout, the head's columns at
      // [shift, shift + hd), zeros beside them and in rows past the end.
      const __half* qg = static_cast<const __half*>(p.q) + (int64_t)h * hd;
      for (int u = tid; u < BM * 8; u += 256) {
        const int r = u >> 3, unit = u & 7;
        const int64_t row = row0 + r;
        __align__(16) __half vals[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
          const int c = unit * 8 + e - shift;
          vals[e] = (row < p.qLen && c >= 0 && c < hd) ? qg[row * p.qStride + c] : __half(0.f);
        }
        const uint32_t addr = sQ + r * 128 + ((unit ^ (r & 7)) << 4);
        const uint4 v4 = *reinterpret_cast<const uint4*>(vals);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v4.x), "r"(v4.y),
                     "r"(v4.z), "r"(v4.w)
                     : "memory");
      }
      fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
      named_barrier_sync(2, 256);
      if (tid == 0) mbar_arrive(smem_u32(&bars.fullQ));
    }

    float seen = p.sinks ? p.sinks[h] : kNegSeed;  // the reference point this thread's l is relative to
    float l = (p.sinks && g == 0) ? 1.f : 0.f;
#pragma unroll 1
    for (int j = g; j < nTiles && ok; j += 2) {
      const int key0 = (kt0 + j) * BK;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.sFull[g]), (j >> 1) & 1, &sAbort));
      if (!ok) break;  // the whole warp leaves together
      tc_fence_after_sync();
      uint32_t sv[BK];
#pragma unroll
      for (int c = 0; c < BK; c += 32)
        tmem_ld32(sCol + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_wait_ld();
      if (C::P_OWN) {  // S(j) is in registers: its buffer may take S(j+2)
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.sFree[g]));
      }
      const bool fullTile = lo <= key0 && end >= key0 + BK - 1;
      if (p.hasKeyBias) {
        const int b0 = p.biasStart - key0, b1 = p.biasEnd - key0;
#pragma unroll
        for (int c = 0; c < BK; c++) {
          const float s = __uint_as_float(sv[c]);
          sv[c] = __float_as_uint((c >= b0 && c < b1) ? s + p.biasValue : s);
        }
      }
      if (!fullTile) {
        // visible columns of this row are the interval [c0, c0 + span]
        const int c0 = lo <= end ? lo - key0 : (1 << 30);
        const unsigned span = lo <= end ? (unsigned)(end - lo) : 0u;
#pragma unroll
        for (int c = 0; c < BK; c++)
          sv[c] = ((unsigned)(c - c0) <= span) ? sv[c] : 0xff800000u;  // -inf
      }
      // Row maximum: four independent chains of 3-input max.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < BK; c += 8) {
#pragma unroll
        for (int u = 0; u < 4; u++)
          mx4[u] = max3(mx4[u], __uint_as_float(sv[c + 2 * u]), __uint_as_float(sv[c + 2 * u + 1]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * kLog2e;

      // ---- max phase, in tile order across the two warpgroups ----
      if (j > 0) {
        bool arrived = false;
        for (int i = 0; i < (1 << 22); i++) {
          if (sMaxDone[w] >= j) { arrived = true; break; }
          if ((i & 63) == 63) {
            if (sAbort) break;
            __nanosleep(64);
          }
        }
        ok = __all_sync(0xffffffffu, arrived);
        if (!ok) {
          sAbort = 1;
          break;
        }
        __threadfence_block();
        tc_fence_after_sync();
      }
      float mref = sMref[rowInTile];
      if (mref != seen) {  // the other warpgroup moved the reference point since this one last looked
        l *= fast_exp2(seen - mref);
        seen = mref;
      }
      if (__any_sync(0xffffffffu, mx > mref + kRescaleThreshold)) {
        const float mnew = fmaxf(mref, mx);
        const float f = fast_exp2(mref - mnew);
        if (j > 0) {
          // O holds the tiles up to j-1 once P V(j-1) has landed (the products complete in order)
          ok = __all_sync(0xffffffffu,
                          mbar_wait(smem_u32(&bars.pvDone[(j - 1) & 1]), ((j - 1) >> 1) & 1, &sAbort));
          if (!ok) break;
          tc_fence_after_sync();
          constexpr int oCols = PADDED ? 64 : HD;
#pragma unroll
          for (int c = 0; c < oCols; c += 32) {
            uint32_t o[32];
            tmem_ld32(oCol + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 32; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
            tmem_st32(oCol + c, o);
          }
          tmem_wait_st();
          tc_fence_before_sync();
        }
        l *= f;
        mref = seen = mnew;
        sMref[rowInTile] = mnew;
      }
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        sMaxDone[w] = j + 1;
      }

      // ---- exponentials, P in two halves ----
      // P's own columns were last read by P V(j-2).
      if (C::P_OWN && j >= 2) {
        ok = __all_sync(0xffffffffu,
                        mbar_wait(smem_u32(&bars.pvDone[g]), ((j >> 1) - 1) & 1, &sAbort));
        if (!ok) break;
      }
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f),
                        make_float2(0.f, 0.f)};
      const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-mref, -mref);
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
        tmem_st32(pCol + half * 32, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.pReady[g][half]));
      }
      const float2 s01 = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
      l += s01.x + s01.y;
    }

    // ---- epilogue: both warpgroups, half of the output columns each ----
    // (every softmax thread passes the two barriers, also after a failed wait)
    named_barrier_sync(2, 256);
    {
      const float mfin = sMref[rowInTile];
      if (mfin != seen) l *= fast_exp2(seen - mfin);
      sL[g][rowInTile] = l;
    }
    named_barrier_sync(2, 256);
    l = sL[0][rowInTile] + sL[1][rowInTile];
    const int64_t row = row0 + rowInTile;
    __half* out = static_cast<__half*>(p.out) + row * ((int64_t)p.qHeads * hd) + (int64_t)h * hd;
    if (nTiles > 0 && ok && !sAbort) {
      ok = mbar_wait(smem_u32(&bars.pvDone[(nTiles - 1) & 1]), ((nTiles - 1) >> 1) & 1, &sAbort);
      if (ok) {
        tc_fence_after_sync();
        const float invL = (l > 0.f && lo <= end) ? 1.f / l : 0.f;  // a row that saw no key: zeros
        constexpr int oCols = PADDED ? 64 : HD;
        constexpr int perGroup = oCols / 2;
#pragma unroll
        for (int c = g * perGroup; c < (g + 1) * perGroup; c += 32) {
          uint32_t o[32];
          tmem_ld32(oCol + c, o);
          tmem_wait_ld();
          if (row < p.qLen) {
            if (PADDED) {
#pragma unroll
              for (int x = 0; x < 32; x += 2) {
                const int col = c + x - shift;  // even: shift is 0 or 4
                if (col >= 0 && col < hd)
                  *reinterpret_cast<__half2*>(out + col) = __floats2half2_rn(
                      __uint_as_float(o[x]) * invL, __uint_as_float(o[x + 1]) * invL);
              }
            } else {
              uint4 pkd[4];
              uint32_t* wds = reinterpret_cast<uint32_t*>(pkd);
#pragma unroll
              for (int x = 0; x < 32; x += 2) {
                const __half2 hp = __floats2half2_rn(__uint_as_float(o[x]) * invL,
                                                     __uint_as_float(o[x + 1]) * invL);
                wds[x / 2] = *reinterpret_cast<const uint32_t*>(&hp);
              }
#pragma unroll
              for (int v = 0; v < 4; v++) reinterpret_cast<uint4*>(out + c)[v] = pkd[v];
            }
          }
        }
      }
    } else if (nTiles == 0 && row < p.qLen) {
      // no row of this tile sees a key
      for (int c = g * (hd / 2); c < (g + 1) * (hd / 2); c += 2)
        *reinterpret_cast<__half2*>(out + c) = __floats2half2_rn(0.f, 0.f);
    }
  }

  // Common exit: every role arrives here, then the allocating warp frees TMEM.
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && sAbort) atomicOr(status, kStatusWaitTimeout);
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

template <int HD, bool PADDED>
cudaError_t launch3(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  using C = Cfg3<HD>;
  CUtensorMap mq, mk, mv;
  // The narrow-head form reads Q with plain loads; its K/V maps span the real columns,
  // so a box that runs past the last head reads zeros there.
  const int64_t qCols = (int64_t)p.qHeads * p.hd, kvCols = (int64_t)p.kvHeads * p.hd;
  if ((!PADDED && !make_map(&mq, p.q, p.qLen, qCols, p.qStride, BM, err)) ||
      !make_map(&mk, p.k, p.kvLen, kvCols, p.kvStride, BK3, err) ||
      !make_map(&mv, p.v, p.kvLen, kvCols, p.kvStride, C::V_ROWS, err))
    return cudaErrorInvalidValue;
  if (PADDED) mq = mk;  // unused by the kernel; a valid map all the same
  auto kern = prefill_tc3_kernel<HD, PADDED>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)((p.qLen + BM - 1) / BM), (unsigned)p.qHeads);
  kern<<<grid, kThreads3, C::SMEM, s>>>(mq, mk, mv, p, status);
  return cudaGetLastError();
}

}  // namespace

bool prefill_tc3_supported(const AttnParams& p, int dtype) {
  if (dtype != RT_F16) return false;
  const bool wide = p.hd == 64 || p.hd == 128 || p.hd == 256;
  const bool narrow = p.hd >= 4 && p.hd <= 60 && p.hd % 4 == 0;
  if (!wide && !narrow) return false;
  if (p.qLen < 2 || p.qLen >= (1ll << 31) - 256 || p.kvLen >= (1ll << 31) - 256) return false;
  auto al = [](const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; };
  // TMA: 16-byte aligned bases and row pitches (Q of a narrow head is read with plain
  // loads and written back in 4-byte pairs)
  if (!al(p.k, 16) || !al(p.v, 16) || (p.kvStride * 2) % 16) return false;
  if (wide && (!al(p.q, 16) || !al(p.out, 16) || (p.qStride * 2) % 16)) return false;
  if (narrow && (!al(p.q, 4) || !al(p.out, 4) || p.qStride % 2)) return false;
  if (!encode_fn()) return false;
  return true;
}

cudaError_t launch_prefill_tc3(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  switch (p.hd) {
    case 64: return launch3<64, false>(p, status, s, err);
    case 128: return launch3<128, false>(p, status, s, err);
    case 256: return launch3<256, false>(p, status, s, err);
  }
  return launch3<64, true>(p, status, s, err);
}

}  // namespace rt
