// Tensor-core prefill attention for f16 storage: a flash-style fused kernel on
// the 5th-generation tensor cores (tcgen05) with accumulators in tensor memory.
//
// One CTA owns 128 query rows of one query head.  Roles:
//   softmax warps (4 x SPLIT): one thread per (query row, column part).  Warp w
//              works on TMEM lanes 32*(w%4)..+31 (= 32 query rows) and, with
//              SPLIT = 2, on one half of the tile's score columns; the two
//              threads of a row exchange their partial row max through shared
//              memory once per tile.  They read the scores S from TMEM, apply the
//              band/segment mask, keep the online-softmax state in fp32, write the
//              probabilities P as f16 (to TMEM over the S columns just read, or to
//              a swizzled shared-memory tile), rescale the output accumulator only
//              when a row's max has grown by more than 2^8, and run the epilogue.
//   producer warp: TMA loads — Q once, then the K ring (lane 0) and the V ring
//              (lane 1) of BK-key tiles, 128-byte swizzle, one mbarrier per tile.
//   two MMA warps: one issues S = Q K^T (A, B from shared memory) into one of two
//              S buffers as soon as a K tile and a free buffer exist; the other
//              issues O += P V (A = P from TMEM or shared memory, B = V tile,
//              MN-major) as soon as P is ready.  Two instruction streams, so that
//              waiting for P never delays the next S and the tensor pipe always
//              has work queued while the softmax warps are busy.
//
// Semantics are the 'attn' op's (window, segments / per-sequence lengths, GQA,
// sinks, key bias, no score scale, empty rows -> zeros); see rt_attn.h.  It
// replaces attnFlash (packages/runntime/src/core/kernels/attention/
// attnFlash.ts:93-276), which has no tensor-core path.
//
// The kernel is a template over where P lives (tensor memory or shared memory)
// and over one or two softmax threads per row; the launcher uses one thread per
// row with P in tensor memory, the fastest measured on B200 (head size 128,
// causal 8192: 880-940 TFLOP/s).  Measured and not faster: P through shared
// memory for an SS-form P V (the stores and the proxy fence cost more than the
// faster MMA gains); two threads per row (the special-function unit, 16 ex2 per
// clock per SM, is the shared limit and the per-tile exchange of row maxima keeps
// both halves' ex2 phases in lockstep); evaluating part of the exponentials by
// polynomial on the FMA pipe (more issue slots than the MUFU cycles it frees;
// RT_POLY_NUM in tc_common.cuh, default 0).  Two query tiles per CTA is faster on
// large grids at head sizes 64 and 128 and lives in prefill_tc2.cu; this kernel
// keeps head size 256 (its accumulator leaves no tensor memory for a second tile)
// and small grids.
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

template <int HD, bool PSMEM, int SPLIT>
struct Cfg {
  static constexpr int BK = HD <= 128 ? 128 : 64;          // keys per tile
  static constexpr int CW = BK / SPLIT;                    // score columns per softmax thread
  static constexpr int SOFTMAX_THREADS = 128 * SPLIT;
  static constexpr int THREADS = SOFTMAX_THREADS + 96;
  // The two products are issued by different warps so that a wait in one
  // instruction stream (P not ready yet) never holds back the other.
  static constexpr int PRODUCER_WARP = 4 * SPLIT, MMA_WARP = 4 * SPLIT + 1, PV_WARP = 4 * SPLIT + 2;
  static constexpr int CHUNKS = HD / 64;                   // 64-column (128-byte) chunks of a row
  static constexpr int Q_BYTES = BM * HD * 2;
  static constexpr int KV_BYTES = BK * HD * 2;             // one K (or V) tile
  // Where P lives.  In tensor memory (over the S columns) P V is a TS MMA; in
  // shared memory (one buffer of 128 x BK f16, written once P V of the previous
  // tile has read it) it is an SS MMA.  Measured rates
  // per K = 16 step at M = 128: SS 64 cycles at N = 128; TS 113 cycles at
  // N = 128 and 137 at N = 256.
  static constexpr bool P_SMEM = PSMEM;
  static constexpr int P_BYTES = P_SMEM ? BM * BK * 2 : 0;  // one P buffer
  // Two P buffers when they fit beside four K/V tiles (then writing P(j) never
  // waits for P V(j-1)); otherwise one.
  static constexpr int P_BUFS = !P_SMEM ? 0 : (Q_BYTES + 2 * P_BYTES + 4 * KV_BYTES <= 224 * 1024 && SPLIT == 1) ? 2 : 1;
  // K and V tiles sit in separate rings: a K slot is free as soon as S(j) has been
  // computed, a V slot only after P V(j), so K can be fetched further ahead.
  static constexpr int PB = P_BUFS > 0 ? P_BUFS : 1;       // divisor that is never zero
  static constexpr int TILE_SLOTS = ((SPLIT == 1 ? 224 : 221) * 1024 - Q_BYTES - P_BUFS * P_BYTES) / KV_BYTES;
  static constexpr int K_SLOTS = (TILE_SLOTS + 1) / 2 > 4 ? 4 : (TILE_SLOTS + 1) / 2;
  static constexpr int V_SLOTS = TILE_SLOTS / 2 > 4 ? 4 : TILE_SLOTS / 2;
  static constexpr int SMEM = Q_BYTES + P_BUFS * P_BYTES + (K_SLOTS + V_SLOTS) * KV_BYTES + 1024;
  static constexpr int S_COLS = BK;                        // f32 score columns per buffer
  static constexpr int O_COL = 2 * S_COLS;                 // O accumulator after the two S buffers
  // P in tensor memory gets columns of its own (two buffers of BK/2 packed f16
  // pairs) when they fit, so that the next S never waits for a P V to finish
  // reading; otherwise P overwrites the S columns it came from.
  static constexpr bool P_OWN_COLS = !PSMEM && (2 * S_COLS + HD + S_COLS <= 512);
  static constexpr int P_COL = P_OWN_COLS ? O_COL + HD : 0;
  static constexpr int P_STRIDE = P_OWN_COLS ? S_COLS / 2 : S_COLS;  // between the two P buffers
  static constexpr int OW = HD / SPLIT;                    // O columns per softmax thread
  static constexpr int TMEM_COLS = 512;
  static_assert(O_COL + HD <= TMEM_COLS, "tensor memory budget");
  static_assert(K_SLOTS >= 2 && V_SLOTS >= 2, "need double-buffered rings");
  static_assert(CW % 32 == 0 && OW % 32 == 0, "column parts are whole 32-column TMEM accesses");
};

struct Barriers {
  uint64_t fullQ;
  uint64_t fullK[4], fullV[4], emptyK[4], emptyV[4];
  uint64_t sFull[2], sFree[2], pReady[2], pvDone[2];
};

template <int HD, bool PSMEM, int SPLIT>
__global__ void __launch_bounds__(Cfg<HD, PSMEM, SPLIT>::THREADS, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                  const __grid_constant__ CUtensorMap mapV, const AttnParams p, int* status) {
  using C = Cfg<HD, PSMEM, SPLIT>;
  constexpr int BK = C::BK, CW = C::CW, OW = C::OW;
  extern __shared__ unsigned char smemRaw[];
  __shared__ Barriers bars;
  __shared__ uint32_t sTmemBase;
  __shared__ int sAbort;
  __shared__ int sLoMin[4], sEndMax[4];
  __shared__ float sRowMax[2][SPLIT == 2 ? 256 : 1];  // partial row max, by tile parity
  __shared__ float sRowSum[SPLIT == 2 ? 256 : 1];     // partial row sums for the epilogue

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
  const uint32_t sP = sQ + C::Q_BYTES;                // the P buffer (when P goes through smem)
  const uint32_t sK = sP + C::P_BUFS * C::P_BYTES;    // K ring
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
      mbar_init(smem_u32(&bars.sFree[b]), C::SOFTMAX_THREADS / 32);   // one arrival per warp
      mbar_init(smem_u32(&bars.pReady[b]), C::SOFTMAX_THREADS / 32);
      mbar_init(smem_u32(&bars.pvDone[b]), 1);
    }
    fence_barrier_init();
  }
  if (warp == C::MMA_WARP) {
    tmem_alloc(smem_u32(&sTmemBase), C::TMEM_COLS);
    tmem_relinquish();
  }

  // Band of this thread's row (softmax threads) and of the whole row tile.
  const int rowInTile = tid & 127, part = tid >> 7;
  int lo = 1, end = 0;  // empty
  if (tid < C::SOFTMAX_THREADS) {
    const int64_t row = row0 + rowInTile;
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
    if (lane == 0 && part == 0) {
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

  if (warp == C::PRODUCER_WARP) {
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
  } else if (warp == C::MMA_WARP) {
    // ------------------------------ MMA issuer: S = Q K^T ----------------------
    if (lane == 0 && nTiles > 0) {
      constexpr uint32_t idescS = instr_desc(BK, false);
      bool ok = mbar_wait(smem_u32(&bars.fullQ), 0, &sAbort);
      for (int j = 0; ok && j < nTiles; j++) {
        const int s = j % C::K_SLOTS, b = j & 1;
        TC_TRACE(10, j);
        ok = mbar_wait(smem_u32(&bars.fullK[s]), (j / C::K_SLOTS) & 1, &sAbort);
        // The S buffer is free once its previous contents are dead: with P written
        // over the S columns, after P V(j-2) has read them; with P elsewhere (shared
        // memory or its own TMEM columns), as soon as the softmax warps have loaded
        // S(j-2) into registers.
        if (ok && j >= 2)
          ok = mbar_wait(smem_u32((C::P_SMEM || C::P_OWN_COLS) ? &bars.sFree[b] : &bars.pvDone[b]),
                         ((j - 2) >> 1) & 1, &sAbort);
        if (!ok) break;
        TC_TRACE(11, j);
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
        TC_TRACE(12, j);
      }
    }
  } else if (warp == C::PV_WARP) {
    // ------------------------------ MMA issuer: O += P V ------------------------
    if (lane == 0 && nTiles > 0) {
      constexpr uint32_t idescO = instr_desc(HD, true);
      bool ok = true;
      for (int t = 0; ok && t < nTiles; t++) {
        const int s = t % C::V_SLOTS, b = t & 1;
        ok = mbar_wait(smem_u32(&bars.fullV[s]), (t / C::V_SLOTS) & 1, &sAbort);
        TC_TRACE(13, t);
        if (ok) ok = mbar_wait(smem_u32(&bars.pReady[b]), (t >> 1) & 1, &sAbort);
        if (!ok) break;
        TC_TRACE(14, t);
        tc_fence_after_sync();
        const uint32_t dV = sV + s * C::KV_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; kk++) {
          // V is [keys][hd] (MN-major B): 16 keys = 2048 bytes further per step;
          // LBO = next 64 columns of hd, SBO = next 8 keys.
          const uint64_t bDesc = smem_desc(dV + kk * 2048, BK * 128, 1024);
          if (C::P_SMEM) {
            // P: [128 rows][BK keys] f16, K-major, 64-key chunks of 128-byte rows
            const uint64_t aDesc =
                smem_desc(sP + (b % C::PB) * C::P_BYTES + (kk >> 2) * (BM * 128) + (kk & 3) * 32,
                          16, 1024);
            mma_f16_ss(tmem + C::O_COL, aDesc, bDesc, idescO, (t > 0 || kk > 0) ? 1u : 0u);
          } else {
            // P: f16 pairs, 8 columns of TMEM per 16 keys
            mma_f16_ts(tmem + C::O_COL, tmem + C::P_COL + b * C::P_STRIDE + kk * 8, bDesc, idescO,
                       (t > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(smem_u32(&bars.emptyV[s]));
        tc_commit(smem_u32(&bars.pvDone[b]));
        TC_TRACE(15, t);
      }
    }
  } else {
    // ------------------------------ softmax + epilogue ------------------------
    // Every softmax warp runs every iteration (and its named barriers) even after a
    // failed wait, so that no warp is left alone at a barrier; work is skipped
    // once `ok` is false.
    const uint32_t laneBase = (uint32_t)((warp & 3) * 32) << 16;
    const int col0 = part * CW;  // first score column of this thread
    float mref = kNegSeed, l = 0.f;
    if (p.sinks) {
      mref = p.sinks[h];  // log2 domain: sink * ln2 * log2e
      if (part == 0) l = 1.f;
    }
    bool ok = true;
    for (int j = 0; j < nTiles; j++) {
      const int b = j & 1;
      const int key0 = (kt0 + j) * BK + col0;
      uint32_t sv[CW];
      float mxLocal = -INFINITY;
      TC_TRACE(0, j);
      if (ok) ok = mbar_wait(smem_u32(&bars.sFull[b]), (j >> 1) & 1, &sAbort);
      if (ok) {
        tc_fence_after_sync();
        TC_TRACE(1, j);
#pragma unroll
        for (int c = 0; c < CW; c += 32)
          tmem_ld32(tmem + laneBase + b * C::S_COLS + col0 + c,
                    *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
        tmem_wait_ld();
        if (C::P_SMEM || C::P_OWN_COLS) {  // S(j) is in registers: its buffer may take S(j+2)
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars.sFree[b]));
        }
        TC_TRACE(2, j);
        const bool fullTile = lo <= key0 && end >= key0 + CW - 1;
        if (p.hasKeyBias) {
          // columns [b0, b1) of this tile get the bias (select, no branch per element)
          const int b0 = p.biasStart - key0, b1 = p.biasEnd - key0;
#pragma unroll
          for (int c = 0; c < CW; c++) {
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
          for (int c = 0; c < CW; c++)
            sv[c] = ((unsigned)(c - c0) <= span) ? sv[c] : 0xff800000u;  // -inf
        }
        // Row max with four independent chains of 3-input max.
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < CW; c += 8) {
#pragma unroll
          for (int u = 0; u < 4; u++)
            mx4[u] = max3(mx4[u], __uint_as_float(sv[c + 2 * u]), __uint_as_float(sv[c + 2 * u + 1]));
        }
        mxLocal = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      if (SPLIT == 2) {
        // The two threads of a row swap their partial maxima (buffer by tile parity:
        // the next write to a slot comes two barriers later).
        sRowMax[b][tid] = mxLocal;
        named_barrier_sync(1, C::SOFTMAX_THREADS);
        mxLocal = fmaxf(mxLocal, sRowMax[b][tid ^ 128]);
      }
      if (ok) {
        const float mx = mxLocal * kLog2e;
        // Lazy rescale: only when some row's max grew by more than 2^8 (whole warp
        // together, because TMEM loads/stores are warp-collective; both column parts
        // of a row see the same numbers and so take the same decision).
        const bool grow = mx > mref + kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // A row still at the seed has seen no key: its accumulator row is exactly zero and
          // needs no pass.  When only such rows have grown, they alone move; the pass over O,
          // when there is one, moves every row.
          const bool scaleO = j > 0 && __any_sync(0xffffffffu, grow && mref != kNegSeed);
          const float mnew = (scaleO || j == 0 || mref == kNegSeed) ? fmaxf(mref, mx) : mref;
          const float f = fast_exp2(mref - mnew);
          mref = mnew;
          l *= f;
          if (scaleO) {
            // O holds the tiles up to j-1: wait for the last P V to land, then scale
            // this thread's share of the accumulator columns.
            ok = mbar_wait(smem_u32(&bars.pvDone[(j - 1) & 1]), ((j - 1) >> 1) & 1, &sAbort);
            if (ok) {
              tc_fence_after_sync();
#pragma unroll
              for (int c = 0; c < OW; c += 32) {
                uint32_t o[32];
                tmem_ld32(tmem + laneBase + C::O_COL + part * OW + c, o);
                tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < 32; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
                tmem_st32(tmem + laneBase + C::O_COL + part * OW + c, o);
              }
            }
          }
        }
      }
      if (ok) {
        TC_TRACE(3, j);
        // p = 2^(s*log2e - mref): one packed FFMA per two scores, MUFU or polynomial,
        // four independent packed sums; packed to f16 pairs.
        const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-mref, -mref);
        float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f),
                          make_float2(0.f, 0.f)};
        uint32_t pk[CW / 2];
#pragma unroll
        for (int c = 0; c < CW; c += 2) {
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
          // The buffer was last read by P V(j - P_BUFS).
          if (j >= C::P_BUFS)
            ok = mbar_wait(smem_u32(&bars.pvDone[(j - C::P_BUFS) & 1]),
                           ((j - C::P_BUFS) >> 1) & 1, &sAbort);
          if (ok) {
            // Row of the A operand: 16-byte units (8 keys) swizzled by row & 7.
            const uint32_t rowBase = sP + (b % C::PB) * C::P_BYTES + rowInTile * 128;
#pragma unroll
            for (int u = 0; u < CW / 8; u++) {
              const int U = part * (CW / 8) + u;
              const uint32_t addr =
                  rowBase + (U >> 3) * (BM * 128) + (((U & 7) ^ (rowInTile & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[4 * u]),
                           "r"(pk[4 * u + 1]), "r"(pk[4 * u + 2]), "r"(pk[4 * u + 3])
                           : "memory");
            }
            fence_proxy_async();  // generic-proxy stores -> visible to the tensor core
          }
        } else {
          static_assert(PSMEM || (CW / 2) % 32 == 0, "P part must be whole 32-column stores");
          // P's own columns were last read by P V(j-2).
          if (C::P_OWN_COLS && j >= 2)
            ok = mbar_wait(smem_u32(&bars.pvDone[b]), ((j - 2) >> 1) & 1, &sAbort);
#pragma unroll
          for (int c = 0; c < CW / 2; c += 32)
            tmem_st32(tmem + laneBase + C::P_COL + b * C::P_STRIDE + part * (CW / 2) + c,
                      *reinterpret_cast<uint32_t(*)[32]>(&pk[c & ~31]));
          tmem_wait_st();
        }
        TC_TRACE(4, j);
        if (ok) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars.pReady[b]));
        }
        TC_TRACE(5, j);
      }
    }

    // Epilogue: O / l -> f16 -> global.  Rows that saw no key are zeros.
    if (SPLIT == 2) {
      sRowSum[tid] = l;
      named_barrier_sync(1, C::SOFTMAX_THREADS);
      l += sRowSum[tid ^ 128];
    }
    const int64_t row = row0 + rowInTile;
    __half* out = static_cast<__half*>(p.out) + row * ((int64_t)p.qHeads * HD) + (int64_t)h * HD +
                  part * OW;
    if (nTiles > 0 && ok) {
      ok = mbar_wait(smem_u32(&bars.pvDone[(nTiles - 1) & 1]), ((nTiles - 1) >> 1) & 1, &sAbort);
      if (ok) {
        tc_fence_after_sync();
        // a row with an empty band has l = 0 (or only the sink): zeros
        const float invL = (l > 0.f && lo <= end) ? 1.f / l : 0.f;
#pragma unroll
        for (int c = 0; c < OW; c += 32) {
          uint32_t o[32];
          tmem_ld32(tmem + laneBase + C::O_COL + part * OW + c, o);
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
    } else if (nTiles == 0) {
      // No row of this unit sees a key (in a padded batch: every unit past a sequence's end):
      // zeros, consecutive threads on consecutive 16-byte pieces of a row.
      constexpr int kPerRow = HD / 8;
      __half* base = static_cast<__half*>(p.out) + row0 * ((int64_t)p.qHeads * HD) + (int64_t)h * HD;
      for (int i = tid; i < BM * kPerRow; i += C::SOFTMAX_THREADS) {
        const int r = i / kPerRow, c = i - r * kPerRow;
        if (row0 + r < p.qLen)
          reinterpret_cast<uint4*>(base + (int64_t)r * p.qHeads * HD)[c] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }

  // Common exit: every role arrives here, then the allocating warp frees TMEM.
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && sAbort) atomicOr(status, kStatusWaitTimeout);
  if (warp == C::MMA_WARP) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

// ---- host side ------------------------------------------------------------------

template <int HD, bool PSMEM, int SPLIT>
cudaError_t launch(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  using C = Cfg<HD, PSMEM, SPLIT>;
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, p.q, p.qLen, (int64_t)p.qHeads * HD, p.qStride, BM, err) ||
      !make_map(&mk, p.k, p.kvLen, (int64_t)p.kvHeads * HD, p.kvStride, C::BK, err) ||
      !make_map(&mv, p.v, p.kvLen, (int64_t)p.kvHeads * HD, p.kvStride, C::BK, err))
    return cudaErrorInvalidValue;
  auto kern = prefill_tc_kernel<HD, PSMEM, SPLIT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)((p.qLen + BM - 1) / BM), (unsigned)p.qHeads);
  kern<<<grid, C::THREADS, C::SMEM, s>>>(mq, mk, mv, p, status);
  return cudaGetLastError();
}

}  // namespace

bool prefill_tc_supported(const AttnParams& p, int dtype) {
  if (dtype != RT_F16) return false;
  if (p.hd != 64 && p.hd != 128 && p.hd != 256) return false;
  if (p.qLen < 2 || p.qLen >= (1ll << 31) - 256 || p.kvLen >= (1ll << 31) - 256) return false;
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
  switch (p.hd) {
    case 64: return launch<64, false, 1>(p, status, s, err);
    case 128: return launch<128, false, 1>(p, status, s, err);
    case 256: return launch<256, false, 1>(p, status, s, err);
  }
  *err = "unsupported head size";
  return cudaErrorInvalidValue;
}

}  // namespace rt
