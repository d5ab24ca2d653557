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
// Head sizes: 64 and 128 (two S buffers), 256 (the accumulator takes half of tensor
// memory, so there is ONE S buffer — free again as soon as its scores are in a warpgroup's
// registers, which is when the next S is issued — beside the two P buffers; K arrives as
// two 128-column halves and V as two 64-key halves so that every ring slot is 32 KB and
// S keeps the full-rate 128-key tile), and the narrow heads 32, 36, 52, ... (any
// multiple of 4 up to 60) padded to 64 inside the tile: K and V tiles are fetched
// with a 64-column box that starts on the 16-byte boundary at or below the head
// (the columns beside the head belong to its neighbours), Q is staged by the
// softmax threads with zeros in those columns, so the neighbours' columns add
// nothing to the scores, and the output columns they produce are dropped.
//
// Pairs (head sizes 128 and 256).  Two CTAs of a cluster, on two SMs, take two adjacent
// 128-row query tiles of the same head and run every product as ONE tcgen05.mma of
// cta_group::2 (M = 256: 128 rows per CTA, each into its own tensor memory), issued by
// the even CTA.  The B operand of such a product is split between the two CTAs' shared
// memories — each holds 64 of a K tile's 128 keys, and half of a V tile's columns — so
// each SM fetches only half of every K/V tile from the L2 (that traffic is what limits
// this kernel: it burns power at head size 128 and its latency cannot be hidden behind
// one SM's 160 KB of tile buffers at head size 256) and its ring holds twice as many
// tiles.  Everything else is per CTA as described above; the odd CTA's MMA warps idle.
// The peer's loads report to the even CTA's barriers (the cta_group::2 form of the bulk
// tensor copy), its softmax warps arrive on them remotely, and the even CTA's commits
// arrive on both CTAs' barriers.  Every copy has one destination CTA.
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

#ifndef RT_TC3_WIDE_STORES
#define RT_TC3_WIDE_STORES 1  // 32-byte stores in the read-out where the rows allow
#endif
#ifndef RT_TC3_CHECK_EMPTY
#define RT_TC3_CHECK_EMPTY 1   // look a padded batch's length up before asking for the Q tile
#endif
#ifndef RT_TC3_RELAXED
#define RT_TC3_RELAXED 0
#endif
constexpr int kThreads3 = 384;
constexpr int kRegsSoftmax3 = 216, kRegsOther3 = 64;  // 2*128*216 + 128*64 <= 384*168
constexpr int BK3 = 128;
constexpr int kMaxSlots = 12;

template <int HD, bool PAIR>
struct Cfg3 {
  static constexpr int CHUNKS = HD / 64;                       // 64-column chunks of a row
  static constexpr int Q_BYTES = BM * HD * 2;
  // One CTA alone at head size 256: K and V tiles arrive in two parts (K: 128 columns each,
  // V: 64 keys each) so that a ring slot is 32 KB.  A pair holds half tiles anyway.
  static constexpr bool SPLIT = HD == 256 && !PAIR;
  static constexpr int KP = SPLIT ? 2 : 1, VP = SPLIT ? 2 : 1;  // parts per key tile
  static constexpr int K_ROWS = PAIR ? BK3 / 2 : BK3;           // keys of a K tile held by this CTA
  static constexpr int K_CHUNKS = SPLIT ? 2 : CHUNKS;           // 64-column chunks in one K part
  static constexpr int V_ROWS = SPLIT ? 64 : BK3;               // keys in one V part
  static constexpr int V_CHUNKS = PAIR ? CHUNKS / 2 : CHUNKS;   // 64-column chunks of V held here
  static constexpr int K_BYTES = K_CHUNKS * K_ROWS * 128, V_BYTES = V_CHUNKS * V_ROWS * 128;
  static constexpr int SLOT_BYTES = K_BYTES > V_BYTES ? K_BYTES : V_BYTES;
  static constexpr int SLOTS_FIT = (225 * 1024 - Q_BYTES) / SLOT_BYTES;
  static constexpr int SLOTS = SLOTS_FIT > kMaxSlots ? kMaxSlots : SLOTS_FIT;
  static constexpr int SMEM = Q_BYTES + SLOTS * SLOT_BYTES + 1024;
  // Tensor memory: S | O | P up to head size 128 (two S buffers, 2 x 64 columns of P behind
  // the accumulator); at head size 256 the accumulator takes the upper half and one S buffer
  // shares the lower half with the two P buffers.
  static constexpr int S_BUFS = HD == 256 ? 1 : 2;
  static constexpr int O_COL = 2 * BK3;
  static constexpr int P_COL = HD == 256 ? BK3 : O_COL + 128;
  static constexpr int TMEM_COLS = 512;
  static constexpr int CTAS = PAIR ? 2 : 1;
  static_assert(SLOTS >= KP + VP + 1, "ring too small");
  static_assert(O_COL + HD <= TMEM_COLS, "tensor memory budget");
  static_assert(!PAIR || HD >= 128, "a pair splits V into 64-column chunks");
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

// ---- the cta_group::2 forms (a pair of CTAs on two SMs acting as one MMA unit) ----------

// In the shared window of a cluster, bit 24 of an address tells the two CTAs of a pair
// apart: cleared it names the even CTA's copy of the same location.
constexpr uint32_t kPeerBit = 1u << 24;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrives on a barrier anywhere in the cluster (here: the even CTA's copy).  Default
// semantics (release at CTA scope): what the consumer reads — P in this CTA's tensor memory
// — is ordered by the tcgen05 fences around the arrival, and a cluster-scope release on
// every arrival costs the arriving warp about a thousand cycles (measured).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Tiled load into this CTA's shared memory whose completion is counted on the EVEN CTA's
// barrier at the same offset (the pair's MMA issuer waits there for both halves).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], "
      "[%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar & ~kPeerBit)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dstSmem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dstSmem),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
// Arrives once on the barrier at `bar`'s offset in each CTA of the pair when all MMAs issued
// so far by this thread have completed in both: one commit per CTA, the second one naming
// the odd CTA's copy of the barrier (measured: as fast as a single commit naming both).
__device__ __forceinline__ void tc_commit_one(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  tc_commit_one(bar);
  tc_commit_one(bar | kPeerBit);
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(dTmem),
      "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_f16_ts_pair(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(dTmem),
      "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Instruction descriptor of a pair's product: M = 256 over the two CTAs.
constexpr uint32_t instr_desc_pair(int n, bool bMnMajor) {
  return (instr_desc(n, bMnMajor) & ~(0x1fu << 24)) | ((uint32_t)(256 >> 4) << 24);
}

// PADDED: the head is narrower than the 64 columns the tile holds (see the file header);
// p.hd is the real size, `shift` = (kvh * hd) & 7 the head's first column inside the box.
// PAIR: two CTAs of a cluster share every K/V tile (see the file header).
template <int HD, bool PADDED, bool PAIR>
__global__ void __launch_bounds__(kThreads3, 1)
prefill_tc3_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, const AttnParams p, int* status) {
  using C = Cfg3<HD, PAIR>;
  constexpr int BK = BK3, KP = C::KP, VP = C::VP, NS = C::SLOTS;
  static_assert(!PADDED || (HD == 64 && !PAIR), "narrow heads are padded to 64 columns, one CTA");
  extern __shared__ unsigned char smemRaw[];
  __shared__ Barriers3 bars;
  __shared__ uint32_t sTmemBase;
  __shared__ int sAbort;
  __shared__ int sLoMin[8], sEndMax[8];
  __shared__ float sMref[BM];          // the rows' reference points (log2 domain)
  __shared__ float sL[2][BM];          // the warpgroups' row sums, for the epilogue
  __shared__ volatile int sMaxDone[4];  // per warp of a warpgroup: tiles whose max phase is over

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  TC_TRACE_DECL
  // Long rows first under a causal mask; the two CTAs of a pair take adjacent row tiles.
  const int cta = PAIR ? (int)cluster_ctarank() : 0;
  const int unit = (int)(gridDim.x / C::CTAS) - 1 - (int)(blockIdx.x / C::CTAS);
  const int qTile = unit * C::CTAS + cta;
  const bool leader = cta == 0;
  const int h = blockIdx.y;
  const int kvh = h / (p.qHeads / p.kvHeads);
  const int64_t row0 = (int64_t)qTile * BM;
  const int hd = PADDED ? p.hd : HD;
  const int shift = PADDED ? ((kvh * hd) & 7) : 0;

  const uint32_t smemBase = (smem_u32(smemRaw) + 1023u) & ~1023u;
  const uint32_t sQ = smemBase;
  const uint32_t sRing = sQ + C::Q_BYTES;

  // One CTA alone: the Q tile needs nothing but the CTA's coordinates, so the producer's lane
  // sets up its barrier and starts its copy before the rest of the set-up (tensor memory,
  // the rows' bands, which read sequence lengths from memory) instead of after it.
  constexpr bool EARLY_Q = !PAIR && !PADDED;
  // (In a padded batch the units past a sequence's end see no key and must not pay for a Q
  // tile: the lane looks the length up first.)
  bool earlyQ = false;
  if (EARLY_Q && tid == 8 * 32) {
    mbar_init(smem_u32(&bars.fullQ), 1);
    fence_barrier_init();
    earlyQ = true;
    if (RT_TC3_CHECK_EMPTY && p.seqStride > 0 && !p.segs) {
      const int64_t b0 = row0 / p.seqStride;
      earlyQ = row0 - b0 * p.seqStride < p.seqLens[b0];
    }
    if (earlyQ) {
      prefetch_tensormap(&mapQ);
      mbar_expect_tx(smem_u32(&bars.fullQ), C::Q_BYTES);
      for (int c = 0; c < C::CHUNKS; c++)
        tma_load_2d(sQ + c * (BM * 128), &mapQ, h * HD + c * 64, (int)row0, smem_u32(&bars.fullQ));
    }
  }
  if (tid == 0) {
    sAbort = 0;
    if (!EARLY_Q) mbar_init(smem_u32(&bars.fullQ), 1);
    for (int s = 0; s < kMaxSlots; s++) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&bars.sFull[b]), 1);
      // one arrival per warp of the warpgroup — of both CTAs' warpgroups in a pair, whose
      // arrivals all go to the even CTA, where the MMA issuers wait
      mbar_init(smem_u32(&bars.sFree[b]), 4 * C::CTAS);
      mbar_init(smem_u32(&bars.pReady[b][0]), 4 * C::CTAS);
      mbar_init(smem_u32(&bars.pReady[b][1]), 4 * C::CTAS);
      mbar_init(smem_u32(&bars.pvDone[b]), 1);
    }
    fence_barrier_init();
  }
  if (warp == 9) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(&sTmemBase), C::TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&sTmemBase), C::TMEM_COLS);
      tmem_relinquish();
    }
  }

  // Band of this thread's row, then of the whole unit (one row tile, or the pair's two):
  // the two CTAs of a pair walk the same key tiles, so each works the range out for both —
  // warps 0-3 from its own rows, warps 4-7 from the other CTA's.
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
    int olo = lo, oend = end;   // the row this thread contributes to the unit's range
    if (PAIR && warp >= 4) {
      const int64_t other = (int64_t)(unit * 2 + (1 - cta)) * BM + rowInTile;
      olo = 1, oend = 0;
      if (other < p.qLen) {
        int64_t l64, e64;
        row_band(p, other, l64, e64);
        if (l64 <= e64) olo = (int)l64, oend = (int)e64;
      }
    }
    if (warp < 4 || PAIR) {
      int wl = olo <= oend ? olo : INT_MAX, we = olo <= oend ? oend : -1;
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
    if (warp < 4) {
      if (lane == 0) sMaxDone[warp] = 0;
      sMref[rowInTile] = p.sinks ? p.sinks[h] : kNegSeed;  // sinks arrive in the log2 domain
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // both CTAs' barriers exist before either is signalled from afar
  tc_fence_after_sync();
  TC_TRACE(99, 0);
  const uint32_t tmem = sTmemBase;
  int tileLo = INT_MAX, tileEnd = -1;
#pragma unroll
  for (int w8 = 0; w8 < (PAIR ? 8 : 4); w8++) {
    tileLo = min(tileLo, sLoMin[w8]);
    tileEnd = max(tileEnd, sEndMax[w8]);
  }
  const int kt0 = tileEnd >= 0 ? tileLo / BK : 0;
  const int nTiles = tileEnd >= 0 ? tileEnd / BK - kt0 + 1 : 0;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther3));
    if (warp == 8) {
      // ------------------------------ TMA producer ------------------------------
      // In a pair every CTA loads its own Q tile and its halves of the K/V tiles into its
      // own ring (which both CTAs walk in step: same sequence numbers, same slots); all
      // completions are counted on the even CTA's barriers, where the byte counts expected
      // are the pair's.
      // (a unit that sees no key leaves only after the Q tile it asked for has landed)
      if (EARLY_Q && lane == 0 && nTiles == 0 && earlyQ) mbar_wait(smem_u32(&bars.fullQ), 0, &sAbort);
      if (lane == 0 && nTiles > 0) {
        prefetch_tensormap(&mapK);
        prefetch_tensormap(&mapV);
        auto load = [&](uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
          if (PAIR) tma_load_2d_pair(dst, map, x, y, bar);
          else tma_load_2d(dst, map, x, y, bar);
        };
        if (!PADDED && !earlyQ) {
          prefetch_tensormap(&mapQ);
          if (leader) mbar_expect_tx(smem_u32(&bars.fullQ), C::CTAS * C::Q_BYTES);
          for (int c = 0; c < C::CHUNKS; c++)
            load(sQ + c * (BM * 128), &mapQ, h * HD + c * 64, (int)row0, smem_u32(&bars.fullQ));
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
          const int key0 = (kt0 + j) * BK + cta * C::K_ROWS;   // a pair: 64 keys each
          for (int part = 0; part < KP && ok; part++) {
            int slot;
            if (!slot_for(slot)) return;
            const uint32_t bar = smem_u32(&bars.full[slot]), dst = sRing + slot * C::SLOT_BYTES;
            if (leader) mbar_expect_tx(bar, C::CTAS * C::K_BYTES);
            for (int c = 0; c < C::K_CHUNKS; c++)
              load(dst + c * (C::K_ROWS * 128), &mapK, xKV + (part * C::K_CHUNKS + c) * 64, key0, bar);
          }
        };
        auto load_v = [&](int j) {
          const int key0 = (kt0 + j) * BK;
          const int x0 = xKV + cta * C::V_CHUNKS * 64;          // a pair: half of the columns each
          for (int part = 0; part < VP && ok; part++) {
            int slot;
            if (!slot_for(slot)) return;
            const uint32_t bar = smem_u32(&bars.full[slot]), dst = sRing + slot * C::SLOT_BYTES;
            if (leader) mbar_expect_tx(bar, C::CTAS * C::V_BYTES);
            for (int c = 0; c < C::V_CHUNKS; c++)
              load(dst + c * (C::V_ROWS * 128), &mapV, x0 + c * 64, key0 + part * C::V_ROWS, bar);
          }
        };
        load_k(0);
        for (int j = 0; j < nTiles && ok; j++) {
          if (j + 1 < nTiles) load_k(j + 1);
          if (ok) load_v(j);
        }
      }
    } else if (warp == 9 && leader) {
      // ------------------------------ MMA issuer: S = Q K^T ----------------------
      // The whole warp walks the loop (waits included); the tensor-core instructions
      // run in one elected lane, which keeps their operands in uniform registers.
      if (nTiles > 0) {
        constexpr uint32_t idescS = PAIR ? instr_desc_pair(BK, false) : instr_desc(BK, false);
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version, SW128
        constexpr uint32_t kLboK = (16u >> 4) << 16;
        auto desc = [](uint32_t lo32) { return ((uint64_t)kDescHi << 32) | lo32; };
        auto wait = [&](uint64_t* bar, int parity) {
          return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), (uint32_t)parity, &sAbort)) != 0;
        };
        // descriptors carry the 18-bit offset inside the CTA's window, not the CTA's rank bits
        const uint32_t aLo = ((sQ & 0x3ffffu) >> 4) | kLboK;
        const int kSteps = PADDED ? (shift + hd + 15) / 16 : HD / 16;  // K = 16 per instruction
        bool ok = wait(&bars.fullQ, 0);
#pragma unroll 1
        for (int j = 0; j < nTiles && ok; j++) {
          const int b = j & 1;
          const uint32_t sBuf = C::S_BUFS == 2 ? b * BK : 0;
          const int s0 = seq_k<KP, VP>(j);
          TC_TRACE(10, j);
#pragma unroll
          for (int part = 0; part < KP; part++) {
            const int slot = (s0 + part) % NS;
            ok = wait(&bars.full[slot], ((s0 + part) / NS) & 1);
            // The S buffer is free once its previous contents are in the registers of the
            // warpgroup that took them: S(j-2) with two buffers, S(j-1) with one.
            if (ok && part == 0 && j >= C::S_BUFS) {
              const int jp = j - C::S_BUFS;
              ok = wait(&bars.sFree[jp & 1], (jp >> 1) & 1);
            }
            if (!ok) break;
            tc_fence_after_sync();
            TC_TRACE(11, j);
            if (elect_one()) {
              const uint32_t bLo = (((sRing + slot * C::SLOT_BYTES) & 0x3ffffu) >> 4) | kLboK;
              constexpr int kPerPart = C::K_CHUNKS * 4;  // K = 16 steps in one part
#pragma unroll
              for (int k2 = 0; k2 < kPerPart; k2++) {
                const int kk = part * kPerPart + k2;
                if (PADDED && k2 >= kSteps) break;
                const uint32_t aOff = (kk >> 2) * ((BM * 128) >> 4) + (kk & 3) * 2;
                const uint32_t bOff = (k2 >> 2) * ((C::K_ROWS * 128) >> 4) + (k2 & 3) * 2;
                if (PAIR) mma_f16_ss_pair(tmem + sBuf, desc(aLo + aOff), desc(bLo + bOff), idescS, kk > 0);
                else mma_f16_ss(tmem + sBuf, desc(aLo + aOff), desc(bLo + bOff), idescS, kk > 0);
              }
              if (PAIR) {
                tc_commit_pair(smem_u32(&bars.empty[slot]));
                if (part == KP - 1) tc_commit_pair(smem_u32(&bars.sFull[b]));
              } else {
                tc_commit(smem_u32(&bars.empty[slot]));
                if (part == KP - 1) tc_commit(smem_u32(&bars.sFull[b]));
              }
            }
            __syncwarp();
            TC_TRACE(12, j);
          }
        }
      }
    } else if (warp == 10 && leader) {
      // ------------------------------ MMA issuer: O += P V ------------------------
      if (nTiles > 0) {
        constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
        constexpr uint32_t kLboV = ((uint32_t)(C::V_ROWS * 128) >> 4) << 16;  // next 64 columns of hd
        auto desc = [](uint32_t lo32) { return ((uint64_t)kDescHi << 32) | lo32; };
        auto wait = [&](uint64_t* bar, int parity) {
          return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), (uint32_t)parity, &sAbort)) != 0;
        };
        const uint32_t idescO = PAIR ? instr_desc_pair(HD, true)
                                     : instr_desc(PADDED ? ((shift + hd + 15) & ~15) : HD, true);
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < nTiles && ok; j++) {
          const int b = j & 1;
          const int s0 = seq_v<KP, VP>(j, nTiles);
          const uint32_t pCol = tmem + C::P_COL + b * 64;
#pragma unroll
          for (int half = 0; half < 2; half++) {
            const int part = VP == 2 ? half : 0;
            const int slot = (s0 + part) % NS;
            TC_TRACE(13 + 3 * half, j);
            if (VP == 2 || half == 0) ok = wait(&bars.full[slot], ((s0 + part) / NS) & 1);
            TC_TRACE(14 + 3 * half, j);
            if (ok) ok = wait(&bars.pReady[b][half], (j >> 1) & 1);
            if (!ok) break;
            tc_fence_after_sync();
            TC_TRACE(15 + 3 * half, j);
            if (elect_one()) {
              const uint32_t bLo = (((sRing + slot * C::SLOT_BYTES) & 0x3ffffu) >> 4) | kLboV;
#pragma unroll
              for (int k2 = 0; k2 < 4; k2++) {
                const int kk = half * 4 + k2;              // 16 keys per step
                const int kLocal = VP == 2 ? k2 : kk;       // within this part's rows
                const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;
                if (PAIR) mma_f16_ts_pair(tmem + C::O_COL, pCol + kk * 8, desc(bLo + kLocal * (2048 >> 4)), idescO, acc);
                else mma_f16_ts(tmem + C::O_COL, pCol + kk * 8, desc(bLo + kLocal * (2048 >> 4)), idescO, acc);
              }
              if (PAIR) {
                if (half == 1) {
                  tc_commit_pair(smem_u32(&bars.empty[slot]));
                  tc_commit_pair(smem_u32(&bars.pvDone[b]));
                }
              } else {
                if (VP == 2 || half == 1) tc_commit(smem_u32(&bars.empty[slot]));
                if (half == 1) tc_commit(smem_u32(&bars.pvDone[b]));
              }
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
    const uint32_t sCol = tmem + laneBase + (C::S_BUFS == 2 ? g * BK : 0);
    const uint32_t pCol = tmem + laneBase + C::P_COL + g * 64;
    const uint32_t oCol = tmem + laneBase + C::O_COL;
    // where the MMA issuers wait for this warp: this CTA, or the even CTA of the pair
    auto arrive = [&](uint64_t* bar) {
      if (PAIR && !leader) mbar_arrive_cluster(smem_u32(bar) & ~kPeerBit);
      else mbar_arrive(smem_u32(bar));
    };
    bool ok = true;

    if (PADDED && nTiles > 0) {
      // Q tile by hand: 16-byte units of the swizzled K-major layout, the head's columns at
      // [shift, shift + hd), zeros beside them and in rows past the end.
      const __half* qg = static_cast<const __half*>(p.q) + (int64_t)h * hd;
      for (int u = tid; u < BM * 8; u += 256) {
        const int r = u >> 3, unit8 = u & 7;
        const int64_t row = row0 + r;
        __align__(16) __half vals[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
          const int c = unit8 * 8 + e - shift;
          vals[e] = (row < p.qLen && c >= 0 && c < hd) ? qg[row * p.qStride + c] : __half(0.f);
        }
        const uint32_t addr = sQ + r * 128 + ((unit8 ^ (r & 7)) << 4);
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
      TC_TRACE(0, j);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars.sFull[g]), (j >> 1) & 1, &sAbort));
      if (!ok) break;  // the whole warp leaves together
      tc_fence_after_sync();
      TC_TRACE(1, j);
      uint32_t sv[BK];
#pragma unroll
      for (int c = 0; c < BK; c += 32)
        tmem_ld32(sCol + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
      tmem_wait_ld();
      TC_TRACE(2, j);
      // S(j) is in registers: its buffer may take the next S
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) arrive(&bars.sFree[g]);
      TC_TRACE(20, j);
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
      TC_TRACE(21, j);

      // ---- max phase, in tile order across the two warpgroups ----
      if (j > 0) {
        // (an acquire load pairs with the release store below: what the other warpgroup's
        // warp wrote before it — reference points, its rescale of O — is visible after it)
        bool arrived = false;
        const uint32_t doneAddr = smem_u32(const_cast<int*>(&sMaxDone[w]));
        for (int i = 0; i < (1 << 22); i++) {
          int done;
#if RT_TC3_RELAXED
          (void)doneAddr;
          done = sMaxDone[w];
#else
          asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(done) : "r"(doneAddr) : "memory");
#endif
          if (done >= j) { arrived = true; break; }
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
        tc_fence_after_sync();
      }
      TC_TRACE(22, j);
      float mref = sMref[rowInTile];
      if (mref != seen) {  // the other warpgroup moved the reference point since this one last looked
        l *= fast_exp2(seen - mref);
        seen = mref;
      }
      const bool grow = mx > mref + kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow)) {
        // A row whose reference point is still the seed has seen no key in any tile so far:
        // its accumulator row is exactly zero and needs no pass (the rows of a band's first,
        // partly masked tile meet their first keys in the second one).  When only such rows
        // have grown, they alone move; the pass over O, when there is one, moves every row.
        const bool pass = j > 0 && __any_sync(0xffffffffu, grow && mref != kNegSeed);
        const float mnew = (pass || j == 0 || mref == kNegSeed) ? fmaxf(mref, mx) : mref;
        const float f = fast_exp2(mref - mnew);
        if (pass) {
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
#if RT_TC3_RELAXED
      if (lane == 0) sMaxDone[w] = j + 1;
#else
      if (lane == 0)
        asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<int*>(&sMaxDone[w]))),
                     "r"(j + 1)
                     : "memory");
#endif
      TC_TRACE(3, j);

      // ---- exponentials, P in two halves ----
      // P's own columns were last read by P V(j-2).
      if (j >= 2) {
#if RT_TC3_RELAXED
        // (nearly always complete by now: one look by one lane, the full wait only if not)
        const uint32_t pvBar = smem_u32(&bars.pvDone[g]);
        const uint32_t pvPar = ((j >> 1) - 1) & 1;
        int done = 0;
        if (lane == 0) done = mbar_test_wait(pvBar, pvPar);
        if (!__shfl_sync(0xffffffffu, done, 0)) {
          ok = __all_sync(0xffffffffu, mbar_wait(pvBar, pvPar, &sAbort));
          if (!ok) break;
        }
#else
        ok = __all_sync(0xffffffffu,
                        mbar_wait(smem_u32(&bars.pvDone[g]), ((j >> 1) - 1) & 1, &sAbort));
        if (!ok) break;
#endif
      }
      TC_TRACE(6, j);
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
        TC_TRACE(7 + half, j);
        tmem_st32(pCol + half * 32, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) arrive(&bars.pReady[g][half]);
        TC_TRACE(4 + half, j);
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
    const bool wide = !PADDED && (reinterpret_cast<uintptr_t>(p.out) & 31u) == 0;   // rows start on 32 bytes
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
              if (RT_TC3_WIDE_STORES && wide) {
                // a row's piece is then one full 32-byte sector per request instead of half of
                // one (the stores of a warp go to 32 different rows)
#pragma unroll
                for (int v = 0; v < 2; v++)
                  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(
                                   out + c + 16 * v),
                               "r"(wds[8 * v]), "r"(wds[8 * v + 1]), "r"(wds[8 * v + 2]), "r"(wds[8 * v + 3]),
                               "r"(wds[8 * v + 4]), "r"(wds[8 * v + 5]), "r"(wds[8 * v + 6]), "r"(wds[8 * v + 7])
                               : "memory");
              } else {
#pragma unroll
                for (int v = 0; v < 4; v++) reinterpret_cast<uint4*>(out + c)[v] = pkd[v];
              }
            }
          }
        }
      }
    } else if (nTiles == 0) {
      // No row of this unit sees a key (in a padded batch: every unit past a sequence's end).
      if (PADDED) {
        if (row < p.qLen)
          for (int c = g * (hd / 2); c < (g + 1) * (hd / 2); c += 2)
            *reinterpret_cast<__half2*>(out + c) = __floats2half2_rn(0.f, 0.f);
      } else {
        // 16-byte stores, consecutive threads on consecutive pieces of a row: a thread per
        // row writing its own row in 4-byte pieces made such a unit cost ~9 us of store
        // traffic, a third of a padded batch's time.
        constexpr int kPerRow = HD / 8;
        __half* base = static_cast<__half*>(p.out) + row0 * ((int64_t)p.qHeads * HD) + (int64_t)h * HD;
        for (int i = tid; i < BM * kPerRow; i += 256) {
          const int r = i / kPerRow, c = i - r * kPerRow;
          if (row0 + r < p.qLen)
            reinterpret_cast<uint4*>(base + (int64_t)r * p.qHeads * HD)[c] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    }
  }

  // Common exit: every role arrives here, then the allocating warp frees TMEM.  In a pair
  // neither CTA leaves while the other may still read its shared memory or signal it.
  tc_fence_before_sync();
  __syncthreads();
  if (PAIR) cluster_sync_all();
  if (tid == 0 && sAbort) atomicOr(status, kStatusWaitTimeout);
  if (warp == 9) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem, C::TMEM_COLS);
    else tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

template <int HD, bool PADDED, bool PAIR>
cudaError_t launch3(const AttnParams& p, int* status, cudaStream_t s, std::string* err) {
  using C = Cfg3<HD, PAIR>;
  CUtensorMap mq, mk, mv;
  // The narrow-head form reads Q with plain loads; its K/V maps span the real columns,
  // so a box that runs past the last head reads zeros there.
  const int64_t qCols = (int64_t)p.qHeads * p.hd, kvCols = (int64_t)p.kvHeads * p.hd;
  if ((!PADDED && !make_map(&mq, p.q, p.qLen, qCols, p.qStride, BM, err)) ||
      !make_map(&mk, p.k, p.kvLen, kvCols, p.kvStride, C::K_ROWS, err) ||
      !make_map(&mv, p.v, p.kvLen, kvCols, p.kvStride, C::V_ROWS, err))
    return cudaErrorInvalidValue;
  if (PADDED) mq = mk;  // unused by the kernel; a valid map all the same
  auto kern = prefill_tc3_kernel<HD, PADDED, PAIR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  if (e != cudaSuccess) return e;
  const unsigned tiles = (unsigned)((p.qLen + BM - 1) / BM);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((tiles + C::CTAS - 1) / C::CTAS * C::CTAS, (unsigned)p.qHeads);
  cfg.blockDim = dim3(kThreads3);
  cfg.dynamicSmemBytes = C::SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C::CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = PAIR ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, p, status);
  return e != cudaSuccess ? e : cudaGetLastError();
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

// Pairs of CTAs need two row tiles of the same head and one of the head sizes whose V tile
// splits into 64-column chunks.
bool prefill_tc3_pair_supported(const AttnParams& p, int dtype) {
  return prefill_tc3_supported(p, dtype) && (p.hd == 128 || p.hd == 256) && p.qLen > BM;
}

cudaError_t launch_prefill_tc3(const AttnParams& p, bool pair, int* status, cudaStream_t s,
                               std::string* err) {
  if (pair) {
    return p.hd == 128 ? launch3<128, false, true>(p, status, s, err)
                       : launch3<256, false, true>(p, status, s, err);
  }
  switch (p.hd) {
    case 64: return launch3<64, false, false>(p, status, s, err);
    case 128: return launch3<128, false, false>(p, status, s, err);
    case 256: return launch3<256, false, false>(p, status, s, err);
  }
  return launch3<64, true, false>(p, status, s, err);
}

}  // namespace rt
