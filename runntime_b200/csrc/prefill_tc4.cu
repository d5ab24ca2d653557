// Persistent tensor-core prefill attention: one CTA per SM walks a queue of (query tile,
// head) units, and the units overlap.
//
// The alternating-warpgroup kernel (prefill_tc3.cu) runs one unit per CTA: a CTA starts
// with an empty pipeline (Q and the first K tile on their way from memory, the first S,
// the first softmax before the first P V can be issued) and ends with a drain (last
// softmax, last P V, read-out of the accumulator) — about 13 000 cycles in which the tensor
// pipe mostly idles, against about 2 100 per key tile in between.  A sliding-window layer
// has 5-10 key tiles per unit and sequences padded to a common length have fewer still, so
// there the fill and the drain are most of the time.  Here the roles of that kernel — a
// TMA producer warp, one warp issuing S = Q K^T, one issuing O += P V, two softmax
// warpgroups taking alternate key tiles — each run their own loop over the units a
// scheduler warp draws from a device-wide counter, every barrier's phase follows a count
// that runs on across units, and a fourth warpgroup does nothing but read finished units
// out of tensor memory.  The tile sequence of the CTA is one long alternation of the two
// softmax warpgroups: while the one that took a unit's last tile finishes its softmax, the
// producer has fetched the next unit's Q and K, the S issuer has computed its first scores
// and the other warpgroup is in its first softmax; when the last P V has landed, the
// read-out warps scale the rows by 1/l (handed over through shared memory), round and store
// them.  Only the accumulator is not doubled: the first P V of a unit waits until the
// previous unit's rows have left tensor memory.
//
// Work queue: unit i is row tile (units - 1 - i % units) of head i / units (long rows
// first under a causal mask); the scheduler warp draws i with one atomicAdd, works out
// the key-tile range of the unit's 128 rows, zero-fills units that see no key itself and
// publishes the others through a four-entry queue in shared memory that every other warp
// reads in order.  The last CTA to draw past the end rewinds the counter for the next
// launch (no memset between launches, so the launch can sit in a CUDA graph).
//
// Head sizes 64 and 128 (two Q buffers, two S buffers) and 256 (one Q buffer — the next Q is
// fetched when the unit's last S has been computed — and one S buffer beside the two P
// buffers, as in prefill_tc3.cu).  f16.  Semantics are the 'attn' op's (see rt_attn.h);
// replaces attnFlash (packages/runntime/src/core/kernels/attention/attnFlash.ts:93-276).
// Every wait is bounded; a wait that runs out sets the status word and the CTA winds down
// through the common exit that frees its tensor memory.
#include <climits>

#include "common.cuh"
#include "sm100.cuh"
#include "tc_common.cuh"

namespace rt {
namespace {

using namespace sm100;
using namespace tc;

#ifndef RT_TC4_ONE_Q
#define RT_TC4_ONE_Q 256   // head sizes from here up have one Q buffer (128: one more ring slot, +2 % measured)
#endif
constexpr int kThreads4 = 512;
constexpr int kRegsSoftmax4 = 216, kRegsOther4 = 40;  // 2*128*216 + 2*128*40 = 512*128
constexpr int BK4 = 128;
constexpr int kDescSlots = 4;     // queue entries between the scheduler and the other warps
constexpr int kDescReaders = 15;  // eight softmax warps, the producer, the two MMA issuers, four read-out warps

template <int HD>
struct Cfg4 {
  static constexpr int CHUNKS = HD / 64;                  // 64-column chunks of a row
  static constexpr int Q_BYTES = BM * HD * 2;
  static constexpr int Q_BUFS = HD >= RT_TC4_ONE_Q ? 1 : 2;
  // Head size 256: K and V tiles arrive in two parts (K: 128 columns each, V: 64 keys each)
  // so that a ring slot is 32 KB.
  static constexpr bool SPLIT = HD == 256;
  static constexpr int KP = SPLIT ? 2 : 1, VP = SPLIT ? 2 : 1;
  static constexpr int K_CHUNKS = SPLIT ? 2 : CHUNKS;
  static constexpr int V_ROWS = SPLIT ? 64 : BK4;
  static constexpr int K_BYTES = K_CHUNKS * BK4 * 128, V_BYTES = CHUNKS * V_ROWS * 128;
  static constexpr int SLOT_BYTES = K_BYTES > V_BYTES ? K_BYTES : V_BYTES;
  static constexpr int SLOTS_FIT = (224 * 1024 - Q_BUFS * Q_BYTES) / SLOT_BYTES;
  static constexpr int SLOTS_MAX = HD == 64 ? 11 : 12;   // (the barriers of a twelfth slot would not fit)
  static constexpr int SLOTS = SLOTS_FIT > SLOTS_MAX ? SLOTS_MAX : SLOTS_FIT;
  static constexpr int SMEM = Q_BUFS * Q_BYTES + SLOTS * SLOT_BYTES;   // 1024-byte aligned by declaration
  // Tensor memory: S | O | P up to head size 128 (two S buffers, 2 x 64 columns of P behind
  // the accumulator); at head size 256 the accumulator takes the upper half and one S buffer
  // shares the lower half with the two P buffers.
  static constexpr int S_BUFS = HD == 256 ? 1 : 2;
  static constexpr int O_COL = 2 * BK4;
  static constexpr int P_COL = HD == 256 ? BK4 : O_COL + 128;
  static constexpr int TMEM_COLS = 512;
  static_assert(SLOTS >= KP + VP + 1, "ring too small");
};

struct Desc4 {
  int item;     // unit index, or -1: no more work
  int kt0;      // first key tile of the unit's band
  int nTiles;   // key tiles in the band (at least one: empty units are not published)
  // Padded-batch form, when the unit's 128 rows lie in one sequence: the sequence's first row
  // and its length, looked up once by the scheduler (else seqBase = -1 and every thread
  // works its row's band out from the arguments).
  int seqBase, seqLen;
  int pad[3];
};

// The band of one row, from the unit's descriptor where that has the sequence (no division,
// no load), else as row_band does.
__device__ __forceinline__ void row_band4(const AttnParams& p, const Desc4& d, int64_t row, int& lo,
                                          int& end) {
  lo = 1, end = 0;   // empty
  if (row >= p.qLen) return;
  int64_t l64, e64;
  if (d.seqBase >= 0) {
    if (row - d.seqBase >= d.seqLen) return;
    const int64_t qPos = p.qPosOffset + row, last = (int64_t)d.seqBase + d.seqLen - 1;
    l64 = qPos - p.wl;
    if (l64 < d.seqBase) l64 = d.seqBase;
    e64 = qPos + p.wr;
    if (e64 > last) e64 = last;
    if (e64 > p.kvLen - 1) e64 = p.kvLen - 1;
  } else {
    row_band(p, row, l64, e64);
  }
  if (l64 <= e64) lo = (int)l64, end = (int)e64;
}

template <int NS>
struct Shared4 {
  uint64_t full[NS], empty[NS];
  uint64_t fullQ[2], qFree[2];
  uint64_t sFull[2], sFree[2], pReady[2][2], pvDone[2];
  uint64_t oFree, lReady;
  uint64_t descFull[kDescSlots], descFree[kDescSlots];
  Desc4 desc[kDescSlots];
  float mref[BM];        // the rows' reference points (log2 domain), current unit
  float lOther[BM];      // mailbox: the row sums of the warpgroup that did not take the last tile ...
  float seenOther[BM];   // ... and the reference points they are relative to
  float invL[BM];        // 1 / row sum of the unit whose accumulator is complete, for the read-out warps
  int maxDone[4];        // per warp of a warpgroup: tiles (CTA-wide count) whose max phase is over
  int lWritten[4], lRead[4];   // mailbox sequence numbers, per warp of a warpgroup
  uint32_t tmemBase;
  int abort;
};

// Ring sequence numbers inside a unit.  The producer issues K(0); then, for every tile j,
// K(j+1) (if there is one) and V(j): K runs one tile ahead of V.
template <int KP, int VP>
__device__ __forceinline__ int seq4_k(int j) { return j == 0 ? 0 : KP + (j - 1) * (KP + VP); }
template <int KP, int VP>
__device__ __forceinline__ int seq4_v(int j, int n) {
  return KP + j * (KP + VP) + (j + 1 < n ? KP : 0);
}

__device__ __forceinline__ int ld_acquire_shared(const int* p) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.s32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_shared(int* p, int v) {
  asm volatile("st.release.cta.shared::cta.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
// Waits (bounded) until *p >= want; the whole warp takes the same decision.
__device__ __forceinline__ bool wait_count(const int* p, int want, volatile int* abortFlag) {
  bool arrived = false;
  for (int i = 0; i < (1 << 22); i++) {
    if (ld_acquire_shared(p) >= want) { arrived = true; break; }
    if ((i & 63) == 63) {
      if (*abortFlag) break;
      __nanosleep(64);
    }
  }
  const bool ok = __all_sync(0xffffffffu, arrived);
  if (!ok) *abortFlag = 1;
  return ok;
}

template <int HD>
__global__ void __launch_bounds__(kThreads4, 1)
prefill_tc4_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                   const __grid_constant__ CUtensorMap mapV, const AttnParams p, int* status,
                   int* work) {
  using C = Cfg4<HD>;
  constexpr int BK = BK4, KP = C::KP, VP = C::VP, NS = C::SLOTS;
  extern __shared__ __align__(1024) unsigned char smemRaw[];   // swizzled tiles need this alignment
  __shared__ Shared4<NS> sh;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  TC_TRACE_DECL
  const int units = (int)((p.qLen + BM - 1) / BM);
  const int total = units * p.qHeads;
  const int group = p.qHeads / p.kvHeads;
  volatile int* abortFlag = &sh.abort;

  const uint32_t smemBase = smem_u32(smemRaw);
  const uint32_t sRing = smemBase + C::Q_BUFS * C::Q_BYTES;
  if (smemBase & 1023u) {   // the declared alignment was not honoured: refuse, loudly
    if (tid == 0) atomicOr(status, kStatusBadState);
    return;
  }

  if (tid == 0) {
    sh.abort = 0;
    for (int s = 0; s < NS; s++) {
      mbar_init(smem_u32(&sh.full[s]), 1);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(smem_u32(&sh.fullQ[b]), 1);
      mbar_init(smem_u32(&sh.qFree[b]), 1);
      mbar_init(smem_u32(&sh.sFull[b]), 1);
      mbar_init(smem_u32(&sh.sFree[b]), 4);       // one arrival per warp of the warpgroup
      mbar_init(smem_u32(&sh.pReady[b][0]), 4);
      mbar_init(smem_u32(&sh.pReady[b][1]), 4);
      mbar_init(smem_u32(&sh.pvDone[b]), 1);
    }
    mbar_init(smem_u32(&sh.oFree), 4);            // the four warps that read a unit out
    mbar_init(smem_u32(&sh.lReady), 4);           // the four warps that took the unit's last tile
    for (int s = 0; s < kDescSlots; s++) {
      mbar_init(smem_u32(&sh.descFull[s]), 1);
      mbar_init(smem_u32(&sh.descFree[s]), kDescReaders);
    }
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&sh.tmemBase), C::TMEM_COLS);
    tmem_relinquish();
  }
  if (tid < 4) sh.maxDone[tid] = 0, sh.lWritten[tid] = 0, sh.lRead[tid] = 0;
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmemBase;

  // Every warp but the scheduler reads the queue in order; entry n sits in slot n % 4.
  auto next_desc = [&](int n, Desc4& d) {
    const int slot = n % kDescSlots;
    const bool ok = __all_sync(
        0xffffffffu, mbar_wait(smem_u32(&sh.descFull[slot]), (uint32_t)(n / kDescSlots) & 1u, abortFlag));
    if (!ok) return false;
    d = sh.desc[slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&sh.descFree[slot]));
    return true;
  };
  auto wait = [&](uint64_t* bar, int parity) {
    return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), (uint32_t)parity & 1u, abortFlag)) != 0;
  };

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther4));
    if (warp == 11) {
      // ------------------------------ scheduler ------------------------------
      const int64_t outStride = (int64_t)p.qHeads * HD;
      int n = 0;
      bool ok = true;
      while (ok) {
        int item = 0;
        if (lane == 0) item = atomicAdd(work, 1);
        item = __shfl_sync(0xffffffffu, item, 0);
        Desc4 d;
        d.item = -1, d.kt0 = 0, d.nTiles = 0, d.seqBase = -1, d.seqLen = 0;
        if (item < total) {
          const int unit = units - 1 - item % units, h = item / units;
          const int64_t row0 = (int64_t)unit * BM;
          if (p.seqStride > 0 && !p.segs) {
            const int64_t b0 = row0 / p.seqStride, base = b0 * p.seqStride;
            if (row0 + BM <= base + p.seqStride) {   // the unit's rows share a sequence
              d.seqBase = (int)base;
              d.seqLen = p.seqLens[b0];
            }
          }
          // the band of the unit's 128 rows: four rows per lane
          int lo = INT_MAX, end = -1;
#pragma unroll
          for (int i = 0; i < BM / 32; i++) {
            int l32, e32;
            row_band4(p, d, row0 + lane + 32 * i, l32, e32);
            if (l32 <= e32) {
              lo = min(lo, l32);
              end = max(end, e32);
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            end = max(end, __shfl_xor_sync(0xffffffffu, end, o));
          }
          if (end < 0) {
            // No row of the unit sees a key: its rows are zeros, written here.
            __half* out = static_cast<__half*>(p.out) + row0 * outStride + (int64_t)h * HD;
            constexpr int kPerRow = HD / 8;   // 16-byte stores per row
            for (int i = lane; i < BM * kPerRow; i += 32) {
              const int r = i / kPerRow, c = i - r * kPerRow;
              if (row0 + r < p.qLen)
                reinterpret_cast<uint4*>(out + r * outStride)[c] = make_uint4(0u, 0u, 0u, 0u);
            }
            continue;
          }
          d.item = item;
          d.kt0 = lo / BK;
          d.nTiles = end / BK - d.kt0 + 1;
        }
        const int slot = n % kDescSlots;
        if (n >= kDescSlots) {
          // Four units ahead of the slowest reader there is nothing to hurry for: poll
          // rarely, so that the softmax warps on this scheduler keep their issue slots.
          const uint32_t bar = smem_u32(&sh.descFree[slot]), parity = (uint32_t)((n / kDescSlots) - 1) & 1u;
          bool freed = false;
          for (int i = 0; i < (1 << 21) && !freed; i++) {
            if (lane == 0) freed = mbar_test_wait(bar, parity);
            freed = __shfl_sync(0xffffffffu, freed, 0);
            if (!freed) {
              if (*abortFlag) break;
              __nanosleep(1000);
            }
          }
          if (!freed) {
            *abortFlag = 1;
            ok = false;
          }
        }
        if (!ok) break;
        if (lane == 0) {
          sh.desc[slot] = d;
          mbar_arrive(smem_u32(&sh.descFull[slot]));   // releases the entry to its readers
        }
        __syncwarp();
        n++;
        if (d.item < 0) {
          // Past the end: the last CTA to get here rewinds the counter for the next launch.
          if (lane == 0 && atomicAdd(work + 1, 1) == (int)gridDim.x - 1) {
            work[1] = 0;
            __threadfence();
            work[0] = 0;
          }
          break;
        }
      }
    } else if (warp == 8) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        prefetch_tensormap(&mapQ);
        prefetch_tensormap(&mapK);
        prefetch_tensormap(&mapV);
      }
      int seq = 0, qn = 0;
      bool ok = true;
      for (int n = 0; ok; n++) {
        Desc4 d;
        if (!next_desc(n, d) || d.item < 0) break;
        if (lane == 0) {
          const int unit = units - 1 - d.item % units, h = d.item / units;
          const int row0 = unit * BM, xKV = (h / group) * HD;
          const int qb = qn % C::Q_BUFS;
          auto slot_for = [&](int& slot) {  // claims the next ring slot, waiting for its release
            slot = seq % NS;
            if (seq >= NS)
              ok = mbar_wait(smem_u32(&sh.empty[slot]), (uint32_t)((seq / NS) - 1) & 1u, abortFlag);
            seq++;
            return ok;
          };
          auto load_k = [&](int j) {
            const int key0 = (d.kt0 + j) * BK;
            for (int part = 0; part < KP && ok; part++) {
              int slot;
              if (!slot_for(slot)) return;
              const uint32_t bar = smem_u32(&sh.full[slot]), dst = sRing + slot * C::SLOT_BYTES;
              mbar_expect_tx(bar, C::K_BYTES);
              for (int c = 0; c < C::K_CHUNKS; c++)
                tma_load_2d(dst + c * (BK * 128), &mapK, xKV + (part * C::K_CHUNKS + c) * 64, key0, bar);
            }
          };
          auto load_v = [&](int j) {
            const int key0 = (d.kt0 + j) * BK;
            for (int part = 0; part < VP && ok; part++) {
              int slot;
              if (!slot_for(slot)) return;
              const uint32_t bar = smem_u32(&sh.full[slot]), dst = sRing + slot * C::SLOT_BYTES;
              mbar_expect_tx(bar, C::V_BYTES);
              for (int c = 0; c < C::CHUNKS; c++)
                tma_load_2d(dst + c * (C::V_ROWS * 128), &mapV, xKV + c * 64, key0 + part * C::V_ROWS, bar);
            }
          };
          // Q goes out before the first K tile: K has to wait for ring slots, which the unit
          // before holds until its last products are through, and the S issuer needs Q first.
          // (With one Q buffer it is free once the last S of the unit before has completed.)
          if (qn >= C::Q_BUFS)
            ok = mbar_wait(smem_u32(&sh.qFree[qb]), (uint32_t)((qn / C::Q_BUFS) - 1) & 1u, abortFlag);
          if (ok) {
            const uint32_t bar = smem_u32(&sh.fullQ[qb]), dst = smemBase + qb * C::Q_BYTES;
            mbar_expect_tx(bar, C::Q_BYTES);
            for (int c = 0; c < C::CHUNKS; c++)
              tma_load_2d(dst + c * (BM * 128), &mapQ, h * HD + c * 64, row0, bar);
          }
          if (ok) load_k(0);
          for (int j = 0; j < d.nTiles && ok; j++) {
            if (j + 1 < d.nTiles) load_k(j + 1);
            if (ok) load_v(j);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        qn++;
      }
    } else if (warp == 9) {
      // ------------------------------ MMA issuer: S = Q K^T ----------------------
      // The whole warp walks the loop (waits included); the tensor-core instructions
      // run in one elected lane, which keeps their operands in uniform registers.
      constexpr uint32_t idescS = instr_desc(BK, false);
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO, version, SW128
      constexpr uint32_t kLboK = (16u >> 4) << 16;
      auto desc = [](uint32_t lo32) { return ((uint64_t)kDescHi << 32) | lo32; };
      int seqBase = 0, qn = 0, tG = 0;
      bool ok = true;
      for (int n = 0; ok; n++) {
        Desc4 d;
        if (!next_desc(n, d) || d.item < 0) break;
        const int qb = qn % C::Q_BUFS;
        const uint32_t aLo = (((smemBase + qb * C::Q_BYTES) & 0x3ffffu) >> 4) | kLboK;
        ok = wait(&sh.fullQ[qb], qn / C::Q_BUFS);
#pragma unroll 1
        for (int j = 0; j < d.nTiles && ok; j++) {
          const int t = tG + j, b = t & 1;
          const uint32_t sBuf = C::S_BUFS == 2 ? b * BK : 0;
          const int s0 = seqBase + seq4_k<KP, VP>(j);
          TC_TRACE(10, t);
#pragma unroll
          for (int part = 0; part < KP; part++) {
            const int slot = (s0 + part) % NS;
            ok = wait(&sh.full[slot], (s0 + part) / NS);
            // The S buffer is free once its previous contents are in the registers of the
            // warpgroup that took them: S(t-2) with two buffers, S(t-1) with one.
            if (ok && part == 0 && t >= C::S_BUFS) {
              const int tp = t - C::S_BUFS;
              ok = wait(&sh.sFree[tp & 1], tp >> 1);
            }
            if (!ok) break;
            tc_fence_after_sync();
            TC_TRACE(11, t);
            if (elect_one()) {
              const uint32_t bLo = (((sRing + slot * C::SLOT_BYTES) & 0x3ffffu) >> 4) | kLboK;
              constexpr int kPerPart = C::K_CHUNKS * 4;  // K = 16 steps in one part
#pragma unroll
              for (int k2 = 0; k2 < kPerPart; k2++) {
                const int kk = part * kPerPart + k2;
                const uint32_t aOff = (kk >> 2) * ((BM * 128) >> 4) + (kk & 3) * 2;
                const uint32_t bOff = (k2 >> 2) * ((BK * 128) >> 4) + (k2 & 3) * 2;
                mma_f16_ss(tmem + sBuf, desc(aLo + aOff), desc(bLo + bOff), idescS, kk > 0);
              }
              tc_commit(smem_u32(&sh.empty[slot]));
              if (part == KP - 1) {
                tc_commit(smem_u32(&sh.sFull[b]));
                // the unit's last S: its Q tile is dead once these products have completed
                if (j == d.nTiles - 1) tc_commit(smem_u32(&sh.qFree[qb]));
              }
            }
            __syncwarp();
            TC_TRACE(12, t);
          }
        }
        tG += d.nTiles;
        seqBase += d.nTiles * (KP + VP);
        qn++;
      }
    } else if (warp == 10) {
      // ------------------------------ MMA issuer: O += P V ------------------------
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kLboV = ((uint32_t)(C::V_ROWS * 128) >> 4) << 16;  // next 64 columns of hd
      constexpr uint32_t idescO = instr_desc(HD, true);
      auto desc = [](uint32_t lo32) { return ((uint64_t)kDescHi << 32) | lo32; };
      int seqBase = 0, qn = 0, tG = 0;
      bool ok = true;
      for (int n = 0; ok; n++) {
        Desc4 d;
        if (!next_desc(n, d) || d.item < 0) break;
#pragma unroll 1
        for (int j = 0; j < d.nTiles && ok; j++) {
          const int t = tG + j, b = t & 1;
          const int s0 = seqBase + seq4_v<KP, VP>(j, d.nTiles);
          const uint32_t pCol = tmem + C::P_COL + b * 64;
#pragma unroll
          for (int half = 0; half < 2; half++) {
            const int part = VP == 2 ? half : 0;
            const int slot = (s0 + part) % NS;
            TC_TRACE(13 + 3 * half, t);
            if (VP == 2 || half == 0) ok = wait(&sh.full[slot], (s0 + part) / NS);
            // a unit's first product overwrites the accumulator: the unit before it must
            // have been read out
            if (ok && j == 0 && half == 0 && qn >= 1) ok = wait(&sh.oFree, qn - 1);
            TC_TRACE(14 + 3 * half, t);
            if (ok) ok = wait(&sh.pReady[b][half], t >> 1);
            if (!ok) break;
            tc_fence_after_sync();
            TC_TRACE(15 + 3 * half, t);
            if (elect_one()) {
              const uint32_t bLo = (((sRing + slot * C::SLOT_BYTES) & 0x3ffffu) >> 4) | kLboV;
#pragma unroll
              for (int k2 = 0; k2 < 4; k2++) {
                const int kk = half * 4 + k2;              // 16 keys per step
                const int kLocal = VP == 2 ? k2 : kk;       // within this part's rows
                const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;
                mma_f16_ts(tmem + C::O_COL, pCol + kk * 8, desc(bLo + kLocal * (2048 >> 4)), idescO, acc);
              }
              if (VP == 2 || half == 1) tc_commit(smem_u32(&sh.empty[slot]));
              if (half == 1) tc_commit(smem_u32(&sh.pvDone[b]));
            }
            __syncwarp();
          }
        }
        tG += d.nTiles;
        seqBase += d.nTiles * (KP + VP);
        qn++;
      }
    } else if (warp >= 12) {
      // ------------------------------ read-out ------------------------------
      // Warp 12 + i reads lanes 32 i .. 32 i + 31 of tensor memory (one query row per lane):
      // when a unit's last product has landed, its rows are scaled by 1/l, rounded to f16 and
      // stored, 16 columns at a time; after the last load the accumulator belongs to the next
      // unit.
      const int rowInTile = (warp - 12) * 32 + lane;
      const uint32_t oCol = tmem + ((uint32_t)((warp - 12) * 32) << 16) + C::O_COL;
      const bool wide = (reinterpret_cast<uintptr_t>(p.out) & 31u) == 0;   // rows start on 32 bytes
      int qn = 0, tG = 0;
      bool ok = true;
      for (int n = 0; ok; n++) {
        Desc4 d;
        if (!next_desc(n, d) || d.item < 0) break;
        const int unit = units - 1 - d.item % units, h = d.item / units;
        const int64_t row = (int64_t)unit * BM + rowInTile;
        const int tLast = tG + d.nTiles - 1;
        ok = wait(&sh.lReady, qn);
        if (!ok) break;
        const float invL = sh.invL[rowInTile];
        ok = wait(&sh.pvDone[tLast & 1], tLast >> 1);
        if (!ok) break;
        tc_fence_after_sync();
        TC_TRACE(30, tLast);
        __half* out = static_cast<__half*>(p.out) + row * ((int64_t)p.qHeads * HD) + (int64_t)h * HD;
#pragma unroll 1
        for (int c = 0; c < HD; c += 16) {
          uint32_t o[16];
          tmem_ld16(oCol + c, o);
          tmem_wait_ld();
          if (c == HD - 16) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.oFree));
          }
          uint32_t pk[8];
#pragma unroll
          for (int x = 0; x < 16; x += 2) {
            const __half2 hp = __floats2half2_rn(__uint_as_float(o[x]) * invL,
                                                 __uint_as_float(o[x + 1]) * invL);
            pk[x / 2] = *reinterpret_cast<const uint32_t*>(&hp);
          }
          if (row < p.qLen) {
            // a 32-byte store where the rows allow it: a row's piece is then one full sector
            // per request (the stores of a warp go to 32 different rows)
            if (wide) {
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(out + c),
                           "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]),
                           "r"(pk[6]), "r"(pk[7])
                           : "memory");
            } else {
              reinterpret_cast<uint4*>(out + c)[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              reinterpret_cast<uint4*>(out + c)[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            }
          }
        }
        TC_TRACE(31, tLast);
        tG += d.nTiles;
        qn++;
      }
    }
  } else {
    // ------------------------------ softmax ------------------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax4));
    const int g = warp >> 2, w = warp & 3;
    const int rowInTile = tid & 127;
    const uint32_t laneBase = (uint32_t)(w * 32) << 16;
    const uint32_t sCol = tmem + laneBase + (C::S_BUFS == 2 ? g * BK : 0);
    const uint32_t pCol = tmem + laneBase + C::P_COL + g * 64;
    const uint32_t oCol = tmem + laneBase + C::O_COL;
    const float seed = kNegSeed;
    int tG = 0;   // tiles of the units before this one (the CTA-wide tile count)
    bool ok = true;
    for (int n = 0; ok; n++) {   // n: units so far (every published unit has a tile)
      int lo, end;   // this thread's row: lo > end unless it sees a key
      int tEnd, keyBase;
      float start;
      {
        Desc4 d;
        if (!next_desc(n, d) || d.item < 0) break;
        const int unit = units - 1 - d.item % units, h = d.item / units;
        row_band4(p, d, (int64_t)unit * BM + rowInTile, lo, end);
        tEnd = tG + d.nTiles;
        keyBase = (d.kt0 - tG) * BK;                 // key0 of tile t is keyBase + t * BK
        start = p.sinks ? p.sinks[h] : seed;         // sinks arrive in the log2 domain
      }
      float seen = start;                            // the reference point l is relative to
      float l = (p.sinks && g == (tG & 1)) ? 1.f : 0.f;   // the sink counts once, in the first tile's warpgroup
      float mref = start;
#pragma unroll 1
      for (int t = tG + ((g - tG) & 1); t < tEnd && ok; t += 2) {
        const int key0 = keyBase + t * BK;
        const bool firstTile = t == tG;
        TC_TRACE(0, t);
        ok = wait(&sh.sFull[g], t >> 1);
        if (!ok) break;  // the whole warp leaves together
        tc_fence_after_sync();
        TC_TRACE(1, t);
        uint32_t sv[BK];
#pragma unroll
        for (int c = 0; c < BK; c += 32)
          tmem_ld32(sCol + c, *reinterpret_cast<uint32_t(*)[32]>(&sv[c]));
        tmem_wait_ld();
        TC_TRACE(2, t);
        // S(t) is in registers: its buffer may take the next S
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.sFree[g]));
        TC_TRACE(20, t);
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
        TC_TRACE(21, t);

        // ---- max phase, in tile order across the two warpgroups and across units ----
        // (the acquire pairs with the release below: what the other warpgroup's warp wrote
        // before it — reference points, its rescale of O — is visible after it)
        if (t > 0) {
          ok = wait_count(&sh.maxDone[w], t, abortFlag);
          if (!ok) break;
          tc_fence_after_sync();
        }
        TC_TRACE(22, t);
        // a unit's first tile starts the rows' reference points; later tiles read them
        if (!firstTile) mref = sh.mref[rowInTile];
        if (mref != seen) {  // the other warpgroup moved the reference point since this one last looked
          l *= fast_exp2(seen - mref);
          seen = mref;
        }
        const bool grow = mx > mref + kRescaleThreshold;
        const bool anyGrow = __any_sync(0xffffffffu, grow);
        if (anyGrow) {
          // A row whose reference point is still the seed has seen no key in any tile so far:
          // its accumulator row is exactly zero and needs no pass.  When only such rows have
          // grown, they alone move; the pass over O, when there is one, moves every row.
          const bool pass = !firstTile && __any_sync(0xffffffffu, grow && mref != seed);
          const float mnew = (pass || firstTile || mref == seed) ? fmaxf(mref, mx) : mref;
          const float f = fast_exp2(mref - mnew);
          if (pass) {
            // O holds the unit's tiles up to j-1 once P V(t-1) has landed (in-order products)
            ok = wait(&sh.pvDone[(t - 1) & 1], (t - 1) >> 1);
            if (!ok) break;
            tc_fence_after_sync();
            // (16 columns at a time: the tile's 128 scores stay in registers meanwhile)
#pragma unroll 1
            for (int c = 0; c < HD; c += 16) {
              uint32_t o[16];
              tmem_ld16(oCol + c, o);
              tmem_wait_ld();
#pragma unroll
              for (int x = 0; x < 16; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * f);
              tmem_st16(oCol + c, o);
            }
            tmem_wait_st();
            tc_fence_before_sync();
          }
          l *= f;
          mref = seen = mnew;
        }
        if (anyGrow || firstTile) sh.mref[rowInTile] = mref;
        __syncwarp();
        if (lane == 0) st_release_shared(&sh.maxDone[w], t + 1);
        TC_TRACE(3, t);

        // ---- exponentials, P in two halves ----
        // P's own columns were last read by P V(t-2).
        if (t >= 2) {
          ok = wait(&sh.pvDone[g], (t >> 1) - 1);
          if (!ok) break;
        }
        TC_TRACE(6, t);
        float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f),
                          make_float2(0.f, 0.f)};
        const float2 scale2 = make_float2(kLog2e, kLog2e), shift2 = make_float2(-mref, -mref);
#pragma unroll
        for (int half = 0; half < 2; half++) {
          // (stored 32 keys at a time: sixteen packed registers live instead of thirty-two)
#pragma unroll
          for (int q = 0; q < 2; q++) {
            uint32_t pk[16];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              const int cc = half * 64 + q * 32 + c;
              const float2 tt = fma2(make_float2(__uint_as_float(sv[cc]), __uint_as_float(sv[cc + 1])),
                                     scale2, shift2);
              const float2 pe = exp2_pair(tt, (q * 32 + c) >> 1);
              sum2[(c >> 1) & 3] = add2(sum2[(c >> 1) & 3], pe);
              const __half2 hp = __floats2half2_rn(pe.x, pe.y);
              pk[c / 2] = *reinterpret_cast<const uint32_t*>(&hp);
            }
            tmem_st16(pCol + half * 32 + q * 16, pk);
          }
          TC_TRACE(7 + half, t);
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh.pReady[g][half]));
          TC_TRACE(4 + half, t);
        }
        const float2 s01 = add2(add2(sum2[0], sum2[1]), add2(sum2[2], sum2[3]));
        l += s01.x + s01.y;
      }
      if (!ok) break;

      // ---- the unit's row sums meet in the warpgroup that took its last tile ----
      // (one message per unit, also when the other warpgroup had no tile in it)
      if (g != ((tEnd - 1) & 1)) {
        // mailbox: free once the previous message has been read
        ok = wait_count(&sh.lRead[w], n, abortFlag);
        if (!ok) break;
        sh.lOther[rowInTile] = l;
        sh.seenOther[rowInTile] = seen;
        __syncwarp();
        if (lane == 0) st_release_shared(&sh.lWritten[w], n + 1);
      } else {
        // `seen` is the rows' final reference point: this warpgroup's max phase was the last
        ok = wait_count(&sh.lWritten[w], n + 1, abortFlag);
        if (!ok) break;
        l += sh.lOther[rowInTile] * fast_exp2(sh.seenOther[rowInTile] - seen);
        __syncwarp();
        if (lane == 0) st_release_shared(&sh.lRead[w], n + 1);
        // The read-out warps take it from here: 1/l per row (zero for a row that saw no key),
        // once they are through with the previous unit's.
        if (n >= 1) {
          ok = wait(&sh.oFree, n - 1);
          if (!ok) break;
        }
        sh.invL[rowInTile] = (l > 0.f && lo <= end) ? 1.f / l : 0.f;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.lReady));
      }
      tG = tEnd;
    }
  }

  // Common exit: every role arrives here, then the allocating warp frees tensor memory.
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && sh.abort) atomicOr(status, kStatusWaitTimeout);
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

template <int HD>
cudaError_t launch4(const AttnParams& p, int* status, int* work, int smCount, cudaStream_t s,
                    std::string* err) {
  using C = Cfg4<HD>;
  CUtensorMap mq, mk, mv;
  const int64_t qCols = (int64_t)p.qHeads * p.hd, kvCols = (int64_t)p.kvHeads * p.hd;
  if (!make_map(&mq, p.q, p.qLen, qCols, p.qStride, BM, err) ||
      !make_map(&mk, p.k, p.kvLen, kvCols, p.kvStride, BK4, err) ||
      !make_map(&mv, p.v, p.kvLen, kvCols, p.kvStride, C::V_ROWS, err))
    return cudaErrorInvalidValue;
  auto kern = prefill_tc4_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  if (e != cudaSuccess) return e;
  const int64_t total = (p.qLen + BM - 1) / BM * p.qHeads;
  const unsigned grid = (unsigned)(total < smCount ? total : smCount);
  kern<<<grid, kThreads4, C::SMEM, s>>>(mq, mk, mv, p, status, work);
  return cudaGetLastError();
}

}  // namespace

bool prefill_tc4_supported(const AttnParams& p, int dtype) {
  if (dtype != RT_F16) return false;
  if (p.hd != 64 && p.hd != 128 && p.hd != 256) return false;
  if (p.qLen < 2 || p.qLen >= (1ll << 31) - 256 || p.kvLen >= (1ll << 31) - 256) return false;
  if ((p.qLen + BM - 1) / BM * p.qHeads >= (1ll << 30)) return false;
  auto al = [](const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; };
  // TMA: 16-byte aligned bases and row pitches; the rows are written back in 16-byte stores
  if (!al(p.q, 16) || !al(p.k, 16) || !al(p.v, 16) || !al(p.out, 16)) return false;
  if ((p.qStride * 2) % 16 || (p.kvStride * 2) % 16) return false;
  if (!encode_fn()) return false;
  return true;
}

// `work`: two ints of device memory, zero before the first launch; the kernel leaves them zero.
cudaError_t launch_prefill_tc4(const AttnParams& p, int* status, int* work, int smCount,
                               cudaStream_t s, std::string* err) {
  switch (p.hd) {
    case 64: return launch4<64>(p, status, work, smCount, s, err);
    case 128: return launch4<128>(p, status, work, smCount, s, err);
    case 256: return launch4<256>(p, status, work, smCount, s, err);
  }
  return cudaErrorInvalidValue;
}

}  // namespace rt
