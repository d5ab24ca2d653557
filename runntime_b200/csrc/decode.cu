// Single-token decode attention over KV caches: bandwidth-bound split-KV.
//
// Grid = (key splits, sequences, head blocks).  A CTA streams its slice of one
// sequence's K and V cache rows through a shared-memory ring filled by bulk
// async copies (TMA, 16-byte aligned, whole rows so every DRAM sector fetched is
// used), issued by a producer warp and signalled through mbarriers.  The 256
// consumer threads are laid out as (key slot, query head): each thread runs a
// private online softmax over the keys of its slot in f32 registers.  At the
// end the slots of a head are merged with a log-sum-exp; with more than one
// split the per-split (m, l, acc) partials go to scratch and the last CTA to
// arrive for the sequence merges them — no second launch, no waiting.
//
// The KV-cache append is fused: the new K/V row is stored to the cache by the
// CTA of split 0 and attended to straight from its source.
//
// Replaces packages/runntime/src/core/kernels/attention/attnDecode.ts:81-187
// (decode), :263-424 (decodeSplit + merge) and the writeRows dispatches that
// precede them (packages/runntime/src/core/kernels/shape/rows.ts:143-162).
#include <mutex>

#include "common.cuh"
#include "sm100.cuh"

namespace rt {
namespace {

using namespace sm100;

// Optional per-CTA timeline for kernel development (off unless the translation unit is
// compiled with RT_DEC_TRACE): thread 0 of every CTA stores the global timer at a few points.
#ifdef RT_DEC_TRACE
constexpr int kDecTraceCtas = 8192, kDecTracePoints = 8;
__device__ unsigned long long gDecTrace[kDecTraceCtas * kDecTracePoints];
#define DEC_TRACE(i)                                                                        \
  do {                                                                                      \
    if (threadIdx.x == 0) {                                                                 \
      const unsigned id_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;  \
      if (id_ < kDecTraceCtas) {                                                            \
        unsigned long long t_;                                                              \
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                              \
        gDecTrace[id_ * kDecTracePoints + (i)] = t_;                                        \
      }                                                                                     \
    }                                                                                       \
  } while (0)
#else
#define DEC_TRACE(i) \
  do {               \
  } while (0)
#endif

constexpr int kConsumers = 256;
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kMaxStages = 8;
// Heads up to 64 wide fit two CTAs per SM (registers and shared memory), so that one
// CTA's set-up, pipeline fill and merge overlap the other's streaming; wider heads get
// the whole SM.
constexpr size_t kSmemBudget = 200 * 1024;
constexpr size_t kSmemBudgetTwoPerSm = 108 * 1024;

__host__ __device__ constexpr int q_stride(int hdp) { return ((hdp / 4) & 1) ? hdp : hdp + 4; }

template <typename T, int VEC>
struct Loader;

// 8 halves per 16-byte load
template <>
struct Loader<__half, 8> {
  static __device__ __forceinline__ void load(const __half* p, float (&f)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <>
struct Loader<__half, 4> {
  static __device__ __forceinline__ void load(const __half* p, float (&f)[4]) {
    const uint2 w = *reinterpret_cast<const uint2*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <>
struct Loader<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
    const float4 w = *reinterpret_cast<const float4*>(p);
    f[0] = w.x; f[1] = w.y; f[2] = w.z; f[3] = w.w;
  }
};
template <typename T>
struct Loader<T, 1> {
  static __device__ __forceinline__ void load(const T* p, float (&f)[1]) { f[0] = to_f32<T>(*p); }
};

// Rows whose pitch is a multiple of 128 bytes (head size 64 or 128) put the same column of
// every key into the same bank: threads that walk their rows in step would collide on every
// load (eight ways for 16-byte loads; measured 1.0 TB/s at head size 128).  Such a thread
// starts at chunk `rot` of its row and wraps around instead: a dot product does not care
// about the order, q is fetched from the same rotated position, and the accumulator keeps
// its chunks in rotated order until it is written out (acc chunk i = row chunk
// (i + rot) mod chunks).
template <int HDP, bool EXACT, int VEC>
struct Rotated {
  static constexpr bool value = EXACT && VEC > 1 && (HDP == 64 || HDP == 128);
};

// One key for one head: score, online-softmax update, accumulate p*v.
// kp/vp may point at shared memory (cache tile) or global memory (appended row).
template <typename T, int HDP, bool EXACT, int VEC, bool QSMEM>
__device__ __forceinline__ void process_key(const T* kp, const T* vp, const float* qv, int hd,
                                            float& m, float& l, float (&acc)[HDP], int rot) {
  constexpr bool ROT = Rotated<HDP, EXACT, VEC>::value;
  constexpr int NCH = HDP / VEC;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int i = 0; i < HDP / VEC; i++) {
    if (EXACT || i * VEC < hd) {
      const int ci = ROT ? ((i + rot) & (NCH - 1)) : i;
      float f[VEC];
      Loader<T, VEC>::load(kp + ci * VEC, f);
      if (ROT) {
        // q chunk from the same position: 16-byte loads (the q rows are 16-byte aligned)
        float qf[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e += 4) {
          const float4 t = *reinterpret_cast<const float4*>(qv + ci * VEC + e);
          qf[e] = t.x, qf[e + 1] = t.y, qf[e + 2] = t.z, qf[e + 3] = t.w;
        }
#pragma unroll
        for (int e = 0; e < VEC; e += 4) {
          s0 = fmaf(qf[e], f[e], s0);
          s1 = fmaf(qf[e + 1], f[e + 1], s1);
          s2 = fmaf(qf[e + 2], f[e + 2], s2);
          s3 = fmaf(qf[e + 3], f[e + 3], s3);
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; e++) {
          if ((i * VEC + e) & 1) s1 = fmaf(qv[i * VEC + e], f[e], s1);
          else s0 = fmaf(qv[i * VEC + e], f[e], s0);
        }
      }
    }
  }
  const float s = ((s0 + s1) + (s2 + s3)) * kLog2e;  // log2 domain
  if (s > m) {
    const float c = fast_exp2(m - s);
    l *= c;
#pragma unroll
    for (int x = 0; x < HDP; x++) acc[x] *= c;
    m = s;
  }
  const float pe = fast_exp2(s - m);
  l += pe;
#pragma unroll
  for (int i = 0; i < HDP / VEC; i++) {
    if (EXACT || i * VEC < hd) {
      const int ci = ROT ? ((i + rot) & (NCH - 1)) : i;
      float f[VEC];
      Loader<T, VEC>::load(vp + ci * VEC, f);
#pragma unroll
      for (int e = 0; e < VEC; e++) acc[i * VEC + e] = fmaf(pe, f[e], acc[i * VEC + e]);
    }
  }
}

// The same for a thread that owns W = hd / R columns of the (key, head) pair, R = 2 or 4
// adjacent lanes sharing the pair (head size 64 and 128: a whole 128-wide row per thread
// costs 512 bytes of every stage and 128 accumulator registers, so few keys fit a tile
// and the threads' long dependent chains leave the SM idle — measured 2.5 TB/s).  The
// partial scores are added across the R lanes by shuffles restricted to the group; m
// and l then evolve identically in all of them.  q lives in registers, loaded once in
// the same rotated chunk order as the row is walked (see Rotated).
template <typename T, int W, int VEC, int R>
__device__ __forceinline__ void process_key_sub(const T* kp, const T* vp, const float (&q)[W],
                                                float& m, float& l, float (&acc)[W], int rot,
                                                unsigned groupMask) {
  constexpr int NCH = W / VEC;
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int i = 0; i < NCH; i++) {
    const int ci = (i + rot) & (NCH - 1);
    float f[VEC];
    Loader<T, VEC>::load(kp + ci * VEC, f);
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
      s0 = fmaf(q[i * VEC + e], f[e], s0);
      s1 = fmaf(q[i * VEC + e + 1], f[e + 1], s1);
    }
  }
  float s = s0 + s1;
#pragma unroll
  for (int o = 1; o < R; o <<= 1) s += __shfl_xor_sync(groupMask, s, o);
  s *= kLog2e;  // log2 domain
  if (s > m) {
    const float c = fast_exp2(m - s);
    l *= c;
#pragma unroll
    for (int x = 0; x < W; x++) acc[x] *= c;
    m = s;
  }
  const float pe = fast_exp2(s - m);
  l += pe;
#pragma unroll
  for (int i = 0; i < NCH; i++) {
    const int ci = (i + rot) & (NCH - 1);
    float f[VEC];
    Loader<T, VEC>::load(vp + ci * VEC, f);
#pragma unroll
    for (int e = 0; e < VEC; e++) acc[i * VEC + e] = fmaf(pe, f[e], acc[i * VEC + e]);
  }
}

// Two keys at once for the same thread: the two dot products, their shuffles and the two
// accumulations are independent instruction streams, which a thread with one key at a time
// does not have (nine warps per SM hide little latency).
template <typename T, int W, int VEC, int R>
__device__ __forceinline__ void process_key_pair(const T* ka, const T* va, const T* kb, const T* vb,
                                                 const float (&q)[W], float& m, float& l,
                                                 float (&acc)[W], int rot, unsigned groupMask) {
  constexpr int NCH = W / VEC;
  float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
  for (int i = 0; i < NCH; i++) {
    const int ci = (i + rot) & (NCH - 1);
    float fa[VEC], fb[VEC];
    Loader<T, VEC>::load(ka + ci * VEC, fa);
    Loader<T, VEC>::load(kb + ci * VEC, fb);
#pragma unroll
    for (int e = 0; e < VEC; e += 2) {
      a0 = fmaf(q[i * VEC + e], fa[e], a0);
      a1 = fmaf(q[i * VEC + e + 1], fa[e + 1], a1);
      b0 = fmaf(q[i * VEC + e], fb[e], b0);
      b1 = fmaf(q[i * VEC + e + 1], fb[e + 1], b1);
    }
  }
  float sa = a0 + a1, sb = b0 + b1;
#pragma unroll
  for (int o = 1; o < R; o <<= 1) {
    sa += __shfl_xor_sync(groupMask, sa, o);
    sb += __shfl_xor_sync(groupMask, sb, o);
  }
  sa *= kLog2e, sb *= kLog2e;  // log2 domain
  const float mn = fmaxf(sa, sb);
  if (mn > m) {
    const float c = fast_exp2(m - mn);
    l *= c;
#pragma unroll
    for (int x = 0; x < W; x++) acc[x] *= c;
    m = mn;
  }
  const float pa = fast_exp2(sa - m), pb = fast_exp2(sb - m);
  l += pa + pb;
#pragma unroll
  for (int i = 0; i < NCH; i++) {
    const int ci = (i + rot) & (NCH - 1);
    float fa[VEC], fb[VEC];
    Loader<T, VEC>::load(va + ci * VEC, fa);
    Loader<T, VEC>::load(vb + ci * VEC, fb);
#pragma unroll
    for (int e = 0; e < VEC; e++) acc[i * VEC + e] = fmaf(pa, fa[e], fmaf(pb, fb[e], acc[i * VEC + e]));
  }
}

// Cross-GPU hand-over, called by the consumer threads of the block that wrote the final
// rows of (sequence b, head block) into this rank's staging buffer.  The rows go to the one
// rank that merges sequence b (its owner): plain, coalesced stores into that rank's
// exchange buffer — peer memory unless the owner is this rank.  The block then counts
// itself in for that owner; the last block to do so fences at system scope and publishes
// this rank's step in the owner's arrival word (one release store), so an owner is told as
// soon as its rows are complete, while the other owners' sequences are still being
// attended.  The last owner group to finish moves this rank's step counter for the merge
// kernel and the next launch.
__device__ __forceinline__ void exchange_rows(const DecodeParams& p, int b, int hq, int h0, int tid,
                                              uint32_t epoch, int headBlocks) {
  const int stride = 2 + p.hd;
  const int owner = owner_of(b, p.batch, p.xWorld), bl = b - owner_first(owner, p.batch, p.xWorld);
  const float* src = p.xStage + ((int64_t)b * p.qHeads + h0) * stride;  // this block's rows: contiguous
  float* dst = p.xPartials[owner] +
               ((((int64_t)(epoch & 1u) * p.xWorld + p.xRank) * p.xPer + bl) * p.qHeads + h0) * stride;
  const int n = hq * stride;
  named_barrier_sync(1, kConsumers);   // the rows this block's threads wrote are visible to all of them
  for (int i = tid; i < n; i += kConsumers) dst[i] = __ldcg(src + i);
  __threadfence();                     // each thread's stores, before the block is counted in
  named_barrier_sync(1, kConsumers);
  if (tid != 0) return;
  unsigned* counts = p.xStep + 2;      // [world] blocks arrived per owner, then owners done
  const int owned = owner_count(owner, p.batch, p.xWorld);
  if (atomicAdd(counts + owner, 1u) != (unsigned)(owned * headBlocks) - 1u) return;
  counts[owner] = 0;                   // ready for the next launch
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.xFlags[owner] + p.xRank), "r"(epoch)
               : "memory");
  if (atomicAdd(counts + p.xWorld, 1u) != (unsigned)p.xWorld - 1u) return;   // every rank owns some
  counts[p.xWorld] = 0;
  __threadfence();
  *reinterpret_cast<volatile uint32_t*>(p.xStep) = epoch;
}

template <typename T, int HDP, bool EXACT, int VEC, bool BULK, int R = 1>
__global__ void __launch_bounds__(BULK ? kConsumers + 32 : kConsumers, HDP / R <= 64 ? 2 : 1)
decode_kernel(const DecodeParams p) {
  constexpr bool QSMEM = true;
  constexpr int W = HDP / R;   // columns of a head per thread (R lanes share a (key, head) pair)
  static_assert(R == 1 || (EXACT && BULK && VEC > 1 && (W % VEC) == 0), "sub-row threads: exact bulk path only");
  constexpr int QS = q_stride(HDP);
  extern __shared__ __align__(128) unsigned char smemRaw[];
  __shared__ int sAbort;
  __shared__ int sAbortSeen;
  __shared__ int sIsLast;
  __shared__ __align__(8) uint64_t sFull[kMaxStages], sEmpty[kMaxStages];

  const int tid = threadIdx.x;
  DEC_TRACE(0);
  // Launched as a programmatic dependent of the kernel before it in the stream (see
  // launch_one): the blocks may become resident while that kernel's last blocks finish, and
  // wait here until all of its writes are visible.  Nothing above reads memory.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int split = blockIdx.x, zb = blockIdx.z;
  const int by = blockIdx.y;   // unique per (attention, sequence): indexes scratch and counters
  int b = by;
  if (p.xWorld > 1) {   // the sequences this rank merges itself come last
    b += p.xRot;
    if (b >= p.batch) b -= p.batch;
  }
  // The second attention of the launch (cross-attention) takes blocks [batch, 2*batch).
  const bool sec = p.hasSecond && by >= p.batch;
  if (sec) b = by - p.batch;
  const void* aQ = sec ? p.s2.q : p.q;
  void* aOut = sec ? p.s2.out : p.out;
  const int32_t* aLens = sec ? p.s2.kvLens : p.kvLens;
  const int64_t aSeqStride = sec ? p.s2.cacheSeqStride : p.cacheSeqStride;
  const int64_t aQStride = sec ? p.s2.qRowStride : p.qRowStride;
  const int aCacheRows = sec ? p.s2.cacheRows : p.cacheRows;
  const int aKvLen = sec ? p.s2.kvLen : p.kvLen;
  const int aWl = sec ? p.s2.wl : p.wl;
  const int hd = p.hd;
  const int group = p.qHeads / p.kvHeads;
  const int kvh0 = zb * p.kvPerCta;
  const int nkv = min(p.kvPerCta, p.kvHeads - kvh0);
  const int hqReal = nkv * group;           // query heads of this CTA
  const int hqMax = p.kvPerCta * group * R;  // thread columns: (head, lane of the head's group)
  const int hq = hqReal * R;
  const int KS = p.keySlots;
  const int sliceElems = nkv * hd;
  const int rowElems = p.kvHeads * hd;
  // Where the final (m, l, acc) rows go, if not into `out`: the caller's buffer, or —
  // with the cross-GPU exchange — this rank's staging buffer, from where exchange_rows
  // sends them to the rank that merges the sequence.  The step now starting is one past
  // the rank's step counter, which only the last block of this launch moves, so all
  // blocks read the same value.
  float* partialsOut = p.partialsOut;
  uint32_t epoch = 0;
  if (p.xWorld > 0) {
    epoch = *reinterpret_cast<volatile uint32_t*>(p.xStep) + 1u;
    partialsOut = p.xStage;
  }

  // Key range of this sequence that lives in the cache.
  // L: visible rows of this cache; Lg: the sequence's length (the two differ only when the
  // cache is one rank's shard of the sequence).
  int64_t lo, end, L = 0, Lg = 0;
  bool hasNew = p.kNew != nullptr && !sec;
  // This sequence's caches: its slice of the slab, or its own allocation.
  const void* const* kPtrs = sec ? p.s2.kPtrs : p.kPtrs;
  const void* const* vPtrs = sec ? p.s2.vPtrs : p.vPtrs;
  const T* kSeq = kPtrs ? static_cast<const T*>(kPtrs[b])
                        : static_cast<const T*>(sec ? p.s2.kCache : p.kCache) + (int64_t)b * aSeqStride;
  const T* vSeq = vPtrs ? static_cast<const T*>(vPtrs[b])
                        : static_cast<const T*>(sec ? p.s2.vCache : p.vCache) + (int64_t)b * aSeqStride;
  // What a consumer thread stages — q and, in split 0, the appended K/V row — is loaded into
  // registers before the sequence's length is looked at: the length decides where the rows
  // go, not where they come from, and under a saturated memory system every load that has
  // to wait for another costs microseconds of set-up.
  constexpr int kPre = 4;   // elements per thread held in registers; longer rows finish in a loop
  const T* qg = static_cast<const T*>(aQ) + (int64_t)b * aQStride;
  const bool roped = p.ropeCos != nullptr && !p.useRange && !sec;
  const bool pre = R == 1 && !roped && tid < kConsumers;
  const bool preNew = pre && hasNew && split == 0 && !p.useRange;
  const T* kn = hasNew ? static_cast<const T*>(p.kNew) + (int64_t)b * p.kNewRowStride + kvh0 * hd : nullptr;
  const T* vn = hasNew ? static_cast<const T*>(p.vNew) + (int64_t)b * p.vNewRowStride + kvh0 * hd : nullptr;
  T qPre[kPre], knPre[kPre], vnPre[kPre];
#pragma unroll
  for (int i = 0; i < kPre; i++) {
    const int idx = tid + i * kConsumers;
    qPre[i] = knPre[i] = vnPre[i] = from_f32<T>(0.f);
    if (pre && idx < hqReal * hd) qPre[i] = qg[kvh0 * group * hd + idx];   // the CTA's heads are contiguous
    if (preNew && idx < sliceElems) {
      knPre[i] = kn[idx];
      vnPre[i] = vn[idx];
    }
  }
  // (a separately allocated cache is only known here: the bulk copies need 16-byte alignment)
  const bool misaligned = kPtrs && BULK &&
                          ((reinterpret_cast<uintptr_t>(kSeq) | reinterpret_cast<uintptr_t>(vSeq)) & 15u);
  if (p.useRange) {
    lo = p.lo;
    end = p.end;
  } else {
    Lg = L = aLens ? aLens[b] : aKvLen;
    if (p.kvSharded) {
      // This cache holds rows [shardStart, shardStart + cacheRows) of the sequence: it sees
      // what falls inside, and takes the appended row (global row Lg-1) only if that is one
      // of its own.
      const int64_t local = Lg - p.shardStart;
      hasNew = hasNew && local >= 1 && local <= p.cacheRows;
      L = local < 0 ? 0 : local > p.cacheRows ? p.cacheRows : local;
    } else if (L > aCacheRows || misaligned) {
      // A length past the cache's capacity (the host checks only the scalar kvLen; this one
      // lives on the device): writeRows would refuse it ('rows exceed dst capacity').  The
      // sequence is treated as empty — nothing appended, nothing read, zeros out — and the
      // status word reports it.  The same for a cache pointer the bulk copies cannot take.
      if (tid == 0) atomicOr(p.status, kStatusBadState);
      Lg = L = 0;
      hasNew = false;
    }
    end = L - 1;
    lo = Lg - 1 - aWl - p.shardStart;
    if (lo < 0) lo = 0;
    if (hasNew) end -= 1;  // row L-1 is the appended one, taken from kNew/vNew
    if (L <= 0) { lo = 1; end = -1; }
  }
  const int64_t n = end >= lo ? end - lo + 1 : 0;
  int64_t chunk = (n + p.splits - 1) / p.splits;
  chunk = (chunk + KS - 1) / KS * KS;
  int64_t s0 = lo + (int64_t)split * chunk, s1 = s0 + chunk;
  if (s1 > end + 1) s1 = end + 1;
  const int ntiles = s1 > s0 ? (int)((s1 - s0 + KS - 1) / KS) : 0;

  const T* kBase = kSeq + kvh0 * hd;
  const T* vBase = vSeq + kvh0 * hd;

  // Shared-memory carve-up: [q][appended K, V slices][ring: stages x (K tile, V tile)];
  // the ring is reused for the slot merge at the end.
  float* sQ = reinterpret_cast<float*>(smemRaw);
  // (threads that own a slice of a head keep q in registers and read the appended row back
  // from the cache: no staging areas)
  const int qBytes = R == 1 ? ((hqMax * QS * 4 + 127) / 128) * 128 : 0;
  const int newBytes = (R == 1 && p.kNew != nullptr) ? ((p.kvPerCta * hd * (int)sizeof(T) + 127) / 128) * 128 : 0;
  T* sKn = reinterpret_cast<T*>(smemRaw + qBytes);           // appended K slice
  T* sVn = reinterpret_cast<T*>(smemRaw + qBytes + newBytes);  // appended V slice
  unsigned char* ring = smemRaw + qBytes + 2 * newBytes;
  const int tileBytes = ((KS * p.kvPerCta * hd * (int)sizeof(T) + 127) / 128) * 128;
  const int stages = BULK ? p.stages : 1;

  if (tid == 0) {
    sAbort = 0;
    sIsLast = 0;
    if (BULK) {
      for (int s = 0; s < stages; s++) {
        mbar_init(smem_u32(&sFull[s]), 1);
        mbar_init(smem_u32(&sEmpty[s]), kConsumerWarps);
      }
      fence_barrier_init();
    }
  }
  __syncthreads();

  if (BULK && tid >= kConsumers) {
    // ---------------- producer warp ----------------
    const int lane = tid - kConsumers;
    const bool flat = (nkv == p.kvHeads);
    for (int it = 0; it < ntiles; it++) {
      const int s = it % stages;
      if (it >= stages) {
        if (!mbar_wait(smem_u32(&sEmpty[s]), ((it / stages) - 1) & 1, &sAbort)) break;
      }
      const int64_t k0 = s0 + (int64_t)it * KS;
      const int nk = (int)min((int64_t)KS, s1 - k0);
      const uint32_t bar = smem_u32(&sFull[s]);
      const uint32_t dK = smem_u32(ring + (size_t)s * 2 * tileBytes);
      const uint32_t dV = dK + tileBytes;
      const uint32_t rowBytes = (uint32_t)sliceElems * sizeof(T);
      if (lane == 0) mbar_expect_tx(bar, 2u * nk * rowBytes);
      __syncwarp();
      if (flat) {
        if (lane == 0) {
          bulk_g2s(dK, kBase + k0 * rowElems, nk * rowBytes, bar);
          bulk_g2s(dV, vBase + k0 * rowElems, nk * rowBytes, bar);
        }
      } else {
        for (int r = lane; r < nk; r += 32) {
          bulk_g2s(dK + r * rowBytes, kBase + (k0 + r) * rowElems, rowBytes, bar);
          bulk_g2s(dV + r * rowBytes, vBase + (k0 + r) * rowElems, rowBytes, bar);
        }
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  const int hv = tid % hqMax;        // thread column
  const int hl = hv / R;             // query head within the CTA
  const int sub = hv % R;            // which W columns of the head
  const int slot = tid / hqMax;
  const bool active = slot < KS && hv < hq;
  const int h = kvh0 * group + hl;   // query head
  const int kvl = hl / group;        // kv head within the CTA's slice
  const unsigned groupMask = R == 1 ? 0u : (((1u << R) - 1u) << ((tid & 31) & ~(R - 1)));

  // Stage q (f32) and, in split 0, the appended K/V slices; with rope tables q and
  // the new K row are rotated here and rounded to T as the separate rope dispatch
  // stores them.  The new row goes to the cache from the same threads (what
  // writeRows would do) and is attended from shared memory after the cache keys.
  const bool appendHere = hasNew && split == 0 && !p.useRange && L >= 1;
  const float* qv = sQ + hl * QS;
  const int64_t ropeRow = p.ropeByPos ? (Lg >= 1 ? Lg - 1 : 0) : b;
  const float* rc = roped ? p.ropeCos + ropeRow * hd : nullptr;
  const float* rs = roped ? p.ropeSin + ropeRow * hd : nullptr;
  {
    if (R > 1) {
      // q goes straight to registers below
    } else if (roped) {
      const int hp = hd >> 1;
      for (int idx = tid; idx < hqReal * hp; idx += kConsumers) {
        const int hh = idx / hp, x = (idx - hh * hp) * 2;
        const T* src = qg + (kvh0 * group + hh) * hd + x;
        float r0, r1;
        rope_pair(to_f32<T>(src[0]), to_f32<T>(src[1]), rc[x], rs[x], r0, r1);
        sQ[hh * QS + x] = to_f32<T>(from_f32<T>(r0));
        sQ[hh * QS + x + 1] = to_f32<T>(from_f32<T>(r1));
      }
    } else {
#pragma unroll
      for (int i = 0; i < kPre; i++) {
        const int idx = tid + i * kConsumers;
        if (idx < hqReal * hd) {
          const int hh = idx / hd, x = idx - hh * hd;
          sQ[hh * QS + x] = to_f32<T>(qPre[i]);
        }
      }
      for (int idx = tid + kPre * kConsumers; idx < hqReal * hd; idx += kConsumers) {
        const int hh = idx / hd, x = idx - hh * hd;
        sQ[hh * QS + x] = to_f32<T>(qg[(kvh0 * group + hh) * hd + x]);
      }
    }
    if (appendHere) {
      T* kc = const_cast<T*>(kBase) + (L - 1) * rowElems;
      T* vc = const_cast<T*>(vBase) + (L - 1) * rowElems;
      if (roped) {
        const int hp = hd >> 1;
        for (int idx = tid; idx < nkv * hp; idx += kConsumers) {
          const int hh = idx / hp, x = (idx - hh * hp) * 2;
          float r0, r1;
          rope_pair(to_f32<T>(kn[hh * hd + x]), to_f32<T>(kn[hh * hd + x + 1]), rc[x], rs[x], r0, r1);
          const T t0 = from_f32<T>(r0), t1 = from_f32<T>(r1);
          if (R == 1) sKn[hh * hd + x] = t0, sKn[hh * hd + x + 1] = t1;
          kc[hh * hd + x] = t0, kc[hh * hd + x + 1] = t1;
        }
      }
      if (preNew) {
#pragma unroll
        for (int i = 0; i < kPre; i++) {
          const int x = tid + i * kConsumers;
          if (x < sliceElems) {
            sKn[x] = knPre[i], kc[x] = knPre[i];
            sVn[x] = vnPre[i], vc[x] = vnPre[i];
          }
        }
      }
      for (int x = tid + (preNew ? kPre * kConsumers : 0); x < sliceElems; x += kConsumers) {
        if (!roped) {
          const T t = kn[x];
          if (R == 1) sKn[x] = t;
          kc[x] = t;
        }
        const T u = vn[x];
        if (R == 1) sVn[x] = u;
        vc[x] = u;
      }
    }
    named_barrier_sync(1, kConsumers);
  }
  DEC_TRACE(1);

  float m = kNegSeed, l = 0.f;
  float acc[W];
  constexpr bool ROT = R > 1 || Rotated<HDP, EXACT, VEC>::value;
  // Threads whose rows start in the same bank take different rotations (see Rotated):
  // with 64-byte slices every second thread does.
  constexpr int kSameBank = (W * (int)sizeof(T) >= 128) ? 1 : 128 / (W * (int)sizeof(T));
  const int rot = ROT ? ((tid / kSameBank) & (W / VEC - 1)) : 0;
#pragma unroll
  for (int x = 0; x < W; x++) acc[x] = 0.f;
  float qr[R > 1 ? W : 1];
  if (R > 1) {
    // This thread's W columns of q, rotated like the rows it will walk, with the rope applied
    // and rounded to T as the separate rope dispatch would store them.
#pragma unroll
    for (int x = 0; x < (R > 1 ? W : 1); x++) qr[x] = 0.f;
    if (hv < hq) {
      const T* src = qg + (int64_t)h * hd + sub * W;
#pragma unroll
      for (int i = 0; i < W / VEC; i++) {
        const int ci = (i + rot) & (W / VEC - 1);
        float f[VEC];
        Loader<T, VEC>::load(src + ci * VEC, f);
#pragma unroll
        for (int e = 0; e < VEC; e += 2) {
          float r0 = f[e], r1 = f[e + 1];
          if (roped) {
            const int x = sub * W + ci * VEC + e;
            rope_pair(f[e], f[e + 1], rc[x], rs[x], r0, r1);
            r0 = to_f32<T>(from_f32<T>(r0));
            r1 = to_f32<T>(from_f32<T>(r1));
          }
          qr[(i * VEC + e) % (R > 1 ? W : 1)] = r0;
          qr[(i * VEC + e + 1) % (R > 1 ? W : 1)] = r1;
        }
      }
    }
  }
  if (active && slot == 0 && split == 0 && p.sinks) {
    m = p.sinks[h];  // sinks are log2-space: sink * ln2 * log2e
    l = 1.f;
  }

  bool ok = true;
  int it = 0;
  if constexpr (R > 1) {
    // Tiles two at a time while the ring is deep enough to keep copies in flight behind them.
    if (stages >= 4) {
      for (; it + 1 < ntiles; it += 2) {
        const int sa = it % stages, sb = (it + 1) % stages;
        if (!mbar_wait(smem_u32(&sFull[sa]), (it / stages) & 1, &sAbort) ||
            !mbar_wait(smem_u32(&sFull[sb]), ((it + 1) / stages) & 1, &sAbort)) {
          ok = false;
          break;
        }
        const T* aK = reinterpret_cast<const T*>(ring + (size_t)sa * 2 * tileBytes);
        const T* bK = reinterpret_cast<const T*>(ring + (size_t)sb * 2 * tileBytes);
        const int nkb = (int)min((int64_t)KS, s1 - (s0 + (int64_t)(it + 1) * KS));  // tile `it` is full
        if (active) {
          const int off = slot * sliceElems + kvl * hd + sub * W;
          const int vOff = tileBytes / (int)sizeof(T);
          if (slot < nkb)
            process_key_pair<T, W, VEC, R>(aK + off, aK + vOff + off, bK + off, bK + vOff + off, qr, m,
                                           l, acc, rot, groupMask);
          else
            process_key_sub<T, W, VEC, R>(aK + off, aK + vOff + off, qr, m, l, acc, rot, groupMask);
        }
        __syncwarp();
        if ((tid & 31) == 0) {
          mbar_arrive(smem_u32(&sEmpty[sa]));
          mbar_arrive(smem_u32(&sEmpty[sb]));
        }
      }
    }
  }
  for (; it < ntiles && ok; it++) {
    const int64_t k0 = s0 + (int64_t)it * KS;
    const int nk = (int)min((int64_t)KS, s1 - k0);
    const int s = BULK ? it % stages : 0;
    T* tK = reinterpret_cast<T*>(ring + (size_t)s * 2 * tileBytes);
    T* tV = reinterpret_cast<T*>(ring + (size_t)s * 2 * tileBytes + tileBytes);
    if (BULK) {
      if (!mbar_wait(smem_u32(&sFull[s]), (it / stages) & 1, &sAbort)) { ok = false; break; }
      if (it == 0) DEC_TRACE(2);
    } else {
      named_barrier_sync(1, kConsumers);
      for (int idx = tid; idx < nk * sliceElems; idx += kConsumers) {
        const int jj = idx / sliceElems, x = idx - jj * sliceElems;
        tK[idx] = kBase[(k0 + jj) * rowElems + x];
        tV[idx] = vBase[(k0 + jj) * rowElems + x];
      }
      named_barrier_sync(1, kConsumers);
    }
    if (active && slot < nk) {
      const int off = slot * sliceElems + kvl * hd + sub * W;
      if constexpr (R > 1) process_key_sub<T, W, VEC, R>(tK + off, tV + off, qr, m, l, acc, rot, groupMask);
      else process_key<T, HDP, EXACT, VEC, QSMEM>(tK + off, tV + off, qv, hd, m, l, acc, rot);
    }
    if (BULK) {
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(smem_u32(&sEmpty[s]));
    }
  }

  DEC_TRACE(3);
  // This block has streamed its keys: once every block has, the next kernel's blocks may
  // take the freed slots (they wait for this grid to finish before they read anything).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // Fused append: split 0 attends to the new row it staged (and stored) above.
  if (appendHere && active && slot == 0) {
    const int off = kvl * hd + sub * W;
    // (sub-row threads read the row this block stored to the cache before the barrier above)
    if constexpr (R > 1)
      process_key_sub<T, W, VEC, R>(kBase + (L - 1) * rowElems + off, vBase + (L - 1) * rowElems + off, qr,
                                    m, l, acc, rot, groupMask);
    else process_key<T, HDP, EXACT, VEC, QSMEM>(sKn + off, sVn + off, qv, hd, m, l, acc, rot);
  }

  // Every consumer is through its tiles (or has given up): the ring is free.  Whether a wait
  // ran out is decided once for the whole block — a thread that finished its tiles before
  // another one's wait ran out must not go on to barriers the other will never reach.
  named_barrier_sync(1, kConsumers);
  if (tid == 0) sAbortSeen = sAbort;
  named_barrier_sync(1, kConsumers);
  if (sAbortSeen) {
    // A wait ran out: record it, let copies in flight land, leave.
    if (tid == 0) atomicOr(p.status, kStatusWaitTimeout);
    for (int i = 0; i < 64; i++) __nanosleep(4000);
    return;
  }

  // ---- merge the key slots of each head (log-sum-exp) ----
  float* sM = reinterpret_cast<float*>(ring);  // [KS][hqMax][2 + W]
  constexpr int MS = 2 + W;
  if (active) {
    float* r = sM + (slot * hqMax + hv) * MS;
    r[0] = m;
    r[1] = l;
    if (ROT) {
#pragma unroll
      for (int i = 0; i < W / VEC; i++) {
        float* dst = r + 2 + ((i + rot) & (W / VEC - 1)) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; e++) dst[e] = acc[i * VEC + e];
      }
    } else {
#pragma unroll
      for (int x = 0; x < W; x++) r[2 + x] = acc[x];
    }
  }
  named_barrier_sync(1, kConsumers);

  const int stride = 2 + hd;  // partials row in global memory
  const int wd = R == 1 ? hd : W;   // columns this thread column owns ...
  const int col0 = sub * W;         // ... starting here in the head
  if (active) {
    // Every thread of a head's column walks the head's KS slot rows: first for the maximum,
    // then for the sum, then once per output column it owns (columns slot, slot+KS, ...).
    // The slot weights are recomputed per column — a register array indexed by the column
    // counter would live in local memory, whose round trips queue behind the cache streams.
    float M = kNegSeed;
    for (int s = 0; s < KS; s++) M = fmaxf(M, sM[(s * hqMax + hv) * MS]);
    float L = 0.f;
    for (int s = 0; s < KS; s++) {
      const float* r = sM + (s * hqMax + hv) * MS;
      L = fmaf(r[1], fast_exp2(r[0] - M), L);
    }
    const bool toPartials = partialsOut != nullptr;
    const bool whole = p.splits == 1;
    const float invL = L > 0.f ? 1.f / L : 0.f;
    float* rowF = !whole ? p.scratch + (((int64_t)by * p.splits + split) * p.qHeads + h) * stride
                         : toPartials ? partialsOut + ((int64_t)b * p.qHeads + h) * stride : nullptr;
    T* rowT = static_cast<T*>(aOut) + ((int64_t)b * p.qHeads + h) * hd + col0;
    if (rowF && slot == 0 && sub == 0) {
      // finished rows carry the maximum in natural-log units, split rows in log2 units
      rowF[0] = !whole ? M : L > 0.f ? M * 0.6931471805599453f : kNegSeed;
      rowF[1] = L;
    }
    for (int x = slot; x < wd; x += KS) {
      float o = 0.f;
#pragma unroll 4
      for (int s = 0; s < KS; s++) {
        const float* r = sM + (s * hqMax + hv) * MS;
        o = fmaf(r[2 + x], fast_exp2(r[0] - M), o);
      }
      if (rowF) rowF[2 + col0 + x] = o;
      else rowT[x] = from_f32<T>(o * invL);
    }
  }
  DEC_TRACE(4);
  if (p.splits == 1) {
    if (p.xWorld > 0) exchange_rows(p, b, hqReal, kvh0 * group, tid, epoch, gridDim.z);
    DEC_TRACE(5);
    return;
  }

  // ---- last CTA of the sequence merges the splits ----
  __threadfence();
  named_barrier_sync(1, kConsumers);
  if (tid == 0) {
    const unsigned old = atomicAdd(&p.counters[by * gridDim.z + zb], 1u);
    sIsLast = (old == (unsigned)p.splits - 1);
  }
  named_barrier_sync(1, kConsumers);
  if (!sIsLast) return;
  __threadfence();
  if (active) {
    const float* base = p.scratch + ((int64_t)by * p.splits * p.qHeads + h) * stride;
    const int64_t ss = (int64_t)p.qHeads * stride;  // between splits
    float M = kNegSeed;
    for (int s = 0; s < p.splits; s++) M = fmaxf(M, __ldcg(base + s * ss));
    float L = 0.f;
    for (int s = 0; s < p.splits; s++)
      L = fmaf(__ldcg(base + s * ss + 1), fast_exp2(__ldcg(base + s * ss) - M), L);
    const bool toPartials = partialsOut != nullptr;
    const float invL = L > 0.f ? 1.f / L : 0.f;
    for (int xx = slot; xx < wd; xx += KS) {
      const int x = col0 + xx;
      float o = 0.f;
      for (int s = 0; s < p.splits; s++)
        o = fmaf(__ldcg(base + s * ss + 2 + x), fast_exp2(__ldcg(base + s * ss) - M), o);
      if (toPartials)
        partialsOut[((int64_t)b * p.qHeads + h) * stride + 2 + x] = o;
      else
        static_cast<T*>(aOut)[((int64_t)b * p.qHeads + h) * hd + x] = from_f32<T>(o * invL);
    }
    if (toPartials && slot == 0 && sub == 0) {
      float* dst = partialsOut + ((int64_t)b * p.qHeads + h) * stride;
      dst[0] = L > 0.f ? M * 0.6931471805599453f : kNegSeed;
      dst[1] = L;
    }
  }
  if (tid == 0) p.counters[by * gridDim.z + zb] = 0;  // ready for the next launch
  if (p.xWorld > 0) exchange_rows(p, b, hqReal, kvh0 * group, tid, epoch, gridDim.z);
}

size_t smem_bytes(const DecodeParams& p, int esize, int hdp, bool bulk) {
  const int group = p.qHeads / p.kvHeads;
  const int hqMax = p.kvPerCta * group;
  const bool staged = p.lanesPerRow <= 1;   // see the kernel's carve-up
  const size_t qBytes = staged ? (((size_t)hqMax * q_stride(hdp) * 4 + 127) / 128) * 128 : 0;
  const size_t tileBytes = (((size_t)p.keySlots * p.kvPerCta * p.hd * esize + 127) / 128) * 128;
  const size_t ringBytes = (size_t)(bulk ? p.stages : 1) * 2 * tileBytes;
  const int lanes = p.lanesPerRow > 1 ? p.lanesPerRow : 1;
  const size_t mergeBytes = (size_t)p.keySlots * hqMax * lanes * (2 + hdp / lanes) * 4;
  const size_t newBytes = (staged && p.kNew) ? 2 * ((((size_t)p.kvPerCta * p.hd * esize) + 127) / 128) * 128 : 0;
  return qBytes + newBytes + (ringBytes > mergeBytes ? ringBytes : mergeBytes);
}

int padded_hd(int hd) { return hd <= 32 ? 32 : hd <= 64 ? 64 : 128; }
bool exact_hd(int hd) { return hd == 36 || hd == 52 || hd == 64 || hd == 128; }

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

// The bulk (TMA) path needs 16-byte aligned rows and slices.
bool bulk_ok(const DecodeParams& p, int esize) {
  if (!exact_hd(p.hd)) return false;
  const int64_t rowBytes = (int64_t)p.kvHeads * p.hd * esize;
  const int64_t sliceBytes = (int64_t)p.kvPerCta * p.hd * esize;
  if (rowBytes % 16 || sliceBytes % 16) return false;
  // (separately allocated caches are checked by the kernel, sequence by sequence)
  if (!p.kPtrs && ((p.cacheSeqStride * esize) % 16 || !aligned16(p.kCache) || !aligned16(p.vCache)))
    return false;
  if (p.hasSecond && !p.s2.kPtrs &&
      ((p.s2.cacheSeqStride * esize) % 16 || !aligned16(p.s2.kCache) || !aligned16(p.s2.vCache)))
    return false;
  if (p.kvHeads % p.kvPerCta) return false;  // a ragged last block changes the slice size
  return true;
}

template <typename T, int HDP, bool EXACT, int VEC, bool BULK, int R = 1>
cudaError_t launch_one(const DecodeParams& p, size_t smem, cudaStream_t s) {
  auto kern = decode_kernel<T, HDP, EXACT, VEC, BULK, R>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int zBlocks = (p.kvHeads + p.kvPerCta - 1) / p.kvPerCta;
  dim3 grid(p.splits, p.batch * (p.hasSecond ? 2 : 1), zBlocks);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(BULK ? kConsumers + 32 : kConsumers);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <typename T>
cudaError_t launch_typed(const DecodeParams& p, cudaStream_t s) {
  constexpr int esize = sizeof(T);
  constexpr int V = sizeof(T) == 2 ? 8 : 4;   // widest vector for the exact paths
  if (bulk_ok(p, esize)) {
    const size_t smem = smem_bytes(p, esize, p.hd, true);
    switch (p.hd) {
      case 36: return launch_one<T, 36, true, 4, true>(p, smem, s);
      case 52: return launch_one<T, 52, true, 4, true>(p, smem, s);
      case 64:
        return p.lanesPerRow == 2 ? launch_one<T, 64, true, V, true, 2>(p, smem, s)
                                  : launch_one<T, 64, true, V, true>(p, smem, s);
      case 128:
        return p.lanesPerRow == 4 ? launch_one<T, 128, true, V, true, 4>(p, smem, s)
                                  : launch_one<T, 128, true, V, true>(p, smem, s);
    }
  }
  if (p.lanesPerRow > 1) return cudaErrorInvalidValue;   // the plan promised the bulk path
  const int hdp = padded_hd(p.hd);
  const size_t smem = smem_bytes(p, esize, hdp, false);
  if (hdp == 32) return launch_one<T, 32, false, 1, false>(p, smem, s);
  if (hdp == 64) return launch_one<T, 64, false, 1, false>(p, smem, s);
  return launch_one<T, 128, false, 1, false>(p, smem, s);
}

}  // namespace

bool plan_decode(DecodeParams& p, int dtype, int smCount, std::string* err) {
  const int esize = dtype == RT_F16 ? 2 : 4;
  const int group = p.qHeads / p.kvHeads;
  if (group > kConsumers) {
    *err = "decode: more than 256 query heads per kv head";
    return false;
  }
  const int hdp = padded_hd(p.hd);
  // Head size 64 and 128: 2 or 4 threads share a (key, head) pair, 32 columns each (see
  // process_key_sub); that needs the bulk path, so fall back to whole rows without it.
  int lanes = p.hd == 128 ? 4 : p.hd == 64 ? 2 : 1;
  if (group * lanes > kConsumers) lanes = 1;
  // One geometry for a given shared-memory budget per CTA.
  struct Geom {
    int kvPerCta, keySlots, stages;
    size_t tile;
    bool fits;
  };
  auto geometry = [&](size_t budgetTotal, int lanesNow) {
    const int wdp = hdp / lanesNow;   // columns per thread
    Geom g{};
    g.kvPerCta = p.kvHeads;
    while (g.kvPerCta * group * lanesNow > kConsumers) g.kvPerCta = (g.kvPerCta + 1) / 2;
    // Key slots per tile: 256 threads' worth, fewer when two stages of that many keys do not
    // fit.  The heads stay together as long as a handful of key slots fit (wide heads then
    // leave some threads idle): a CTA that owns all the heads fetches a tile with one bulk
    // copy per tensor, while one that owns a single head needs a copy of hd elements per
    // key — measured 1.0 TB/s at 32 heads x 128, the copy engine's rate for 256-byte copies.
    constexpr int kMinKeySlots = 4;
    size_t budget;
    for (;;) {
      const size_t qBytes = lanesNow > 1 ? 128 :   // sub-row threads stage neither q nor the new row
                            (size_t)g.kvPerCta * group * q_stride(hdp) * 4 + 128 +
                            (p.kNew ? 2 * ((size_t)g.kvPerCta * p.hd * esize + 128) : 0);
      budget = budgetTotal > qBytes ? budgetTotal - qBytes : 0;
      g.keySlots = kConsumers / (g.kvPerCta * group * lanesNow);
      const size_t perSlot = 2ull * g.kvPerCta * p.hd * esize;            // K+V bytes of one key
      const size_t mergePerSlot = (size_t)g.kvPerCta * group * lanesNow * (2 + wdp) * 4;
      const size_t capTile = budget / 2 > 256 ? (budget / 2 - 256) / perSlot : 0;   // two stages must fit
      const size_t capMerge = budget / mergePerSlot;
      const size_t cap = capTile < capMerge ? capTile : capMerge;
      if (cap < (size_t)(g.keySlots < kMinKeySlots ? g.keySlots : kMinKeySlots) && g.kvPerCta > 1) {
        g.kvPerCta = (g.kvPerCta + 1) / 2;
        continue;
      }
      g.fits = cap >= 1;
      if (g.fits && (size_t)g.keySlots > cap) g.keySlots = (int)cap;
      break;
    }
    g.tile = ((2ull * g.keySlots * g.kvPerCta * p.hd * esize + 255) / 256) * 256 + 256;
    const int stages = g.fits ? (int)(budget / g.tile) : 0;
    g.stages = stages < 2 ? 2 : stages > kMaxStages ? kMaxStages : stages;
    return g;
  };
  // Up to 64 columns per thread, two CTAs fit an SM (registers), each with half of the
  // shared memory: one's set-up and merge overlap the other's streaming.  Sub-row threads
  // with only a few sequences to work on do better with one CTA per SM and a deep ring
  // (fewer, longer key splits; two tiles per barrier round): measured at 32 heads x 128,
  // KV 4096, 8 / 16 / 32 / 64 sequences: 147 / 195 / 261 / 249 us with one against
  // 270 / 286 / 234 / 248 us with two; the same crossing at 8 heads and at head size 64.
  Geom g{};
  int ctasPerSm = 1;
  for (;; lanes = 1) {
    const bool twoFit = hdp / lanes <= 64;
    const Geom one = geometry(kSmemBudget, lanes);
    g = one;
    ctasPerSm = 1;
    if (twoFit) {
      const Geom two = geometry(kSmemBudgetTwoPerSm, lanes);
      const int64_t seqCtas = (int64_t)p.batch * ((p.kvHeads + one.kvPerCta - 1) / one.kvPerCta);
      // Fewer blocks than SMs (a decode step of a small batch): a block alone on its SM takes
      // the whole shared memory for a ring twice as deep or more, and a block's copy rate is
      // what its ring keeps in flight over the memory latency (measured: 63 GB/s with two
      // 36 KB stages).
      const bool alone = seqCtas * (p.hasSecond ? 2 : 1) <= smCount;
      const bool fewSequences = one.fits && ((lanes > 1 && seqCtas * 8 <= smCount) || alone);
      if (two.fits && !fewSequences) {
        g = two;
        ctasPerSm = 2;
      }
    }
    p.kvPerCta = g.kvPerCta;
    p.lanesPerRow = lanes;
    if (lanes > 1 && !(g.fits && bulk_ok(p, esize))) continue;   // once more with whole rows
    if (!g.fits) {
      *err = "decode: heads too wide for shared memory";
      return false;
    }
    break;
  }
  const int kvPerCta = g.kvPerCta, keySlots = g.keySlots;
  p.kvPerCta = kvPerCta;
  p.keySlots = keySlots;
  p.stages = g.stages;

  if (p.splits <= 0) {
    const int zBlocks = (p.kvHeads + kvPerCta - 1) / kvPerCta;
    const int64_t ctas = (int64_t)p.batch * (p.hasSecond ? 2 : 1) * zBlocks;
    int64_t nmax = p.useRange ? (p.end >= p.lo ? p.end - p.lo + 1 : 0) : p.kvLen;
    if (p.hasSecond && p.s2.kvLen > nmax) nmax = p.s2.kvLen;
    if (p.kvSharded) {   // the longest stretch of a sequence this shard can hold
      nmax -= p.shardStart;
      nmax = nmax < 1 ? 1 : nmax > p.cacheRows ? p.cacheRows : nmax;
    }
    if (!p.useRange && p.wl < nmax) nmax = (int64_t)p.wl + 1;
    int64_t maxS = nmax / (4ll * keySlots);  // at least four tiles per split
    if (maxS > 32) maxS = 32;
    if (maxS < 1) maxS = 1;
    // Cost in units of one tile's streaming time: every CTA pays a fixed set-up,
    // pipeline-fill and merge cost (about three tiles' worth, measured), CTAs run in
    // waves of `resident` at a time, and splitting adds the partials pass.  Measured
    // on B200: with at least one wave of sequences, not splitting is fastest.
    const int64_t resident = (int64_t)smCount * ctasPerSm;
    int best = 1;
    int64_t bestCost = INT64_MAX;
    for (int s = 1; s <= maxS; s++) {
      const int64_t tilesPerCta = (nmax + (int64_t)s * keySlots - 1) / ((int64_t)s * keySlots);
      const int64_t waves = (ctas * s + resident - 1) / resident;
      const int64_t cost = waves * (3 + tilesPerCta) + (s > 1 ? 3 : 0);
      if (cost < bestCost) {
        bestCost = cost;
        best = s;
      }
    }
    p.splits = best;
  }
  return true;
}

cudaError_t launch_decode(const DecodeParams& p, int dtype, cudaStream_t s) {
  return dtype == RT_F16 ? launch_typed<__half>(p, s) : launch_typed<float>(p, s);
}

}  // namespace rt

// ---- decode without any allocation ---------------------------------------------
//
// Some hosts of this library must not allocate device memory when they call it:
// a real-time audio or serving loop that has pinned its memory budget up front,
// a plugin that runs inside another framework's memory pool, or code that runs
// while the device allocator is locked.  rt_attn_decode needs a context, and a
// context allocates (its stream, its status word, and the split scratch that
// grows on demand).  This entry point runs the same decode kernel with no
// context: the split scratch, the arrival counters and the status word live in
// the fixed-size device array below, which every GPU that loads the library
// holds until the process exits.
namespace rt {
namespace {

constexpr size_t kStaticScratchFloats = 1u << 20;   // 4 MiB of (m, l, acc) partials
constexpr size_t kStaticCounters = 4096;            // one per (sequence, head block)

struct StaticDecodeArea {
  float partials[kStaticScratchFloats];
  unsigned counters[kStaticCounters];
  int status;
};

static __device__ __align__(256) StaticDecodeArea gStaticDecodeArea;

constexpr int kMaxDevices = 64;
std::mutex gStaticMutex;
StaticDecodeArea* gStaticAddr[kMaxDevices];  // device address of the area, per device
int gStaticSmCount[kMaxDevices];

// Recorded where rt_last_error(NULL) finds it: this entry point has no context.
int static_fail(int code, const std::string& msg) {
  set_thread_error(msg.c_str());
  return code;
}

// The current device's copy of the area.  Set-up, once per device, with that device
// current: in host code the array's name is only a handle, the kernel needs its device
// address.
int static_area(StaticDecodeArea** area, int* smCount) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return static_fail(RT_EXECUTION_FAILED, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (device < 0 || device >= kMaxDevices)
    return static_fail(RT_UNSUPPORTED_DEVICE, "rt_attn_decode_noalloc: device ordinal " +
                                                  std::to_string(device) + " is past the " +
                                                  std::to_string(kMaxDevices) +
                                                  " devices this entry point keeps an address for");
  std::lock_guard<std::mutex> lock(gStaticMutex);
  if (!gStaticAddr[device]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, gStaticDecodeArea);
    if (e != cudaSuccess || !ptr)
      return static_fail(RT_EXECUTION_FAILED,
                         std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess || sms < 1)
      return static_fail(RT_EXECUTION_FAILED,
                         std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
    gStaticSmCount[device] = sms;
    gStaticAddr[device] = static_cast<StaticDecodeArea*>(ptr);
  }
  *area = gStaticAddr[device];
  *smCount = gStaticSmCount[device];
  return RT_OK;
}

}  // namespace
}  // namespace rt

extern "C" {

int rt_attn_decode_noalloc_status(void* cuda_stream) {
  using namespace rt;
  StaticDecodeArea* area;
  int smCount;
  if (int s = static_area(&area, &smCount)) return s;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaStreamSynchronize(stream);
  int status = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&status, &area->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess)
    return static_fail(RT_EXECUTION_FAILED,
                       std::string("rt_attn_decode_noalloc_status: ") + cudaGetErrorString(e));
  if (status == 0) return RT_OK;
  cudaMemset(&area->status, 0, sizeof(int));
  return static_fail(RT_EXECUTION_FAILED,
                     (status & kStatusWaitTimeout)
                         ? "rt_attn_decode_noalloc: a bounded device-side wait ran out"
                         : "rt_attn_decode_noalloc: a kvLens entry exceeds cacheRows");
}

int rt_attn_decode_noalloc(const rt_decode_args* a, void* cuda_stream) {
  using namespace rt;
  if (!a) return static_fail(RT_INVALID_ARGUMENT, "rt_attn_decode_noalloc: args is NULL");
  if (!a->q || (!a->kCache && !a->kCachePtrs) || (!a->vCache && !a->vCachePtrs) ||
      (!a->out && !a->partialsOut))
    return static_fail(RT_INVALID_ARGUMENT,
                       "rt_attn_decode_noalloc: q, kCache, vCache and out (or partialsOut) must be "
                       "device pointers");
  if (a->dtype != RT_F32 && a->dtype != RT_F16)
    return static_fail(RT_INVALID_ARGUMENT, "rt_attn_decode_noalloc: dtype is neither f32 nor f16");
  if (a->exchange)
    return static_fail(RT_INVALID_ARGUMENT,
                       "rt_attn_decode_noalloc: the cross-GPU exchange needs rt_attn_decode");
  if (a->batch < 1 || a->batch > 65535 || a->cacheRows < 1 || a->qHeads < 1 || a->headDim < 1 ||
      a->headDim > 128 || a->kvHeads < 1 || a->qHeads % a->kvHeads != 0 || a->kvLen < 0 ||
      (!a->kvSharded && a->kvLen > a->cacheRows) || (!a->kvLens && a->kvLen < 1) || a->windowLeft < 0 ||
      a->splits < 0 || a->splits > 64 || (a->kNew == nullptr) != (a->vNew == nullptr) ||
      a->cacheSeqStride < 0 ||
      (!a->kCachePtrs && a->batch > 1 &&
       a->cacheSeqStride < (int64_t)a->cacheRows * a->kvHeads * a->headDim) ||
      decode_rope_args_error(*a) != nullptr)
    return static_fail(RT_INVALID_ARGUMENT,
                       "rt_attn_decode_noalloc: a size or option is out of range (same rules as "
                       "rt_attn_decode)");

  StaticDecodeArea* area;
  int smCount;
  cudaError_t e;
  if (int s = static_area(&area, &smCount)) return s;

  DecodeParams p{};
  decode_params_from_args(*a, p);
  std::string err;
  if (!plan_decode(p, a->dtype, smCount, &err)) return static_fail(RT_INVALID_ARGUMENT, err);
  const size_t zBlocks = (size_t)(p.kvHeads + p.kvPerCta - 1) / p.kvPerCta;
  const size_t sets = p.hasSecond ? 2 : 1;
  const size_t needFloats = p.splits > 1 ? sets * p.batch * p.splits * p.qHeads * (2 + p.hd) : 0;
  const size_t needCounters = p.splits > 1 ? sets * p.batch * zBlocks : 0;
  if (needFloats > kStaticScratchFloats || needCounters > kStaticCounters)
    return static_fail(
        RT_INVALID_ARGUMENT,
        "rt_attn_decode_noalloc: batch*splits*qHeads*(2+headDim) = " + std::to_string(needFloats) +
            " floats (limit " + std::to_string(kStaticScratchFloats) + ") or batch*headBlocks = " +
            std::to_string(needCounters) + " counters (limit " + std::to_string(kStaticCounters) +
            ") exceeds the fixed scratch; pass fewer splits or a smaller batch");
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // The area keeps the last call's contents.  Partials are fully rewritten
  // before they are read; the arrival counters must start at zero.
  if (needCounters) {
    e = cudaMemsetAsync(area->counters, 0, needCounters * sizeof(unsigned), stream);
    if (e != cudaSuccess)
      return static_fail(RT_EXECUTION_FAILED,
                         std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  }
  p.scratch = area->partials;
  p.counters = area->counters;
  p.status = &area->status;
  e = launch_decode(p, a->dtype, stream);
  if (e != cudaSuccess)
    return static_fail(RT_EXECUTION_FAILED, std::string("decode launch: ") + cudaGetErrorString(e));
  return RT_OK;
}

}  // extern "C"
