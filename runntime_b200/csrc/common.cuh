// Shared declarations of the attention library's translation units.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <type_traits>

#include "rt_attn.h"

namespace rt {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegSeed = -1e30f;  // finite seed of the running max: buffers never hold +-Inf

// Bits of the device-side status word (rt_ctx::status_dev).  A kernel whose
// bounded wait runs out ORs a bit in and returns; rt_sync reports it.
constexpr int kStatusWaitTimeout = 1;
constexpr int kStatusBadState = 2;

// One attention problem as the kernels see it.  k and v already point at
// their column block when the tensors are packed; strides are in elements.
struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  const float* sinks;
  const float* segs;
  const int32_t* seqLens;
  int64_t qLen, kvLen;
  int64_t qStride, kvStride;
  int64_t qPosOffset;
  int32_t qHeads, kvHeads, hd;
  int32_t wl, wr;
  int32_t hasKeyBias, biasStart, biasEnd;
  float biasValue;
  int32_t seqStride;
  int32_t maxSegment;
};

// Visible key range [lo, end] (inclusive) of query row `row`; empty when lo > end.
// Rule: packages/runntime/src/core/kernels/attention/attn.ts:150-156 (window,
// then segment clip), with the padded-batch form derived from seqLens.
__device__ __forceinline__ void row_band(const AttnParams& p, int64_t row, int64_t& lo,
                                         int64_t& end) {
  const int64_t qPos = p.qPosOffset + row;
  lo = qPos - p.wl;
  if (lo < 0) lo = 0;
  end = qPos + p.wr;
  if (end > p.kvLen - 1) end = p.kvLen - 1;
  if (p.segs) {
    const int64_t s0 = (int64_t)p.segs[2 * row];
    const int64_t s1 = (int64_t)p.segs[2 * row + 1] - 1;
    if (s0 > lo) lo = s0;
    if (s1 < end) end = s1;
  } else if (p.seqStride > 0) {
    const int64_t b = row / p.seqStride;
    const int64_t r = row - b * p.seqStride;
    const int64_t len = p.seqLens[b];
    if (r >= len) {
      lo = 1;
      end = 0;
    } else {
      const int64_t s0 = b * p.seqStride;
      if (s0 > lo) lo = s0;
      if (s0 + len - 1 < end) end = s0 + len - 1;
    }
  }
}

// A second attention computed by the same decode launch (the cross-attention that follows
// the self-attention of a decoder layer): its own q, out, caches and lengths; no append, no
// rope; same heads, head size, dtype and sinks.
struct DecodeSecond {
  const void* q;
  void* out;
  void* kCache;
  void* vCache;
  const void* const* kPtrs;
  const void* const* vPtrs;
  const int32_t* kvLens;
  int64_t cacheSeqStride, qRowStride;
  int32_t cacheRows, kvLen, wl;
};

struct DecodeParams {
  const void* q;
  void* out;
  void* kCache;
  void* vCache;
  const void* kNew;
  const void* vNew;
  const int32_t* kvLens;
  const float* sinks;
  float* partialsOut;   // final destination is partials (m, l, acc) instead of out
  float* scratch;       // [batch, splits, qHeads, 2+hd] f32, used when splits > 1
  unsigned* counters;   // [batch * headBlocks], zero between launches
  int* status;
  int64_t cacheSeqStride;
  int64_t lo, end;      // explicit key range (useRange), for the single-sequence op
  int32_t useRange;
  int32_t batch, kvLen, qHeads, kvHeads, hd, wl, splits;
  int32_t cacheRows;    // capacity of each cache in rows: a device-side length past it is refused
  int32_t kvPerCta;     // kv heads handled by one CTA
  int32_t keySlots;     // keys processed concurrently by one CTA
  int32_t stages;       // smem ring depth (bulk path)
  int32_t lanesPerRow;  // threads that share one (key, head) pair, each a slice of the head (1, 2, 4)
  // fused rope (null tables = off) and row strides of q / kNew / vNew, in elements
  const float* ropeCos;
  const float* ropeSin;
  int32_t ropeByPos;
  int64_t qRowStride, kNewRowStride, vNewRowStride;
  // cross-GPU exchange of the final partials (xWorld = 0: off); see rt_exchange
  float* xPartials[RT_MAX_PEERS];
  uint32_t* xFlags[RT_MAX_PEERS];
  uint32_t* xStep;      // this rank's counter block: step, (unused), [world] arrivals per owner, owners done
  float* xStage;        // this rank's final rows before they go to their owners: [batch, qHeads, 2+hd]
  int32_t xWorld, xRank;
  int32_t xPer;         // sequences per owner: rank o merges sequences [o*xPer, (o+1)*xPer)
  int32_t xRot;         // added to blockIdx.y: a rank's own sequences are attended last
  // KV-sequence sharding with append: this cache holds global rows [shardStart,
  // shardStart + cacheRows) of every sequence and kvLens are global lengths
  int32_t kvSharded, shardStart;
  // per-sequence cache pointers (device arrays [batch]) instead of one slab; NULL = slab
  const void* const* kPtrs;
  const void* const* vPtrs;
  // a second attention in the same launch: blockIdx.y in [batch, 2*batch)
  int32_t hasSecond;
  DecodeSecond s2;
};

// Who merges which sequences in the cross-GPU exchange: contiguous blocks balanced to within
// one sequence (the first batch % world ranks own one more); every rank owns at least one,
// which the API ensures by refusing batch < world (a rank with nothing to merge would have
// nothing to wait for and could run steps ahead of the others).
#ifdef __CUDACC__
#define RT_HD __host__ __device__
#else
#define RT_HD
#endif
RT_HD inline int exchange_per(int batch, int world) { return (batch + world - 1) / world; }
RT_HD inline int owner_first(int o, int batch, int world) {
  const int base = batch / world, extra = batch % world;
  return o * base + (o < extra ? o : extra);
}
RT_HD inline int owner_count(int o, int batch, int world) {
  return batch / world + (o < batch % world ? 1 : 0);
}
RT_HD inline int owner_of(int b, int batch, int world) {
  const int base = batch / world, extra = batch % world, cut = extra * (base + 1);
  return b < cut ? b / (base + 1) : extra + (b - cut) / base;
}

// Copies the caller's decode arguments (already validated) into kernel parameters.
inline void decode_params_from_args(const rt_decode_args& a, DecodeParams& p) {
  p.q = a.q;
  p.out = a.out;
  p.kCache = a.kCache;
  p.vCache = a.vCache;
  p.kNew = a.kNew;
  p.vNew = a.vNew;
  p.kvLens = a.kvLens;
  p.sinks = a.sinks;
  p.partialsOut = a.partialsOut;
  p.cacheSeqStride = a.cacheSeqStride;
  p.batch = a.batch;
  p.cacheRows = a.cacheRows;
  p.kvLen = a.kvLens ? (a.kvLen > 0 ? a.kvLen : a.cacheRows) : a.kvLen;
  p.qHeads = a.qHeads;
  p.kvHeads = a.kvHeads;
  p.hd = a.headDim;
  p.wl = a.windowLeft;
  p.splits = a.splits;
  p.ropeCos = a.ropeCos;
  p.ropeSin = a.ropeSin;
  p.ropeByPos = a.ropeByPosition;
  p.qRowStride = a.qRowStride ? a.qRowStride : (int64_t)a.qHeads * a.headDim;
  p.kNewRowStride = a.kNewRowStride ? a.kNewRowStride : (int64_t)a.kvHeads * a.headDim;
  p.vNewRowStride = a.vNewRowStride ? a.vNewRowStride : (int64_t)a.kvHeads * a.headDim;
  p.xWorld = 0;
  if (a.exchange) {
    p.xWorld = a.exchange->world;
    p.xRank = a.exchange->rank;
    for (int r = 0; r < RT_MAX_PEERS; r++) {
      p.xPartials[r] = r < a.exchange->world ? a.exchange->partials[r] : nullptr;
      p.xFlags[r] = r < a.exchange->world ? a.exchange->flags[r] : nullptr;
    }
    p.xStep = a.exchange->step;
    p.xStage = a.exchange->stage;
    p.xPer = exchange_per(a.batch, a.exchange->world);
    p.xRot = owner_first((a.exchange->rank + 1) % a.exchange->world, a.batch, a.exchange->world);
    p.partialsOut = nullptr;
  }
  p.kvSharded = a.kvSharded;
  p.shardStart = a.shardStart;
  p.kPtrs = a.kCachePtrs;
  p.vPtrs = a.vCachePtrs;
  p.hasSecond = 0;
  if (a.second) {
    const rt_decode_second& x = *a.second;
    p.hasSecond = 1;
    p.s2.q = x.q;
    p.s2.out = x.out;
    p.s2.kCache = x.kCache;
    p.s2.vCache = x.vCache;
    p.s2.kPtrs = x.kCachePtrs;
    p.s2.vPtrs = x.vCachePtrs;
    p.s2.kvLens = x.kvLens;
    p.s2.cacheSeqStride = x.cacheSeqStride;
    p.s2.qRowStride = x.qRowStride ? x.qRowStride : (int64_t)a.qHeads * a.headDim;
    p.s2.cacheRows = x.cacheRows;
    p.s2.kvLen = x.kvLens ? (x.kvLen > 0 ? x.kvLen : x.cacheRows) : x.kvLen;
    p.s2.wl = x.windowLeft;
  }
}

// What is wrong with the rope / stride fields of decode arguments, or NULL.
inline const char* decode_rope_args_error(const rt_decode_args& a) {
  if ((a.ropeCos == nullptr) != (a.ropeSin == nullptr)) return "ropeCos and ropeSin go together";
  if (a.ropeCos && a.headDim % 2 != 0) return "rope: headDim must be a positive even integer";
  if (a.qRowStride < 0 || (a.qRowStride && a.qRowStride < (int64_t)a.qHeads * a.headDim))
    return "qRowStride is smaller than one q row";
  const int64_t kvw = (int64_t)a.kvHeads * a.headDim;
  if (a.kNewRowStride < 0 || (a.kNewRowStride && a.kNewRowStride < kvw) ||
      a.vNewRowStride < 0 || (a.vNewRowStride && a.vNewRowStride < kvw))
    return "kNewRowStride / vNewRowStride is smaller than one kv row";
  if (a.exchange) {
    const rt_exchange& x = *a.exchange;
    if (x.world < 1 || x.world > RT_MAX_PEERS || x.rank < 0 || x.rank >= x.world)
      return "exchange: world must be 1..8 and rank inside it";
    if (!x.step || !x.stage || !a.out) return "exchange: step, stage and out must be given";
    if (a.batch < x.world) return "exchange: batch must be at least world (every rank merges a sequence)";
    if (x.phases < 0 || x.phases > 3) return "exchange: phases must be 0..3";
    for (int r = 0; r < x.world; r++)
      if (!x.partials[r] || !x.flags[r]) return "exchange: a peer buffer is NULL";
  }
  if ((a.kCachePtrs == nullptr) != (a.vCachePtrs == nullptr)) return "kCachePtrs and vCachePtrs go together";
  if (a.second) {
    const rt_decode_second& x = *a.second;
    if (a.exchange || a.partialsOut || a.kvSharded)
      return "second: not with the cross-GPU exchange, partialsOut or a sharded cache";
    if (!x.q || !x.out || (!x.kCache && !x.kCachePtrs) || (!x.vCache && !x.vCachePtrs))
      return "second: q, out and the caches must be device pointers";
    if ((x.kCachePtrs == nullptr) != (x.vCachePtrs == nullptr)) return "second: kCachePtrs and vCachePtrs go together";
    if (x.cacheRows < 1 || x.kvLen < 0 || x.kvLen > x.cacheRows || (!x.kvLens && x.kvLen < 1))
      return "second: kvLen must lie within cacheRows";
    if (x.windowLeft < 0 || x.windowLeft > RT_WINDOW_INF) return "second: windowLeft must be a non-negative integer or Infinity";
    if (x.cacheSeqStride < 0 || (!x.kCachePtrs && a.batch > 1 &&
                                 x.cacheSeqStride < (int64_t)x.cacheRows * a.kvHeads * a.headDim))
      return "second: cacheSeqStride is smaller than one cache";
    if (x.qRowStride < 0 || (x.qRowStride && x.qRowStride < (int64_t)a.qHeads * a.headDim))
      return "second: qRowStride is smaller than one q row";
  }
  if (a.kvSharded != 0 && a.kvSharded != 1) return "kvSharded must be 0 or 1";
  if (a.shardStart < 0 || (!a.kvSharded && a.shardStart != 0))
    return "shardStart must be non-negative, and zero unless kvSharded is set";
  return nullptr;
}

#ifdef __CUDACC__
// One interleaved pair of the rotary embedding:
// packages/runntime/src/core/kernels/attention/rope.ts:60-68.  Spelled with
// intrinsics so that every kernel using it rounds the same way (the compiler is
// otherwise free to contract a*b - c*d differently from one kernel to the next).
__device__ __forceinline__ void rope_pair(float x0, float x1, float c, float s, float& r0,
                                          float& r1) {
  r0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
  r1 = __fmaf_rn(x1, c, __fmul_rn(x0, s));
}
#endif

#ifdef __CUDACC__
// The epilogue activations of matmul (codes and formulas: packages/runntime/src/core/
// kernels/activations.ts:6-86; gelu uses the reference's erf polynomial, Abramowitz-Stegun
// 7.1.26).  A template, so that a kernel branches on the code once per tile and not per
// element — written as a switch in the element loop the compiler evaluates every case
// for every element and selects.
template <int ACT>
__device__ __forceinline__ float act_apply(float x) {
  if (ACT == 1) return tanhf(x);
  if (ACT == 2) {
    const float z = x * 0.70710678118654752f, az = fabsf(z);
    const float t = 1.f / (1.f + az * 0.3275911f);
    const float poly = t * (0.254829592f + t * (-0.284496736f + t * (1.421413741f +
                       t * (-1.453152027f + t * 1.061405429f))));
    return 0.5f * x * (1.f + copysignf(1.f - poly * __expf(-az * az), z));
  }
  if (ACT == 3) return x / (1.f + __expf(-x));
  if (ACT == 4) return fmaxf(x, 0.f);
  if (ACT == 5) {  // torch's gelu(approximate='tanh'), tanh as 1 - 2/(e^{2u} + 1)
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (2.f - 2.f / (__expf(2.f * u) + 1.f));
  }
  if (ACT == 6) return fmaxf(x, 0.f) + (__expf(fminf(x, 0.f)) - 1.f);
  return x;
}
// Calls f(std::integral_constant<int, ACT>) for the runtime code `act` (0..6).
template <typename F>
__device__ __forceinline__ void act_dispatch(int act, F&& f) {
  switch (act) {
    case 1: f(std::integral_constant<int, 1>{}); break;
    case 2: f(std::integral_constant<int, 2>{}); break;
    case 3: f(std::integral_constant<int, 3>{}); break;
    case 4: f(std::integral_constant<int, 4>{}); break;
    case 5: f(std::integral_constant<int, 5>{}); break;
    case 6: f(std::integral_constant<int, 6>{}); break;
    default: f(std::integral_constant<int, 0>{}); break;
  }
}
#endif

// Launchers (defined one per .cu).  Each returns a cudaError_t from the launch.
cudaError_t launch_prefill_simt(const AttnParams& p, int dtype, cudaStream_t s);
bool prefill_tc_supported(const AttnParams& p, int dtype);
cudaError_t launch_prefill_tc(const AttnParams& p, int dtype, int* status, cudaStream_t s,
                              std::string* err);
// Two query tiles per CTA (head sizes 64 and 128, more than 128 query rows).
bool prefill_tc2_supported(const AttnParams& p, int dtype);
cudaError_t launch_prefill_tc2(const AttnParams& p, int* status, cudaStream_t s, std::string* err);
// One query tile per CTA, two softmax warpgroups on alternate key tiles (head sizes 64, 128,
// 256, and heads narrower than 64 padded inside the tile).
bool prefill_tc3_supported(const AttnParams& p, int dtype);
// ... and the same with pairs of CTAs (a cluster of two) sharing every K/V tile.
bool prefill_tc3_pair_supported(const AttnParams& p, int dtype);
cudaError_t launch_prefill_tc3(const AttnParams& p, bool pair, int* status, cudaStream_t s,
                               std::string* err);
// Persistent form (one CTA per SM over a queue of units); `work`: two zeroed ints the kernel
// leaves zeroed.
bool prefill_tc4_supported(const AttnParams& p, int dtype);
cudaError_t launch_prefill_tc4(const AttnParams& p, int* status, int* work, int smCount,
                               cudaStream_t s, std::string* err);
// Fills kvPerCta/keySlots/stages/splits; returns false with a message when the shape cannot run.
bool plan_decode(DecodeParams& p, int dtype, int smCount, std::string* err);
cudaError_t launch_decode(const DecodeParams& p, int dtype, cudaStream_t s);
cudaError_t launch_merge_partials(const float* partials, int parts, int64_t units, int hd,
                                  void* out, int dtype, cudaStream_t s);
// Merge of the exchanged partials on the rank that owns sequences [firstSeq, firstSeq+owned):
// waits (at most `limit` polls) for every rank's arrival word to reach *step.
cudaError_t launch_merge_exchanged(const float* buffer, const uint32_t* flags, const uint32_t* step,
                                   int world, int per, int owned, int firstSeq, int heads, int hd,
                                   void* out, int dtype, int* status, int limit, cudaStream_t s);
cudaError_t launch_rope(const void* x, const float* cosT, const float* sinT, void* out,
                        int64_t rows, int64_t srcCols, int hd, int64_t srcStart, int64_t width,
                        int dtype, cudaStream_t s);
// Scratch (f32 partial sums of the K slices) a matmul of this shape wants; 0 = none.
size_t matmul_scratch_need(int64_t M, int64_t K, int64_t N, int dtype);
cudaError_t launch_matmul(const void* a, const void* b, const void* bias, const void* addend,
                          void* out, int64_t M, int64_t K, int64_t N, int act, int dtype,
                          float* scratch, cudaStream_t s);
// Tensor-core path of matmul (f16, more than 16 rows, aligned shapes).
bool matmul_tc_supported(const void* a, const void* b, const void* out, int64_t M, int64_t K,
                         int64_t N, int dtype);
cudaError_t launch_matmul_tc(const void* a, const void* b, const void* bias, const void* addend,
                             void* out, int64_t M, int64_t K, int64_t N, int act, int* status,
                             cudaStream_t s, std::string* err);
cudaError_t launch_argmax_dot(const void* w, const void* x, float* out, int64_t V, int64_t N,
                              int dtype, unsigned long long* scratch, cudaStream_t s);
cudaError_t launch_local_attn(const void* qkv, const float* rel, const float* qScale, void* out,
                              int64_t rows, int heads, int hd, int window, float kScale,
                              float softcap, int dtype, cudaStream_t s);
cudaError_t launch_softmax(const void* x, void* out, const float* segs, int64_t rows, int64_t cols,
                           int64_t wl, int64_t wr, int dtype, cudaStream_t s);
cudaError_t launch_slice(const void* x, void* out, int64_t rows, int64_t srcColBytes,
                         int64_t offsetBytes, int64_t widthBytes, cudaStream_t s);
cudaError_t launch_write_rows(void* dst, const void* src, int64_t dstOffsetBytes, int64_t bytes,
                              cudaStream_t s);

// Records `msg` as the calling thread's last error (what rt_last_error(NULL) returns).
void set_thread_error(const char* msg);

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

}  // namespace rt
