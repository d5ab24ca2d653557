/* rt_attn.h — C ABI of the B200 attention library (librt_attn.so).
 *
 * This is the boundary a host runtime binds (N-API, ctypes, cgo ...): plain
 * pointers, sizes and status codes.  Every pointer named "device" is a CUDA
 * device address on the context's GPU; they stand where the reference holds
 * GPUBuffer handles.  All work is enqueued on the context's stream in call
 * order (the reference relies on in-pass dispatch order the same way,
 * packages/runntime/src/core/kernels/attention/attnDecode.ts:228-235); only
 * rt_sync and rt_buf_download wait for the device.
 *
 * Every function returns an rt_status.  On failure rt_last_error() gives the
 * message; argument errors are detected before anything is enqueued.  A
 * context is to be used from one thread at a time.
 */
#ifndef RT_ATTN_H
#define RT_ATTN_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define RT_API __attribute__((visibility("default")))
#else
#define RT_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes, one per entry of the reference's RUNNTIME_ERROR_CODES
 * (packages/runntime/src/core/error.ts:4-21), in the same order, after RT_OK. */
typedef enum {
  RT_OK = 0,
  RT_LOAD_FAILED = 1,
  RT_LOAD_ABORTED = 2,
  RT_CHECKPOINT_MISMATCH = 3,
  RT_UNSUPPORTED_DEVICE = 4,
  RT_EXECUTION_FAILED = 5,
  RT_INVALID_ARGUMENT = 6,
  RT_RESOURCE_DISPOSED = 7,
  RT_NOT_INITIALIZED = 8
} rt_status;

/* Storage element types (packages/runntime/src/core/kernels/elem.ts:1-6);
 * accumulation and softmax state are always f32.  f16 is raw IEEE halfwords. */
typedef enum { RT_F32 = 0, RT_F16 = 1 } rt_dtype;

/* Finite stand-in for an unbounded window side
 * (packages/runntime/src/core/graph/ops/shared.ts:37). */
#define RT_WINDOW_INF 0x3fffffff

typedef struct rt_ctx rt_ctx;

/* ---- context: replaces initRuntime/gpuExecutor/dispose --------------------
 * (packages/runntime/src/core/gpu/eval.ts:80-88,135,274-283).  Owns a stream
 * and the split-KV scratch, which grows monotonically like the executor's
 * scratch (eval.ts:194-203).  After rt_ctx_destroy every use of the handle is
 * an error (RT_RESOURCE_DISPOSED is returned while the handle's memory is
 * still recognisable; do not rely on it). */
RT_API int rt_ctx_create(int device, rt_ctx** out);
RT_API int rt_ctx_destroy(rt_ctx* ctx);
/* external != 0: enqueue on the caller's stream `cuda_stream` (a cudaStream_t;
 * NULL is the legacy default stream) instead of the context's own, so that
 * the library's kernels order with the caller's other work.  external == 0
 * restores the context's stream. */
RT_API int rt_ctx_set_stream(rt_ctx* ctx, void* cuda_stream, int external);
/* Context options.  RT_OPT_PREFILL_TC (default 1): route eligible f16 prefill
 * shapes to a tensor-core kernel of the library's choice (head sizes 64, 128,
 * 256 and the narrow heads: one 128-row query tile per thread block whose key
 * tiles alternate between two softmax warpgroups).  0 sends every prefill to the FP32-pipe kernel; 2 forces one tile
 * with one warpgroup, 3 two tiles per block, 4 the alternating form, 5 the
 * alternating form on pairs of thread blocks that share every K/V tile, 6 the
 * alternating form as one persistent thread block per SM over a queue of query
 * tiles — each where that kernel applies (all compute the same op; the switch exists for
 * testing and measurement). */
#define RT_OPT_PREFILL_TC 1
/* RT_OPT_WAIT_POLLS (default 1 << 20, about a second): how often the merge of a
 * cross-GPU decode step polls for the other ranks' rows before it gives up, writes
 * zeros and makes rt_sync return RT_EXECUTION_FAILED. */
#define RT_OPT_WAIT_POLLS 2
RT_API int rt_ctx_set_option(rt_ctx* ctx, int option, int value);
/* Message of the last failure on this context (or, with ctx == NULL, of the
 * last failed call on this thread that had no context to record it in). */
RT_API const char* rt_last_error(const rt_ctx* ctx);
/* Waits for everything enqueued so far; reports asynchronous kernel status
 * (a bounded device-side wait that ran out is RT_EXECUTION_FAILED). */
RT_API int rt_sync(rt_ctx* ctx);
/* Number of kernels this context has launched since creation. */
RT_API int64_t rt_launch_count(const rt_ctx* ctx);

/* ---- buffers: replace createStorageFor / writeF32 / writeF16 / readback ----
 * (packages/runntime/src/core/gpu/buffers.ts:83-121,171-181,302-308).
 * A zero-byte allocation is RT_INVALID_ARGUMENT, as uploading an empty tensor
 * is in the reference (buffers.ts:108-111). */
RT_API int rt_buf_alloc(rt_ctx* ctx, size_t bytes, void** device_ptr);
RT_API int rt_buf_free(rt_ctx* ctx, void* device_ptr);
RT_API int rt_buf_upload(rt_ctx* ctx, void* device_ptr, size_t offset, const void* host, size_t bytes);
RT_API int rt_buf_download(rt_ctx* ctx, const void* device_ptr, size_t offset, void* host,
                    size_t bytes);

/* ---- the 'attn' op ---------------------------------------------------------
 * One call = one pending 'attn' node of the reference; the fields are its
 * attrs vector and inputs (packages/runntime/src/core/graph/ops/attention.ts:
 * 122-140, 207-211) and the dispatch it replaces is attnSpec
 * (packages/runntime/src/core/gpu/dispatch/attention.ts:45-199).
 *
 * Layouts, all row-major: q [qLen, qHeads*headDim], k and v
 * [kvLen, kvHeads*headDim], out [qLen, qHeads*headDim]; with qkvPacked = 1,
 * q == k == v point at one [qLen, (qHeads+2*kvHeads)*headDim] tensor whose
 * column blocks are q|k|v and kvLen == qLen.  Key j is visible to row i when
 * qPos-windowLeft <= j <= qPos+windowRight (qPos = qPosOffset+i), clipped to
 * [segments[2i], segments[2i+1]) when segments is given.  No score scale is
 * applied.  sinks[h]*ln2 seeds the running max with weight 1 in the
 * denominator only.  A row that sees no key is written as zeros.
 *
 * Two batch extensions (zero / NULL for the plain reference op):
 *   seqStride > 0 with seqLens != NULL: rows are `batch` sequences of
 *   seqStride rows back to back (qLen == kvLen == batch*seqStride); row r of
 *   sequence b = r / seqStride sees only keys [b*seqStride, b*seqStride +
 *   seqLens[b]) and rows at or past seqLens[b] are written as zeros.  This is
 *   the segments form computed on the fly; segments must then be NULL.
 */
typedef struct {
  const void* q;          /* device */
  const void* k;          /* device */
  const void* v;          /* device */
  void* out;              /* device */
  const float* sinks;     /* device [qHeads] or NULL */
  const float* segments;  /* device [qLen, 2] f32 or NULL */
  int32_t dtype;          /* rt_dtype of q, k, v and out */
  int32_t qkvPacked;
  int64_t qLen;
  int64_t kvLen;
  int32_t qHeads;
  int32_t kvHeads;
  int32_t headDim;
  int32_t windowLeft;     /* RT_WINDOW_INF = unbounded */
  int32_t windowRight;
  int32_t maxSegment;     /* longest segment, 0 = unknown; a sizing hint only */
  int64_t qPosOffset;
  int32_t hasKeyBias;
  int32_t biasStart;
  int32_t biasEnd;
  float biasValue;
  int32_t seqStride;        /* batch extension, see above */
  const int32_t* seqLens;   /* device [qLen / seqStride] or NULL */
} rt_attn_args;

/* Runs the op.  qLen == 1 takes the decode kernel (headDim <= 128, no
 * segments, no key bias — the reference's limits, ops/attention.ts:10-12,
 * 96-98,119-120); otherwise a prefill kernel (headDim <= 512; qkvPacked
 * needs headDim <= 128). */
RT_API int rt_attn(rt_ctx* ctx, const rt_attn_args* args);

/* Which kernel rt_attn would run for these arguments: writes a short static
 * name into *route: "decode", "prefill_simt" (FP32 pipes), or one of the
 * tensor-core kernels "prefill_tc3" (the default), "prefill_tc3_pair",
 * "prefill_tc4", "prefill_tc2", "prefill_tc" (see RT_OPT_PREFILL_TC). */
RT_API int rt_attn_route(rt_ctx* ctx, const rt_attn_args* args, const char** route);

/* ---- batched single-token decode over KV caches -----------------------------
 * The decode step of the KV-cache engine (packages/runntime/src/zoo/moonshine/
 * decoder.ts:58-76,105-109; transcriber.ts:111-118,161-203) for `batch`
 * independent sequences in one launch.  The reference runs one sequence per
 * call; batch = 1 is that call.
 *
 * kCache/vCache: `batch` caches of [cacheRows, kvHeads*headDim] each,
 * cacheSeqStride ELEMENTS apart.  Sequence b attends, with its single query
 * row q[b], to cache rows [max(0, L_b-1-windowLeft), L_b-1] where
 * L_b = kvLens[b] (or kvLen when kvLens is NULL): causal self-attention with
 * the query at the last position, or cross-attention over all L_b rows when
 * windowLeft is RT_WINDOW_INF.
 *
 * Fused append: when kNew and vNew are given ([batch, kvHeads*headDim]) the
 * kernel first stores kNew[b]/vNew[b] into cache row L_b-1 — exactly what
 * writeRows(cache, new, L_b-1) does (ops/shape.ts:230-259), rows past the view
 * keep their contents — and attends to them.
 *
 * Fused rope: when ropeCos and ropeSin are given (pair-duplicated f32 tables,
 * any scale folded in, as for rt_rope) q[b] and kNew[b] are the UN-rotated
 * rows and the kernel rotates them itself — rounding the result to `dtype`
 * exactly as the separate rope dispatch stores it — before the append and the
 * scores.  Table row: L_b-1 when ropeByPosition is set (one table
 * [positions, headDim] for the whole model), else b (tables [batch, headDim]
 * gathered by the caller; with batch 1 that is the reference's cosRow/sinRow).
 * Together with the row strides this lets q, kNew and vNew point into the one
 * fused qkv row the projection wrote, so a decoder layer's rope x 2, slice,
 * writeRows x 2 and attention (decoder.ts:58-76) become one launch.
 *
 * partialsOut != NULL: instead of `out`, writes un-normalised partials
 * f32 [batch, qHeads, 2+headDim] = (m, l, acc) per head for a later
 * rt_attn_merge_partials (KV-sequence sharding across GPUs); keyOffset is
 * not needed because the softmax algebra is position-free. */
/* Exchange of the partials between the GPUs that hold the KV rows of the same
 * sequences (KV-sequence sharding: rank r's caches hold rows [r*cacheRows,
 * (r+1)*cacheRows) of every sequence).  Every pointer below is an address in
 * THIS process: a peer's block mapped here (rt_xmem_* below does that; any other
 * peer mapping works too).  With it rt_attn_decode
 *   1. attends to this rank's rows and sends the (m, l, acc) rows of each
 *      sequence, from the decode kernel, with plain stores, to the ONE rank that
 *      merges that sequence: the ranks own contiguous blocks of sequences,
 *      balanced to within one (the first batch % world ranks own one more; batch
 *      must be at least world).  The last thread block to finish an owner's
 *      sequences publishes this rank's step in that owner's arrival word;
 *   2. runs a merge kernel over this rank's own sequences that first waits
 *      (bounded, about a second; RT_OPT_WAIT_POLLS) until every rank's arrival word
 *      has reached the step: the decode step, the all-gather and the merge of
 *      packages/runntime/src/core/kernels/attention/attnDecode.ts:388-424 lifted
 *      across devices, without a library collective and without a second signal
 *      launch.
 * `out` therefore receives the rows of this rank's own sequences only; the rest
 * of `out` is left alone: the
 * output stays sharded by sequence, which is how the layers after attention want
 * it.  Every rank must make the same sequence of calls.  Buffers alternate
 * between two halves by step parity, so a rank one step ahead never overwrites
 * rows a slower peer is still merging.  All words start at zero.  After a wait
 * has run out (rt_sync: RT_EXECUTION_FAILED) the counters are no longer
 * consistent: make a new exchange. */
#define RT_MAX_PEERS 8
typedef struct {
  int32_t world;                   /* ranks sharing the sequences, 1..RT_MAX_PEERS */
  int32_t rank;                    /* this rank */
  float* partials[RT_MAX_PEERS];   /* rank r's buffer: f32 [2][world][per*qHeads][2+headDim],
                                      per = ceil(batch / world) */
  uint32_t* flags[RT_MAX_PEERS];   /* rank r's arrival words: [world] */
  uint32_t* step;                  /* this rank's counters: [world + 3] words (step, spare,
                                      thread blocks arrived per owner, owners done) */
  float* stage;                    /* this rank's staging rows: f32 [batch*qHeads][2+headDim] */
  int32_t phases;                  /* 0 or 3: the whole step; 1: attend and send only; 2: wait and
                                      merge only (for callers that put other work in between) */
} rt_exchange;

/* A second attention computed by the same launch: the cross-attention over the encoder
 * states that follows the self-attention of a decoder layer (packages/runntime/src/zoo/
 * moonshine/decoder.ts:58-76 then :105-109) — its own query rows, output, caches and
 * lengths; no append and no rope; heads, head size, dtype and sinks are the call's. */
typedef struct {
  const void* q;          /* device [batch, qHeads*headDim] */
  void* out;              /* device [batch, qHeads*headDim] */
  void* kCache;           /* device slab, or NULL with kCachePtrs */
  void* vCache;
  const void* const* kCachePtrs; /* device [batch] of device pointers, or NULL */
  const void* const* vCachePtrs;
  const int32_t* kvLens;  /* device [batch] or NULL */
  int64_t cacheSeqStride; /* elements between the sequences' caches (slab form) */
  int64_t qRowStride;     /* elements between q rows; 0 = dense */
  int32_t cacheRows;
  int32_t kvLen;          /* used when kvLens == NULL */
  int32_t windowLeft;     /* RT_WINDOW_INF for cross-attention */
} rt_decode_second;

typedef struct {
  const void* q;          /* device [batch, qHeads*headDim] */
  void* out;              /* device [batch, qHeads*headDim] (unused with partialsOut) */
  void* kCache;           /* device */
  void* vCache;           /* device */
  const void* kNew;       /* device [batch, kvHeads*headDim] or NULL */
  const void* vNew;       /* device or NULL (both or neither) */
  const int32_t* kvLens;  /* device [batch] or NULL */
  const float* sinks;     /* device [qHeads] or NULL */
  float* partialsOut;     /* device [batch, qHeads, 2+headDim] or NULL */
  int64_t cacheSeqStride; /* elements between consecutive sequences' caches */
  int32_t dtype;
  int32_t batch;
  int32_t cacheRows;      /* capacity of each cache, rows */
  int32_t kvLen;          /* used when kvLens == NULL */
  int32_t qHeads;
  int32_t kvHeads;
  int32_t headDim;
  int32_t windowLeft;
  int32_t splits;         /* key splits per sequence; 0 = let the library choose */
  int32_t ropeByPosition; /* rope table row: 0 = b, 1 = L_b-1 */
  const float* ropeCos;   /* device f32 [batch or positions, headDim] or NULL */
  const float* ropeSin;   /* device or NULL (both or neither) */
  int64_t qRowStride;     /* elements between q rows; 0 = qHeads*headDim (dense) */
  int64_t kNewRowStride;  /* elements between kNew rows; 0 = kvHeads*headDim */
  int64_t vNewRowStride;  /* elements between vNew rows; 0 = kvHeads*headDim */
  const rt_exchange* exchange; /* host pointer or NULL: merge with the other ranks' rows into out */
  /* KV-sequence sharding with append (0 / 0 for a cache that holds whole sequences):
   * with kvSharded = 1 each cache holds rows [shardStart, shardStart + cacheRows) of its
   * sequence, and kvLen / kvLens are the sequences' GLOBAL lengths.  The kernel attends
   * to the rows of [0, L_b) that fall inside the shard and appends kNew/vNew (global
   * row L_b-1) only on the rank whose shard contains that row; every rank passes the
   * same q, kNew, vNew and lengths.  ropeByPosition uses the global position. */
  int32_t kvSharded;
  int32_t shardStart;
  /* Per-sequence caches: device arrays [batch] of device pointers, each to one sequence's
   * [cacheRows, kvHeads*headDim] cache — separately allocated caches, as the reference's
   * per-sequence, per-layer K and V tensors are (transcriber.ts:111-118) — instead of the
   * slab (kCache / vCache / cacheSeqStride are then ignored).  Each cache must start on a
   * 16-byte boundary; one that does not makes its sequence come out as zeros and rt_sync
   * report it. */
  const void* const* kCachePtrs;
  const void* const* vCachePtrs;
  const rt_decode_second* second; /* host pointer or NULL: a second attention, same launch */
} rt_decode_args;

RT_API int rt_attn_decode(rt_ctx* ctx, const rt_decode_args* args);

/* rt_attn_decode for callers that may not allocate.  It has no counterpart in
 * the reference.  Who needs it: a host that fixed its device-memory budget
 * before the model started (a real-time transcription loop, an embedded
 * player), code running inside another framework's memory pool, or a caller
 * that holds the allocator lock — for them cudaMalloc is off limits, and
 * rt_attn_decode needs a context, which allocates a stream, a status word and
 * a split scratch that grows on demand.  This call takes no context and calls
 * no allocating routine: the split-KV scratch, the arrival counters and the
 * status word sit in one fixed device array inside the library (about 4 MiB,
 * held by every GPU that loads the library until the process exits).
 *
 * Same arguments and results as rt_attn_decode, enqueued on `cuda_stream` (a
 * cudaStream_t; NULL is the legacy default stream) of the CURRENT device.
 * Limits: batch*splits*qHeads*(2+headDim) <= 1,048,576 floats and
 * batch*headBlocks <= 4096 when more than one split is used (the library picks
 * the split count when args->splits is 0; pass splits = 1 to need no scratch at
 * all); larger requests are refused with RT_INVALID_ARGUMENT and a message
 * that names the two figures.  The first call on each device looks up the
 * array's device address; make that first call outside any stream capture.
 * All calls on a device share the one array, which keeps the previous call's
 * contents (the counters are cleared on the stream before each launch): two
 * calls whose kernels may overlap on the GPU — different streams, or the same
 * call from two threads — race on it, so serialise them.  Errors are reported
 * through the return code and rt_last_error(NULL); what a kernel finds wrong
 * while it runs (a bounded wait that ran out, a kvLens entry past cacheRows) is
 * recorded in the array's status word, which rt_attn_decode_noalloc_status
 * reads. */
RT_API int rt_attn_decode_noalloc(const rt_decode_args* args, void* cuda_stream);

/* What rt_sync is to rt_attn_decode, for the entry point above (it has no
 * counterpart in the reference either): waits for `cuda_stream`, reads the
 * status word of the current device's fixed array and, if a kernel recorded a
 * failure there, clears the word and returns RT_EXECUTION_FAILED with the
 * reason in rt_last_error(NULL).  Allocates nothing. */
RT_API int rt_attn_decode_noalloc_status(void* cuda_stream);

/* ---- set-up of the exchange without a launcher or a collective library --------
 * Allocates this rank's block (exchange buffer, control words, staging rows; all
 * zero) on `device` and maps the other ranks' blocks, so that a host with no
 * torch.distributed / NCCL — the TypeScript host of this library — can run the
 * KV-sequence-sharded decode.  One process per GPU: rt_xmem_export gives a
 * RT_XMEM_HANDLE_BYTES handle (a CUDA IPC handle) to send to the other processes
 * by any channel, rt_xmem_import maps a received one.  One process owning several
 * devices: rt_xmem_attach takes the peer's rt_xmem directly (peer access between
 * the two devices is enabled).  rt_xmem_exchange fills the rt_exchange once every
 * rank is mapped.  No counterpart in the reference, which has no multi-device code. */
typedef struct rt_xmem rt_xmem;
#define RT_XMEM_HANDLE_BYTES 64
RT_API int rt_xmem_create(int device, int32_t world, int32_t rank, int32_t batch, int32_t qHeads,
                          int32_t headDim, rt_xmem** out);
RT_API int rt_xmem_export(rt_xmem* m, void* handle);
RT_API int rt_xmem_import(rt_xmem* m, int32_t peer, const void* handle);
RT_API int rt_xmem_attach(rt_xmem* m, int32_t peer, rt_xmem* other);
RT_API int rt_xmem_exchange(rt_xmem* m, rt_exchange* out);
RT_API int rt_xmem_destroy(rt_xmem* m);

/* Merges `parts` sets of partials (m, l, acc) — the algebra of attnDecodeMerge
 * (packages/runntime/src/core/kernels/attention/attnDecode.ts:405-422) lifted
 * across devices.  partials: f32 [parts, units, 2+headDim]; out:
 * [units, headDim] in `dtype`.  An empty shard contributes (-1e30, 0, 0...). */
RT_API int rt_attn_merge_partials(rt_ctx* ctx, const float* partials, int32_t parts, int64_t units,
                           int32_t headDim, void* out, int32_t dtype);

/* ---- rope: the rotary embedding applied to q and k just before attention ------
 * out [rows, width] = interleaved-pair rotation of columns [srcStart,
 * srcStart+width) of x [rows, cols] by the pair-duplicated f32 tables cos, sin
 * [rows, headDim] (any scale pre-folded): (x0, x1) -> (x0 c - x1 s, x1 c + x0 s).
 * Replaces the 'rope' op and kernel (packages/runntime/src/core/graph/ops/
 * attention.ts:214-252; packages/runntime/src/core/kernels/attention/rope.ts:36-112). */
RT_API int rt_rope(rt_ctx* ctx, const void* x, const float* cosT, const float* sinT, void* out,
                   int64_t rows, int64_t cols, int32_t headDim, int64_t srcStart, int64_t width,
                   int32_t dtype);

/* ---- matmul: the projections either side of attention ---------------------------
 * out [m, n] = act(a [m, k] * B + bias [n]) + addend [m, n], B = rows
 * [baseRow, baseRow+k) of b [bRows, n] (a view into a taller fused weight; baseRow 0
 * and bRows = k for a plain weight).  bias and addend may be NULL.  activation:
 * 0 none, 1 tanh, 2 gelu, 3 silu, 4 relu, 5 geluTanh, 6 elu
 * (packages/runntime/src/core/kernels/activations.ts:6-14), applied before the
 * addend.  All tensors in `dtype`, f32 accumulation.  Replaces the 'matmul' op for
 * plain f32/f16 weights: the fused qkv / q / kv projections and o_proj with its
 * residual addend (packages/runntime/src/core/graph/ops/matmul.ts:28-99;
 * packages/runntime/src/core/nn/layers.ts:252-263).  Quantized weights are not
 * covered. */
RT_API int rt_matmul(rt_ctx* ctx, const void* a, const void* b, const void* bias,
                     const void* addend, void* out, int64_t m, int64_t k, int64_t n, int64_t bRows,
                     int64_t baseRow, int32_t activation, int32_t dtype);

/* ---- argmaxDot: fused gemv + argmax, the greedy decoding head ---------------------
 * out[0] (f32) = the row index v of w [rows, cols] with the largest w[v] . x
 * (x one row of `cols`), the lowest index on ties; the logits are never written
 * (packages/runntime/src/core/graph/ops/matmul.ts:316-333). */
RT_API int rt_argmax_dot(rt_ctx* ctx, const void* w, const void* x, float* out, int64_t rows,
                         int64_t cols, int32_t dtype);

/* ---- localAttention: short causal window with soft-capped, biased scores -------
 * qkv [rows, 3*heads*headDim] (columns q|k|v); row t of each head sees keys
 * t-window+1 .. t (window <= 32).  The score of the key j rows back is
 * softcap * tanh(sum_d (q_d qScale_d) (k_d kScale + rel[j][h*headDim+d]) / softcap);
 * rel f32 [window, heads*headDim], qScale f32 [headDim]; softmax over the keys,
 * weighted sum of the values; out [rows, heads*headDim] in `dtype`.  headDim is
 * a multiple of 4.  Replaces the 'localAttention' op and attnLocal kernel
 * (packages/runntime/src/core/graph/ops/attention.ts:255-300;
 * packages/runntime/src/core/kernels/attention/attnLocal.ts:58-123). */
RT_API int rt_local_attention(rt_ctx* ctx, const void* qkv, const float* rel, const float* qScale,
                              void* out, int64_t rows, int32_t heads, int32_t headDim,
                              int32_t window, float kScale, float softcap, int32_t dtype);

/* ---- softmax: row-wise over the last dim, optionally masked ---------------------
 * out [rows, cols] = softmax of each row of x.  With `segments` (f32 [rows, 2],
 * a [start, end) key range per row) x is square attention scores: row r keeps
 * keys j with start <= j < end and r - windowLeft <= j <= r + windowRight
 * (RT_WINDOW_INF = unbounded); the rest come out 0, and a row that keeps nothing
 * is all 0.  Replaces the 'softmax' op of the matmul-attention path
 * (packages/runntime/src/core/graph/ops/reduce.ts:12-39; kernel
 * packages/runntime/src/core/kernels/reduce/softmax.ts:111-186). */
RT_API int rt_softmax(rt_ctx* ctx, const void* x, void* out, const float* segments, int64_t rows,
                      int64_t cols, int32_t windowLeft, int32_t windowRight, int32_t dtype);

/* ---- slice: a row or column block of a 2-D tensor as its own tensor ------------
 * out [rowEnd-rowStart, colEnd-colStart] = x[rowStart:rowEnd, colStart:colEnd] of
 * x [rows, cols].  Replaces the 'sliceRows' / 'sliceCols' ops that cut v out of
 * the fused qkv row and k | v out of the fused cross projection
 * (packages/runntime/src/core/graph/ops/shape.ts:69-135; decoder.ts:55,72,93-97). */
RT_API int rt_slice(rt_ctx* ctx, const void* x, void* out, int64_t rows, int64_t cols,
                    int64_t rowStart, int64_t rowEnd, int64_t colStart, int64_t colEnd,
                    int32_t dtype);

/* ---- writeRows: the KV-cache append as its own op ----------------------------
 * dst rows [startRow, startRow+rows) = src (packages/runntime/src/core/graph/
 * ops/shape.ts:236-259; kernel packages/runntime/src/core/kernels/shape/
 * rows.ts:143-162).  dst is caller-owned and never freed by the library. */
RT_API int rt_kv_append(rt_ctx* ctx, void* dst, const void* src, int64_t startRow, int64_t rows,
                 int64_t cols, int64_t dstRows, int32_t dtype);

#ifdef __cplusplus
}
#endif
#endif /* RT_ATTN_H */
