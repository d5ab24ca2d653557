// The C ABI: context, buffers, argument validation and kernel routing.
// Declarations and the reference interfaces they replace are in rt_attn.h.
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <string>
#include <vector>

#include <cmath>
#include "common.cuh"

struct rt_ctx {
  uint32_t magic;
  int device;
  int smCount;
  cudaStream_t own;
  cudaStream_t stream;
  float* scratch;
  size_t scratchBytes;
  unsigned* counters;
  size_t counterCount;
  int* statusDev;
  int64_t launches;
  int useTc;
  int waitPolls;   // polls of the cross-GPU merge's wait before it gives up
  std::string err;
};

namespace {

constexpr uint32_t kLive = 0x52544358u;  // 'RTCX'
// statusDev: the status word, then the two words of the persistent prefill kernel's work
// queue (units drawn, CTAs finished), zero between launches.
constexpr int kStatusWords = 3;
constexpr uint32_t kDead = 0x44454144u;  // 'DEAD'

thread_local std::string tlsError;

// Disposed contexts stay allocated (a few dozen bytes each) so that a late use
// of the handle is recognised instead of touching freed memory.
std::mutex gGraveyardMutex;
std::vector<rt_ctx*> gGraveyard;

int fail(rt_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx && ctx->magic == kLive) ctx->err = buf;
  tlsError = buf;
  return code;
}

int enter(rt_ctx* ctx) {
  if (!ctx) return fail(nullptr, RT_NOT_INITIALIZED, "no context: call rt_ctx_create first");
  if (ctx->magic == kDead) return fail(nullptr, RT_RESOURCE_DISPOSED, "context was destroyed");
  if (ctx->magic != kLive) return fail(nullptr, RT_INVALID_ARGUMENT, "not a context handle");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess)
    return fail(ctx, RT_EXECUTION_FAILED, "cudaSetDevice(%d): %s", ctx->device,
                cudaGetErrorString(e));
  return RT_OK;
}

#define RT_ENTER(ctx)                     \
  do {                                    \
    int _s = enter(ctx);                  \
    if (_s != RT_OK) return _s;           \
  } while (0)

#define RT_CUDA(ctx, call)                                                              \
  do {                                                                                  \
    cudaError_t _e = (call);                                                            \
    if (_e != cudaSuccess)                                                              \
      return fail(ctx, RT_EXECUTION_FAILED, "%s: %s", #call, cudaGetErrorString(_e));   \
  } while (0)

const char* dtype_name(int d) { return d == RT_F16 ? "f16" : "f32"; }
int elem_size(int d) { return d == RT_F16 ? 2 : 4; }

int ensure_scratch(rt_ctx* ctx, size_t bytes, size_t counters) {
  if (bytes > ctx->scratchBytes) {
    // The old block may still be read by enqueued work.
    RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->scratch) RT_CUDA(ctx, cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratchBytes = 0;
    size_t want = bytes + bytes / 2;
    RT_CUDA(ctx, cudaMalloc(&ctx->scratch, want));
    ctx->scratchBytes = want;
  }
  if (counters > ctx->counterCount) {
    RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->counters) RT_CUDA(ctx, cudaFree(ctx->counters));
    ctx->counters = nullptr;
    ctx->counterCount = 0;
    size_t want = counters * 2;
    RT_CUDA(ctx, cudaMalloc(&ctx->counters, want * sizeof(unsigned)));
    RT_CUDA(ctx, cudaMemsetAsync(ctx->counters, 0, want * sizeof(unsigned), ctx->stream));
    ctx->counterCount = want;
  }
  return RT_OK;
}

// Argument rules of the 'attn' op; messages follow
// packages/runntime/src/core/graph/ops/attention.ts:45-121,160-205.
int validate_attn(rt_ctx* ctx, const rt_attn_args* a) {
  const char* op = a->qkvPacked ? "sdpaPacked" : "sdpa";
  if (!a->q || !a->k || !a->v || !a->out)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: q, k, v and out must be device pointers", op);
  if (a->dtype != RT_F32 && a->dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: dtype %d is neither f32 nor f16", op, a->dtype);
  if (a->qLen < 1 || a->kvLen < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: empty tensor (qLen %lld, kvLen %lld)", op,
                (long long)a->qLen, (long long)a->kvLen);
  if (a->headDim < 1 || a->qHeads < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: qHeads %d and headDim %d must be positive", op,
                a->qHeads, a->headDim);
  if (a->kvHeads <= 0 || a->qHeads % a->kvHeads != 0)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: qHeads %d not divisible by kvHeads %d", op,
                a->qHeads, a->kvHeads);
  if (a->qHeads > 65535)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: qHeads %d exceeds 65535", op, a->qHeads);
  if (a->qkvPacked) {
    if (a->headDim > 128)
      return fail(ctx, RT_INVALID_ARGUMENT, "sdpaPacked: headDim %d exceeds the kernel's max (128)",
                  a->headDim);
    if (a->qLen == 1)
      return fail(ctx, RT_INVALID_ARGUMENT,
                  "sdpaPacked: qLen must be > 1 (decode has no packed route)");
    if (a->kvLen != a->qLen || a->k != a->q || a->v != a->q)
      return fail(ctx, RT_INVALID_ARGUMENT,
                  "sdpaPacked: q, k and v must be the one packed tensor and kvLen == qLen");
    if (a->hasKeyBias)
      return fail(ctx, RT_INVALID_ARGUMENT, "sdpaPacked: no key bias on the packed form");
  }
  const int maxHd = a->qLen == 1 ? 128 : 512;
  if (a->headDim > maxHd)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: headDim %d exceeds the kernel's max (%d)", op,
                a->headDim, maxHd);
  if (a->windowLeft < 0 || a->windowLeft > RT_WINDOW_INF)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "%s: windowLeft %d must be a non-negative integer or Infinity", op, a->windowLeft);
  if (a->windowRight < 0 || a->windowRight > RT_WINDOW_INF)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "%s: windowRight %d must be a non-negative integer or Infinity", op,
                a->windowRight);
  if (a->qPosOffset < 0)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: qPosOffset %lld must be a non-negative integer", op,
                (long long)a->qPosOffset);
  if (a->windowRight != RT_WINDOW_INF && a->qPosOffset + a->qLen > a->kvLen)
    return fail(ctx, RT_INVALID_ARGUMENT, "%s: qPosOffset+qLen %lld exceeds key rows kvLen %lld", op,
                (long long)(a->qPosOffset + a->qLen), (long long)a->kvLen);
  if (a->segments && a->qLen == 1)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "sdpa: segments need qLen > 1 (decode has no segment route)");
  if (a->maxSegment != 0) {
    if (!a->segments) return fail(ctx, RT_INVALID_ARGUMENT, "%s: maxSegment needs segments", op);
    if (a->maxSegment < 1)
      return fail(ctx, RT_INVALID_ARGUMENT, "%s: maxSegment %d must be a positive integer", op,
                  a->maxSegment);
  }
  if (a->hasKeyBias) {
    if (a->biasStart < 0 || a->biasStart > a->biasEnd || a->biasEnd > a->kvLen)
      return fail(ctx, RT_INVALID_ARGUMENT, "sdpa: keyBias keys [%d, %d) must lie within the %lld keys",
                  a->biasStart, a->biasEnd, (long long)a->kvLen);
    if (!(a->biasValue - a->biasValue == 0.f))
      return fail(ctx, RT_INVALID_ARGUMENT, "sdpa: keyBias value %f must be finite",
                  (double)a->biasValue);
    if (a->qLen == 1)
      return fail(ctx, RT_INVALID_ARGUMENT,
                  "sdpa: keyBias needs qLen > 1 (decode has no key bias route)");
  }
  if (a->seqStride != 0 || a->seqLens) {
    if (a->seqStride < 1 || !a->seqLens)
      return fail(ctx, RT_INVALID_ARGUMENT, "%s: seqStride and seqLens go together", op);
    if (a->segments)
      return fail(ctx, RT_INVALID_ARGUMENT, "%s: seqLens and segments are exclusive", op);
    if (a->kvLen != a->qLen || a->qLen % a->seqStride != 0)
      return fail(ctx, RT_INVALID_ARGUMENT,
                  "%s: the batched form needs qLen == kvLen == batch*seqStride", op);
  }
  return RT_OK;
}

rt::AttnParams to_params(const rt_attn_args* a) {
  rt::AttnParams p{};
  const int es = elem_size(a->dtype);
  const int64_t qw = (int64_t)a->qHeads * a->headDim, kvw = (int64_t)a->kvHeads * a->headDim;
  p.q = a->q;
  p.out = a->out;
  if (a->qkvPacked) {
    p.qStride = p.kvStride = qw + 2 * kvw;
    p.k = static_cast<const char*>(a->q) + qw * es;
    p.v = static_cast<const char*>(a->q) + (qw + kvw) * es;
  } else {
    p.qStride = qw;
    p.kvStride = kvw;
    p.k = a->k;
    p.v = a->v;
  }
  p.sinks = a->sinks;
  p.segs = a->segments;
  p.seqLens = a->seqLens;
  p.seqStride = a->seqStride;
  p.qLen = a->qLen;
  p.kvLen = a->kvLen;
  p.qPosOffset = a->qPosOffset;
  p.qHeads = a->qHeads;
  p.kvHeads = a->kvHeads;
  p.hd = a->headDim;
  p.wl = a->windowLeft;
  p.wr = a->windowRight;
  p.hasKeyBias = a->hasKeyBias;
  p.biasStart = a->biasStart;
  p.biasEnd = a->biasEnd;
  p.biasValue = a->biasValue;
  p.maxSegment = a->maxSegment;
  return p;
}

int run_decode(rt_ctx* ctx, rt::DecodeParams& p, int dtype) {
  std::string err;
  if (!rt::plan_decode(p, dtype, ctx->smCount, &err))
    return fail(ctx, RT_INVALID_ARGUMENT, "%s", err.c_str());
  const int zBlocks = (p.kvHeads + p.kvPerCta - 1) / p.kvPerCta;
  if (p.splits > 1) {
    const size_t sets = p.hasSecond ? 2 : 1;   // a second attention has its own partials and counters
    const size_t bytes = sets * p.batch * p.splits * p.qHeads * (2 + p.hd) * sizeof(float);
    int s = ensure_scratch(ctx, bytes, sets * p.batch * zBlocks);
    if (s != RT_OK) return s;
  }
  p.scratch = ctx->scratch;
  p.counters = ctx->counters;
  p.status = ctx->statusDev;
  RT_CUDA(ctx, rt::launch_decode(p, dtype, ctx->stream));
  ctx->launches++;
  return RT_OK;
}

}  // namespace

void rt::set_thread_error(const char* msg) { tlsError = msg; }

extern "C" {

int rt_ctx_create(int device, rt_ctx** out) {
  if (!out) return fail(nullptr, RT_INVALID_ARGUMENT, "rt_ctx_create: out is NULL");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(nullptr, RT_UNSUPPORTED_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
  if (device < 0 || device >= count)
    return fail(nullptr, RT_INVALID_ARGUMENT, "device %d out of range (%d devices)", device, count);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess)
    return fail(nullptr, RT_UNSUPPORTED_DEVICE, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return fail(nullptr, RT_UNSUPPORTED_DEVICE,
                "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                prop.minor);
  rt_ctx* ctx = new rt_ctx();
  ctx->magic = kLive;
  ctx->device = device;
  ctx->smCount = prop.multiProcessorCount;
  ctx->scratch = nullptr;
  ctx->scratchBytes = 0;
  ctx->counters = nullptr;
  ctx->counterCount = 0;
  ctx->launches = 0;
  ctx->useTc = 1;
  ctx->waitPolls = 1 << 20;   // about a second with the kernel's sleeps
  if ((e = cudaSetDevice(device)) != cudaSuccess ||
      (e = cudaStreamCreateWithFlags(&ctx->own, cudaStreamNonBlocking)) != cudaSuccess ||
      (e = cudaMalloc(&ctx->statusDev, kStatusWords * sizeof(int))) != cudaSuccess ||
      (e = cudaMemset(ctx->statusDev, 0, kStatusWords * sizeof(int))) != cudaSuccess) {
    delete ctx;
    return fail(nullptr, RT_EXECUTION_FAILED, "context setup: %s", cudaGetErrorString(e));
  }
  ctx->stream = ctx->own;
  *out = ctx;
  return RT_OK;
}

int rt_ctx_destroy(rt_ctx* ctx) {
  RT_ENTER(ctx);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->counters) cudaFree(ctx->counters);
  cudaFree(ctx->statusDev);
  cudaStreamDestroy(ctx->own);
  ctx->scratch = nullptr;
  ctx->counters = nullptr;
  ctx->statusDev = nullptr;
  ctx->magic = kDead;
  std::lock_guard<std::mutex> lock(gGraveyardMutex);
  gGraveyard.push_back(ctx);
  return RT_OK;
}

int rt_ctx_set_stream(rt_ctx* ctx, void* cuda_stream, int external) {
  RT_ENTER(ctx);
  ctx->stream = external ? static_cast<cudaStream_t>(cuda_stream) : ctx->own;
  return RT_OK;
}

int rt_ctx_set_option(rt_ctx* ctx, int option, int value) {
  RT_ENTER(ctx);
  if (option == RT_OPT_PREFILL_TC) {
    if (value < 0 || value > 6)
      return fail(ctx, RT_INVALID_ARGUMENT, "rt_ctx_set_option: RT_OPT_PREFILL_TC takes 0..6, got %d",
                  value);
    ctx->useTc = value;
    return RT_OK;
  }
  if (option == RT_OPT_WAIT_POLLS) {
    if (value < 1)
      return fail(ctx, RT_INVALID_ARGUMENT, "rt_ctx_set_option: RT_OPT_WAIT_POLLS takes a positive count, got %d",
                  value);
    ctx->waitPolls = value;
    return RT_OK;
  }
  return fail(ctx, RT_INVALID_ARGUMENT, "rt_ctx_set_option: unknown option %d", option);
}

const char* rt_last_error(const rt_ctx* ctx) {
  if (ctx && ctx->magic == kLive) return ctx->err.c_str();
  return tlsError.c_str();
}

int rt_sync(rt_ctx* ctx) {
  RT_ENTER(ctx);
  RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  int status = 0;
  RT_CUDA(ctx, cudaMemcpy(&status, ctx->statusDev, sizeof(int), cudaMemcpyDeviceToHost));
  if (status != 0) {
    // (with the status word, the work counter of the persistent prefill kernel, which a
    // block that gave up never rewound)
    cudaMemset(ctx->statusDev, 0, kStatusWords * sizeof(int));
    // A block that gave up never counted itself in: the arrival counters of the split
    // merge are no longer zero, and the next split launch would pick the wrong last block.
    if (ctx->counters) cudaMemset(ctx->counters, 0, ctx->counterCount * sizeof(unsigned));
    return fail(ctx, RT_EXECUTION_FAILED,
                "a kernel reported status 0x%x (%s)", status,
                (status & rt::kStatusWaitTimeout)
                    ? "a bounded device-side wait ran out"
                    : "a device-side length exceeds its buffer (kvLens entry past cacheRows) or a "
                      "per-sequence cache pointer is not 16-byte aligned");
  }
  return RT_OK;
}

int64_t rt_launch_count(const rt_ctx* ctx) {
  return (ctx && ctx->magic == kLive) ? ctx->launches : -1;
}

int rt_buf_alloc(rt_ctx* ctx, size_t bytes, void** device_ptr) {
  RT_ENTER(ctx);
  if (!device_ptr) return fail(ctx, RT_INVALID_ARGUMENT, "rt_buf_alloc: device_ptr is NULL");
  *device_ptr = nullptr;
  if (bytes == 0) return fail(ctx, RT_INVALID_ARGUMENT, "rt_buf_alloc: empty tensor (0 bytes)");
  RT_CUDA(ctx, cudaMalloc(device_ptr, bytes));
  return RT_OK;
}

int rt_buf_free(rt_ctx* ctx, void* device_ptr) {
  RT_ENTER(ctx);
  if (!device_ptr) return RT_OK;
  RT_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  RT_CUDA(ctx, cudaFree(device_ptr));
  return RT_OK;
}

int rt_buf_upload(rt_ctx* ctx, void* device_ptr, size_t offset, const void* host, size_t bytes) {
  RT_ENTER(ctx);
  if (!device_ptr || !host) return fail(ctx, RT_INVALID_ARGUMENT, "rt_buf_upload: NULL pointer");
  RT_CUDA(ctx, cudaMemcpyAsync(static_cast<char*>(device_ptr) + offset, host, bytes,
                               cudaMemcpyHostToDevice, ctx->stream));
  return RT_OK;
}

int rt_buf_download(rt_ctx* ctx, const void* device_ptr, size_t offset, void* host, size_t bytes) {
  RT_ENTER(ctx);
  if (!device_ptr || !host) return fail(ctx, RT_INVALID_ARGUMENT, "rt_buf_download: NULL pointer");
  RT_CUDA(ctx, cudaMemcpyAsync(host, static_cast<const char*>(device_ptr) + offset, bytes,
                               cudaMemcpyDeviceToHost, ctx->stream));
  return rt_sync(ctx);
}

// 0 = FP32-pipe kernel, 1 = tensor cores, one query tile per CTA, 2 = two tiles per CTA,
// 3 = one tile with two softmax warpgroups on alternate key tiles, 4 = the same in pairs of
// CTAs that share every K/V tile, 5 = the persistent form of 3 (one CTA per SM, units
// overlapping).
static int prefill_kernel_of(const rt_ctx* ctx, const rt::AttnParams& p, int dtype) {
  if (!ctx->useTc) return 0;
  const bool tc3 = rt::prefill_tc3_supported(p, dtype);
  if (ctx->useTc == 6 && rt::prefill_tc4_supported(p, dtype)) return 5;
  if (ctx->useTc == 5 && rt::prefill_tc3_pair_supported(p, dtype)) return 4;
  if ((ctx->useTc == 4 || ctx->useTc == 5) && tc3) return 3;
  if (!rt::prefill_tc_supported(p, dtype)) return (tc3 && ctx->useTc == 1) ? 3 : 0;  // heads narrower than 64
  if (ctx->useTc == 3 && rt::prefill_tc2_supported(p, dtype)) return 2;
  // The library's own choice: the alternating-warpgroup kernel (measured, a second of
  // back-to-back launches: the large causal prefill at head size 128, 914 TFLOP/s against 858
  // for two tiles per block and 770 for one tile with one softmax warpgroup; the sliding-window
  // GQA prefill at head size 256 over padded sequences, 584 against 545 for one tile — once a
  // unit past a sequence's end stopped costing it 9 us of 4-byte zero stores).
  if (ctx->useTc == 1 && tc3) return 3;
  return 1;
}

static const char* route_of(const rt_ctx* ctx, const rt_attn_args* a) {
  if (a->qLen == 1) return "decode";
  const int k = prefill_kernel_of(ctx, to_params(a), a->dtype);
  return k == 5 ? "prefill_tc4" : k == 4 ? "prefill_tc3_pair" : k == 3 ? "prefill_tc3" : k == 2 ? "prefill_tc2" : k == 1 ? "prefill_tc" : "prefill_simt";
}

int rt_attn_route(rt_ctx* ctx, const rt_attn_args* args, const char** route) {
  RT_ENTER(ctx);
  if (!args || !route) return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_route: NULL argument");
  int s = validate_attn(ctx, args);
  if (s != RT_OK) return s;
  *route = route_of(ctx, args);
  return RT_OK;
}

int rt_attn(rt_ctx* ctx, const rt_attn_args* a) {
  RT_ENTER(ctx);
  if (!a) return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn: args is NULL");
  int s = validate_attn(ctx, a);
  if (s != RT_OK) return s;
  if (a->qLen == 1) {
    rt::DecodeParams p{};
    p.q = a->q;
    p.out = a->out;
    p.kCache = const_cast<void*>(a->k);
    p.vCache = const_cast<void*>(a->v);
    p.sinks = a->sinks;
    p.useRange = 1;
    const int64_t qPos = a->qPosOffset;
    p.lo = qPos - a->windowLeft < 0 ? 0 : qPos - a->windowLeft;
    p.end = qPos + a->windowRight > a->kvLen - 1 ? a->kvLen - 1 : qPos + a->windowRight;
    p.batch = 1;
    p.kvLen = (int32_t)(a->kvLen > INT32_MAX ? INT32_MAX : a->kvLen);
    p.qHeads = a->qHeads;
    p.kvHeads = a->kvHeads;
    p.hd = a->headDim;
    p.wl = a->windowLeft;
    p.splits = 0;
    return run_decode(ctx, p, a->dtype);
  }
  const rt::AttnParams p = to_params(a);
  const int kernel = prefill_kernel_of(ctx, p, a->dtype);
  if (kernel != 0) {
    std::string err;
    cudaError_t e = kernel == 5   ? rt::launch_prefill_tc4(p, ctx->statusDev, ctx->statusDev + 1, ctx->smCount,
                                                           ctx->stream, &err)
                    : kernel >= 3 ? rt::launch_prefill_tc3(p, kernel == 4, ctx->statusDev, ctx->stream, &err)
                    : kernel == 2 ? rt::launch_prefill_tc2(p, ctx->statusDev, ctx->stream, &err)
                                  : rt::launch_prefill_tc(p, a->dtype, ctx->statusDev, ctx->stream, &err);
    if (e != cudaSuccess)
      return fail(ctx, RT_EXECUTION_FAILED, "prefill_tc launch: %s %s", cudaGetErrorString(e),
                  err.c_str());
  } else {
    RT_CUDA(ctx, rt::launch_prefill_simt(p, a->dtype, ctx->stream));
  }
  ctx->launches++;
  return RT_OK;
}

int rt_attn_decode(rt_ctx* ctx, const rt_decode_args* a) {
  RT_ENTER(ctx);
  if (!a) return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: args is NULL");
  if (!a->q || (!a->kCache && !a->kCachePtrs) || (!a->vCache && !a->vCachePtrs) ||
      (!a->out && !a->partialsOut))
    return fail(ctx, RT_INVALID_ARGUMENT,
                "rt_attn_decode: q, kCache, vCache and out (or partialsOut) must be device pointers");
  if (a->dtype != RT_F32 && a->dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: dtype %d is neither f32 nor f16", a->dtype);
  if (a->batch < 1 || a->cacheRows < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: empty tensor (batch %d, cacheRows %d)",
                a->batch, a->cacheRows);
  if (a->batch > 65535)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: batch %d exceeds 65535", a->batch);
  if (a->headDim < 1 || a->qHeads < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: qHeads %d and headDim %d must be positive",
                a->qHeads, a->headDim);
  if (a->kvHeads <= 0 || a->qHeads % a->kvHeads != 0)
    return fail(ctx, RT_INVALID_ARGUMENT, "sdpa: qHeads %d not divisible by kvHeads %d", a->qHeads,
                a->kvHeads);
  if (a->headDim > 128)
    return fail(ctx, RT_INVALID_ARGUMENT, "sdpa: headDim %d exceeds the kernel's max (128)",
                a->headDim);
  if (a->kvLen < 0 || (!a->kvSharded && a->kvLen > a->cacheRows))
    return fail(ctx, RT_INVALID_ARGUMENT,
                "writeRows: rows [%d, %d) exceed dst capacity %d", a->kvLen - 1, a->kvLen,
                a->cacheRows);
  if (!a->kvLens && a->kvLen < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: kvLen %d must be positive", a->kvLen);
  if ((a->kNew == nullptr) != (a->vNew == nullptr))
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: kNew and vNew go together");
  if (a->windowLeft < 0 || a->windowLeft > RT_WINDOW_INF)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "sdpa: windowLeft %d must be a non-negative integer or Infinity", a->windowLeft);
  if (a->splits < 0 || a->splits > 64)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: splits %d out of range [0, 64]",
                a->splits);
  if (a->cacheSeqStride < 0 ||
      (!a->kCachePtrs && a->batch > 1 &&
       a->cacheSeqStride < (int64_t)a->cacheRows * a->kvHeads * a->headDim))
    return fail(ctx, RT_INVALID_ARGUMENT,
                "rt_attn_decode: cacheSeqStride %lld is smaller than one cache",
                (long long)a->cacheSeqStride);
  if (const char* why = rt::decode_rope_args_error(*a))
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_decode: %s", why);
  rt::DecodeParams p{};
  rt::decode_params_from_args(*a, p);
  const int phases = a->exchange && a->exchange->phases ? a->exchange->phases : 3;
  if (phases & 1) {
    const int s = run_decode(ctx, p, a->dtype);
    if (s != RT_OK) return s;
  }
  if (!a->exchange || !(phases & 2)) return RT_OK;
  const rt_exchange& x = *a->exchange;
  const int per = rt::exchange_per(a->batch, x.world);
  const int first = rt::owner_first(x.rank, a->batch, x.world);
  const int owned = rt::owner_count(x.rank, a->batch, x.world);
  RT_CUDA(ctx, rt::launch_merge_exchanged(x.partials[x.rank], x.flags[x.rank], x.step, x.world, per,
                                          owned, first, a->qHeads, a->headDim, a->out, a->dtype,
                                          ctx->statusDev, ctx->waitPolls, ctx->stream));
  if (owned > 0) ctx->launches++;
  return RT_OK;
}

int rt_attn_merge_partials(rt_ctx* ctx, const float* partials, int32_t parts, int64_t units,
                           int32_t headDim, void* out, int32_t dtype) {
  RT_ENTER(ctx);
  if (!partials || !out)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_merge_partials: NULL pointer");
  if (parts < 1 || units < 1 || headDim < 1)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "rt_attn_merge_partials: empty tensor (parts %d, units %lld, headDim %d)", parts,
                (long long)units, headDim);
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "rt_attn_merge_partials: bad dtype %d", dtype);
  RT_CUDA(ctx, rt::launch_merge_partials(partials, parts, units, headDim, out, dtype, ctx->stream));
  ctx->launches++;
  return RT_OK;
}

int rt_rope(rt_ctx* ctx, const void* x, const float* cosT, const float* sinT, void* out,
            int64_t rows, int64_t cols, int32_t headDim, int64_t srcStart, int64_t width,
            int32_t dtype) {
  RT_ENTER(ctx);
  if (!x || !cosT || !sinT || !out) return fail(ctx, RT_INVALID_ARGUMENT, "rope: NULL pointer");
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "rope: bad dtype %d", dtype);
  if (rows < 1 || cols < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "rope: empty tensor (%lld x %lld)", (long long)rows,
                (long long)cols);
  if (headDim <= 0 || headDim % 2 != 0)
    return fail(ctx, RT_INVALID_ARGUMENT, "rope: headDim %d must be a positive even integer",
                headDim);
  if (srcStart < 0 || srcStart % 2 != 0)
    return fail(ctx, RT_INVALID_ARGUMENT, "rope: srcStart %lld must be a non-negative even integer",
                (long long)srcStart);
  if (width <= 0 || srcStart + width > cols)
    return fail(ctx, RT_INVALID_ARGUMENT, "rope: window [%lld, %lld) exceeds %lld input cols",
                (long long)srcStart, (long long)(srcStart + width), (long long)cols);
  if (width % headDim != 0)
    return fail(ctx, RT_INVALID_ARGUMENT, "rope: width %lld must be a multiple of headDim %d",
                (long long)width, headDim);
  RT_CUDA(ctx, rt::launch_rope(x, cosT, sinT, out, rows, cols, headDim, srcStart, width, dtype,
                               ctx->stream));
  ctx->launches++;
  return RT_OK;
}

int rt_matmul(rt_ctx* ctx, const void* a, const void* b, const void* bias, const void* addend,
              void* out, int64_t m, int64_t k, int64_t n, int64_t bRows, int64_t baseRow,
              int32_t activation, int32_t dtype) {
  RT_ENTER(ctx);
  if (!a || !b || !out) return fail(ctx, RT_INVALID_ARGUMENT, "matmul: NULL pointer");
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "matmul: both inputs must be f32 or both f16");
  if (m < 1 || k < 1 || n < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "matmul: empty tensor (a=[%lld,%lld] b=[%lld,%lld])",
                (long long)m, (long long)k, (long long)bRows, (long long)n);
  if (baseRow < 0 || baseRow + k > bRows)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "matmul: bad baseRow %lld — need integer >= 0 with baseRow+K (%lld) <= rows (%lld)",
                (long long)baseRow, (long long)k, (long long)bRows);
  if (activation < 0 || activation > 6)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "unknown activation code %d — valid codes are 0..6", activation);
  const char* bp = static_cast<const char*>(b) + baseRow * n * elem_size(dtype);
  if (ctx->useTc && rt::matmul_tc_supported(a, bp, out, m, k, n, dtype)) {
    std::string err;
    cudaError_t e = rt::launch_matmul_tc(a, bp, bias, addend, out, m, k, n, activation,
                                         ctx->statusDev, ctx->stream, &err);
    if (e != cudaSuccess)
      return fail(ctx, RT_EXECUTION_FAILED, "matmul_tc launch: %s %s", cudaGetErrorString(e),
                  err.c_str());
    ctx->launches++;
    return RT_OK;
  }
  const size_t need = rt::matmul_scratch_need(m, k, n, dtype);
  if (need) {
    const int s = ensure_scratch(ctx, need, 1);
    if (s != RT_OK) return s;
  }
  RT_CUDA(ctx, rt::launch_matmul(a, bp, bias, addend, out, m, k, n, activation, dtype,
                                 need ? ctx->scratch : nullptr, ctx->stream));
  ctx->launches += ((m > 8 && m <= 16) ? 2 : 1) + (need ? 1 : 0);
  return RT_OK;
}

int rt_argmax_dot(rt_ctx* ctx, const void* w, const void* x, float* out, int64_t rows, int64_t cols,
                  int32_t dtype) {
  RT_ENTER(ctx);
  if (!w || !x || !out) return fail(ctx, RT_INVALID_ARGUMENT, "argmaxDot: NULL pointer");
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "argmaxDot: bad dtype %d", dtype);
  if (rows < 1 || cols < 1 || rows > 0xffffffffll)
    return fail(ctx, RT_INVALID_ARGUMENT, "argmaxDot: empty or oversized tensor (%lld x %lld)",
                (long long)rows, (long long)cols);
  int s = ensure_scratch(ctx, 64, 1);
  if (s != RT_OK) return s;
  RT_CUDA(ctx, rt::launch_argmax_dot(w, x, out, rows, cols, dtype,
                                     reinterpret_cast<unsigned long long*>(ctx->scratch), ctx->stream));
  ctx->launches += 2;
  return RT_OK;
}

int rt_local_attention(rt_ctx* ctx, const void* qkv, const float* rel, const float* qScale,
                       void* out, int64_t rows, int32_t heads, int32_t headDim, int32_t window,
                       float kScale, float softcap, int32_t dtype) {
  RT_ENTER(ctx);
  if (!qkv || !rel || !qScale || !out)
    return fail(ctx, RT_INVALID_ARGUMENT, "localAttention: NULL pointer");
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "localAttention: bad dtype %d", dtype);
  if (rows < 1) return fail(ctx, RT_INVALID_ARGUMENT, "localAttention: empty tensor (%lld rows)",
                            (long long)rows);
  if (heads < 1 || headDim < 4 || headDim % 4 != 0)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "localAttention: heads %d must be a positive integer and headDim %d a multiple of 4",
                heads, headDim);
  if (window < 1 || window > 32)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "localAttention: window %d must be an integer from 1 to 32", window);
  if (!(softcap > 0.f) || !std::isfinite(kScale))
    return fail(ctx, RT_INVALID_ARGUMENT,
                "localAttention: softcap must be positive and kScale finite, got %g, %g",
                (double)softcap, (double)kScale);
  const uintptr_t word = 4 * (uintptr_t)elem_size(dtype);
  if (reinterpret_cast<uintptr_t>(qkv) % word || reinterpret_cast<uintptr_t>(out) % word ||
      reinterpret_cast<uintptr_t>(rel) % 16 || reinterpret_cast<uintptr_t>(qScale) % 16)
    return fail(ctx, RT_INVALID_ARGUMENT,
                "localAttention: tensors must start on a four-element boundary");
  RT_CUDA(ctx, rt::launch_local_attn(qkv, rel, qScale, out, rows, heads, headDim, window, kScale,
                                     softcap, dtype, ctx->stream));
  ctx->launches++;
  return RT_OK;
}

int rt_softmax(rt_ctx* ctx, const void* x, void* out, const float* segments, int64_t rows,
               int64_t cols, int32_t windowLeft, int32_t windowRight, int32_t dtype) {
  RT_ENTER(ctx);
  if (!x || !out) return fail(ctx, RT_INVALID_ARGUMENT, "softmax: NULL pointer");
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "softmax: bad dtype %d", dtype);
  if (rows < 1 || cols < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "softmax: empty tensor (%lld x %lld)", (long long)rows,
                (long long)cols);
  if (segments && rows != cols)
    return fail(ctx, RT_INVALID_ARGUMENT, "softmax: a masked softmax needs square scores, got [%lld, %lld]",
                (long long)rows, (long long)cols);
  if (segments && (windowLeft < 0 || windowRight < 0))
    return fail(ctx, RT_INVALID_ARGUMENT,
                "softmax: %s must be a non-negative integer or Infinity, got %d",
                windowLeft < 0 ? "windowLeft" : "windowRight",
                windowLeft < 0 ? windowLeft : windowRight);
  RT_CUDA(ctx, rt::launch_softmax(x, out, segments, rows, cols, windowLeft, windowRight, dtype,
                                  ctx->stream));
  ctx->launches++;
  return RT_OK;
}

int rt_slice(rt_ctx* ctx, const void* x, void* out, int64_t rows, int64_t cols, int64_t rowStart,
             int64_t rowEnd, int64_t colStart, int64_t colEnd, int32_t dtype) {
  RT_ENTER(ctx);
  if (!x || !out) return fail(ctx, RT_INVALID_ARGUMENT, "slice: NULL pointer");
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "slice: bad dtype %d", dtype);
  if (rows < 1 || cols < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "slice: empty tensor (%lld x %lld)", (long long)rows,
                (long long)cols);
  if (rowStart < 0 || rowEnd > rows || rowStart >= rowEnd)
    return fail(ctx, RT_INVALID_ARGUMENT, "slice: bad range [%lld, %lld) for %lld rows",
                (long long)rowStart, (long long)rowEnd, (long long)rows);
  if (colStart < 0 || colEnd > cols || colStart >= colEnd)
    return fail(ctx, RT_INVALID_ARGUMENT, "slice: bad range [%lld, %lld) for %lld cols",
                (long long)colStart, (long long)colEnd, (long long)cols);
  const int es = elem_size(dtype);
  RT_CUDA(ctx, rt::launch_slice(x, out, rowEnd - rowStart, cols * es,
                                (rowStart * cols + colStart) * es, (colEnd - colStart) * es,
                                ctx->stream));
  ctx->launches++;
  return RT_OK;
}

int rt_kv_append(rt_ctx* ctx, void* dst, const void* src, int64_t startRow, int64_t rows,
                 int64_t cols, int64_t dstRows, int32_t dtype) {
  RT_ENTER(ctx);
  if (!dst || !src) return fail(ctx, RT_INVALID_ARGUMENT, "writeRows: NULL pointer");
  if (dtype != RT_F32 && dtype != RT_F16)
    return fail(ctx, RT_INVALID_ARGUMENT, "writeRows: bad dtype %d", dtype);
  if (rows < 1 || cols < 1 || dstRows < 1)
    return fail(ctx, RT_INVALID_ARGUMENT, "writeRows: empty tensor (%lld x %lld into %lld rows)",
                (long long)rows, (long long)cols, (long long)dstRows);
  if (startRow < 0 || startRow + rows > dstRows)
    return fail(ctx, RT_INVALID_ARGUMENT, "writeRows: rows [%lld, %lld) exceed dst capacity %lld",
                (long long)startRow, (long long)(startRow + rows), (long long)dstRows);
  const int es = elem_size(dtype);
  (void)dtype_name;
  RT_CUDA(ctx, rt::launch_write_rows(dst, src, startRow * cols * es, rows * cols * es, ctx->stream));
  ctx->launches++;
  return RT_OK;
}

}  // extern "C"
