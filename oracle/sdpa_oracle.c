/* CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA kernels are compared against.  It is used
 * by the tests, by the smoke check and by the CPU-baseline leg of the
 * benchmark; the product library never links, loads or calls it.
 *
 * It restates, from the formulas, what the reference computes:
 *   - oracle_sdpa_f64:  softmax(q.k^T) v per (query row, head) in f64 with a
 *     two-pass softmax over the keys the window and the row's segment leave
 *     visible.  Semantics follow the reference's own test oracle
 *     packages/runntime/test/core/kernels/attention/checkSdpa.ts:58-108:
 *     no score scale, sink adds exp(sink*ln2) to the denominator only, the key
 *     bias adds its value to keys [start,end), a row that sees no key is 0,
 *     GQA maps head h to kv head h / (qHeads/kvHeads).
 *   - oracle_sdpa_rows_f32 / _f16: the shader's operation order — one serial
 *     online softmax per (row, head) in f32, f16 storage widened on load and
 *     rounded once at the store — following
 *     packages/runntime/src/core/kernels/attention/attn.ts:105-199.  OpenMP
 *     over (row, head); this is the timed CPU baseline.
 *   - oracle_write_rows: dst[startRow*cols + i] = src[i]
 *     (packages/runntime/src/core/kernels/shape/rows.ts:143-162).
 *   - oracle_merge_partials: (m, l, acc) merge algebra of
 *     packages/runntime/src/core/kernels/attention/attnDecode.ts:405-422.
 *   - oracle_rope_f64: the rotary embedding that precedes attention in a decoder
 *     layer (packages/runntime/src/core/kernels/attention/rope.ts:36-70).
 *   - oracle_local_attention_f64: the short-window soft-capped attention of
 *     packages/runntime/src/core/kernels/attention/attnLocal.ts:58-123.
 *   - oracle_softmax_f64: the (optionally masked) row softmax of the
 *     matmul-attention path (packages/runntime/src/core/kernels/reduce/softmax.ts:111-186).
 *   - oracle_random_f32 / oracle_round_f16: the reference tests' input
 *     generator (packages/runntime/test/gpu.ts:114-130).
 *
 * Parity pin: the reference stores no golden vectors for attention and its
 * TypeScript oracle cannot execute where this is built (no Node).  The oracle
 * is pinned against analytic known-answer cases and against an independently
 * written numpy f64 restatement whose outputs are committed as fixtures; with
 * respect to outputs of the reference itself, parity is unpinned.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define WINDOW_INF 0x3fffffff

typedef struct {
  int64_t qLen, kvLen;
  int32_t qHeads, kvHeads, headDim;
  int64_t windowLeft, windowRight; /* WINDOW_INF = unbounded */
  int64_t qPosOffset;
  int32_t packed;     /* 1: q,k,v are column blocks of one [T,(qH+2kvH)*hd] tensor */
  int32_t hasKeyBias;
  int64_t biasStart, biasEnd;
  double biasValue;
} oracle_dims;

static void strides(const oracle_dims* c, int64_t* qs, int64_t* kvs, int64_t* kOff,
                    int64_t* vOff) {
  int64_t qw = (int64_t)c->qHeads * c->headDim, kvw = (int64_t)c->kvHeads * c->headDim;
  if (c->packed) {
    *qs = qw + 2 * kvw; *kvs = *qs; *kOff = qw; *vOff = qw + kvw;
  } else {
    *qs = qw; *kvs = kvw; *kOff = 0; *vOff = 0;
  }
}

/* Visible key range [lo, end] (inclusive) of query row i. */
static void band(const oracle_dims* c, const float* segs, int64_t i, int64_t* lo, int64_t* end) {
  int64_t qPos = c->qPosOffset + i;
  int64_t l = qPos - c->windowLeft; if (l < 0) l = 0;
  int64_t e = qPos + c->windowRight; if (e > c->kvLen - 1) e = c->kvLen - 1;
  if (segs) {
    int64_t s0 = (int64_t)segs[2 * i], s1 = (int64_t)segs[2 * i + 1] - 1;
    if (s0 > l) l = s0;
    if (s1 < e) e = s1;
  }
  *lo = l; *end = e;
}

/* f64 two-pass softmax; q,k,v are f32 arrays (already f16-rounded when the
 * kernel under test stores f16).  With packed=1, q, k and v all point at the
 * packed tensor.  out is [qLen, qHeads*headDim] f64. */
void oracle_sdpa_f64(const float* q, const float* k, const float* v, const float* sinks,
                     const float* segs, const oracle_dims* c, double* out) {
  int64_t qs, kvs, kOff, vOff;
  strides(c, &qs, &kvs, &kOff, &vOff);
  const int hd = c->headDim, group = c->qHeads / c->kvHeads;
  const int64_t qw = (int64_t)c->qHeads * hd;
#pragma omp parallel
  {
    double* sc = (double*)malloc(sizeof(double) * (size_t)(c->kvLen > 0 ? c->kvLen : 1));
#pragma omp for collapse(2) schedule(dynamic, 16)
    for (int64_t i = 0; i < c->qLen; i++) {
      for (int h = 0; h < c->qHeads; h++) {
        int64_t lo, end;
        band(c, segs, i, &lo, &end);
        const int kvh = h / group;
        double* o = out + i * qw + (int64_t)h * hd;
        for (int x = 0; x < hd; x++) o[x] = 0.0;
        double mx = sinks ? (double)sinks[h] * M_LN2 : -INFINITY;
        const float* qr = q + i * qs + (int64_t)h * hd;
        for (int64_t j = lo; j <= end; j++) {
          const float* kr = k + j * kvs + kOff + (int64_t)kvh * hd;
          double s = 0.0;
          for (int x = 0; x < hd; x++) s += (double)qr[x] * (double)kr[x];
          if (c->hasKeyBias && j >= c->biasStart && j < c->biasEnd) s += c->biasValue;
          sc[j - lo] = s;
          if (s > mx) mx = s;
        }
        if (mx == -INFINITY) continue;
        double sum = sinks ? exp((double)sinks[h] * M_LN2 - mx) : 0.0;
        for (int64_t j = lo; j <= end; j++) {
          double p = exp(sc[j - lo] - mx);
          sc[j - lo] = p;
          sum += p;
        }
        /* A row whose band is empty but has a sink: numerator is 0 -> zeros. */
        for (int64_t j = lo; j <= end; j++) {
          const float* vr = v + j * kvs + vOff + (int64_t)kvh * hd;
          const double p = sc[j - lo];
          for (int x = 0; x < hd; x++) o[x] += p * (double)vr[x];
        }
        for (int x = 0; x < hd; x++) o[x] /= sum;
      }
    }
    free(sc);
  }
}

/* ---- shader-order f32 online softmax (the timed CPU baseline) ------------ */

#define ROWS_BODY(LOADQ, LOADK, LOADV, STORE)                                              \
  int64_t qs, kvs, kOff, vOff;                                                             \
  strides(c, &qs, &kvs, &kOff, &vOff);                                                     \
  const int hd = c->headDim, group = c->qHeads / c->kvHeads;                               \
  const int64_t qw = (int64_t)c->qHeads * hd;                                              \
  _Pragma("omp parallel") {                                                                \
    float* acc = (float*)malloc(sizeof(float) * (size_t)hd * 2);                           \
    float* qf = acc + hd;                                                                  \
    _Pragma("omp for collapse(2) schedule(dynamic, 16)")                                   \
    for (int64_t i = 0; i < c->qLen; i++) {                                                \
      for (int h = 0; h < c->qHeads; h++) {                                                \
        int64_t lo, end;                                                                   \
        band(c, segs, i, &lo, &end);                                                       \
        const int kvh = h / group;                                                         \
        for (int x = 0; x < hd; x++) { acc[x] = 0.f; qf[x] = LOADQ(i * qs + (int64_t)h * hd + x); } \
        float m = -1e30f, l = 0.f;                                                         \
        if (sinks) { m = sinks[h] * (float)M_LN2; l = 1.f; }                               \
        for (int64_t j = lo; j <= end; j++) {                                              \
          const int64_t kb = j * kvs + kOff + (int64_t)kvh * hd;                           \
          float s = 0.f;                                                                   \
          for (int x = 0; x < hd; x++) s += qf[x] * LOADK(kb + x);                         \
          if (c->hasKeyBias && j >= c->biasStart && j < c->biasEnd) s += (float)c->biasValue; \
          const float mNew = s > m ? s : m;                                                \
          const float corr = expf(m - mNew), p = expf(s - mNew);                           \
          l = l * corr + p; m = mNew;                                                      \
          const int64_t vb = j * kvs + vOff + (int64_t)kvh * hd;                           \
          for (int x = 0; x < hd; x++) acc[x] = acc[x] * corr + LOADV(vb + x) * p;         \
        }                                                                                  \
        const float invL = l > 0.f ? 1.f / l : 0.f;                                        \
        for (int x = 0; x < hd; x++) STORE(i * qw + (int64_t)h * hd + x, acc[x] * invL);   \
      }                                                                                    \
    }                                                                                      \
    free(acc);                                                                             \
  }

void oracle_sdpa_rows_f32(const float* q, const float* k, const float* v, const float* sinks,
                          const float* segs, const oracle_dims* c, float* out) {
#define LQ(i) q[i]
#define LK(i) k[i]
#define LV(i) v[i]
#define ST(i, x) out[i] = (x)
  ROWS_BODY(LQ, LK, LV, ST)
#undef LQ
#undef LK
#undef LV
#undef ST
}

void oracle_sdpa_rows_f16(const _Float16* q, const _Float16* k, const _Float16* v,
                          const float* sinks, const float* segs, const oracle_dims* c,
                          _Float16* out) {
#define LQ(i) (float)q[i]
#define LK(i) (float)k[i]
#define LV(i) (float)v[i]
#define ST(i, x) out[i] = (_Float16)(x)
  ROWS_BODY(LQ, LK, LV, ST)
#undef LQ
#undef LK
#undef LV
#undef ST
}

/* ---- KV-cache append ------------------------------------------------------ */

void oracle_write_rows(void* dst, const void* src, int64_t startRow, int64_t rows, int64_t cols,
                       int32_t elemBytes) {
  memcpy((char*)dst + (size_t)startRow * cols * elemBytes, src, (size_t)rows * cols * elemBytes);
}

/* ---- rotary embedding ------------------------------------------------------ */

/* Interleaved-pair rotation of columns [srcStart, srcStart+width) of x
 * [rows, cols] by pair-duplicated f32 tables cos/sin [rows, headDim]; f64.
 * Semantics: packages/runntime/test/core/kernels/attention/rope.gpu.test.ts:27-49
 * (kernel: packages/runntime/src/core/kernels/attention/rope.ts:36-70). */
void oracle_rope_f64(const float* x, const float* cosT, const float* sinT, int64_t rows,
                     int64_t cols, int32_t headDim, int64_t srcStart, int64_t width,
                     double* out) {
  for (int64_t t = 0; t < rows; t++) {
    for (int64_t col = 0; col < width; col += 2) {
      const double c = cosT[t * headDim + (col % headDim)];
      const double s = sinT[t * headDim + (col % headDim)];
      const double x0 = x[t * cols + srcStart + col], x1 = x[t * cols + srcStart + col + 1];
      out[t * width + col] = x0 * c - x1 * s;
      out[t * width + col + 1] = x1 * c + x0 * s;
    }
  }
}

/* ---- localAttention ---------------------------------------------------------- */

/* Local attention from its definition, in f64: row t of head h scores the key j
 * rows back as cap * tanh(sum_d q_d qScale_d (k_d kScale + rel[j][d]) / cap) for
 * j < min(window, t + 1), softmaxes the scores and sums the values.  Semantics:
 * packages/runntime/test/core/kernels/attention/attnLocal.gpu.test.ts:24-65. */
void oracle_local_attention_f64(const float* qkv, const float* rel, const float* qScale,
                                int64_t rows, int32_t heads, int32_t headDim, int32_t window,
                                double kScale, double softcap, double* out) {
  const int64_t width = (int64_t)heads * headDim;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < rows; t++) {
    double scores[64];
    const int n = (int)(window < t + 1 ? window : t + 1);
    for (int h = 0; h < heads; h++) {
      const float* q = qkv + t * 3 * width + (int64_t)h * headDim;
      double mx = -INFINITY;
      for (int j = 0; j < n; j++) {
        const float* k = qkv + (t - j) * 3 * width + width + (int64_t)h * headDim;
        double s = 0.0;
        for (int i = 0; i < headDim; i++) {
          const double key = (double)k[i] * kScale + (double)rel[j * width + h * headDim + i];
          s += (double)q[i] * (double)qScale[i] * key;
        }
        scores[j] = softcap * tanh(s / softcap);
        if (scores[j] > mx) mx = scores[j];
      }
      double sum = 0.0;
      for (int j = 0; j < n; j++) sum += exp(scores[j] - mx);
      for (int i = 0; i < headDim; i++) {
        double acc = 0.0;
        for (int j = 0; j < n; j++)
          acc += exp(scores[j] - mx) *
                 (double)qkv[(t - j) * 3 * width + 2 * width + (int64_t)h * headDim + i];
        out[t * width + (int64_t)h * headDim + i] = acc / sum;
      }
    }
  }
}

/* ---- softmax ---------------------------------------------------------------- */

/* Row-wise softmax from the definition, in f64; with segs ([rows, 2] f32) row r
 * keeps key j when segs[2r] <= j < segs[2r+1] and r - wl <= j <= r + wr, the rest
 * come out 0 and are left out of the max and the sum.  Semantics:
 * packages/runntime/test/core/kernels/reduce/softmax.gpu.test.ts:18-37,129-160. */
void oracle_softmax_f64(const float* x, const float* segs, int64_t rows, int64_t cols, int64_t wl,
                        int64_t wr, double* out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; r++) {
    int64_t lo = 0, hi = cols;
    if (segs) {
      lo = (int64_t)segs[2 * r];
      hi = (int64_t)segs[2 * r + 1];
      if (r - wl > lo) lo = r - wl;
      if (r + wr + 1 < hi) hi = r + wr + 1;
      if (hi > cols) hi = cols;
      if (lo < 0) lo = 0;
    }
    double mx = -INFINITY, sum = 0.0;
    for (int64_t j = lo; j < hi; j++)
      if (x[r * cols + j] > mx) mx = x[r * cols + j];
    for (int64_t j = lo; j < hi; j++) sum += exp((double)x[r * cols + j] - mx);
    for (int64_t j = 0; j < cols; j++)
      out[r * cols + j] = (j >= lo && j < hi) ? exp((double)x[r * cols + j] - mx) / sum : 0.0;
  }
}

/* ---- (m, l, acc) merge ---------------------------------------------------- */

/* partials: [parts][units][2+hd] f32 with (m, l, acc[hd]) where acc is the
 * un-normalised numerator relative to m; out: [units][hd] f64. */
void oracle_merge_partials(const float* partials, int32_t parts, int64_t units, int32_t hd,
                           double* out) {
  const int64_t stride = 2 + hd;
  for (int64_t u = 0; u < units; u++) {
    double M = -1e30;
    for (int p = 0; p < parts; p++) {
      double mp = partials[((int64_t)p * units + u) * stride];
      if (mp > M) M = mp;
    }
    double L = 0.0;
    for (int p = 0; p < parts; p++) {
      const float* r = partials + ((int64_t)p * units + u) * stride;
      L += (double)r[1] * exp((double)r[0] - M);
    }
    for (int x = 0; x < hd; x++) {
      double s = 0.0;
      for (int p = 0; p < parts; p++) {
        const float* r = partials + ((int64_t)p * units + u) * stride;
        s += (double)r[2 + x] * exp((double)r[0] - M);
      }
      out[u * hd + x] = L > 0.0 ? s / L : 0.0;
    }
  }
}

/* ---- input generator ------------------------------------------------------ */

/* 32-bit LCG, values s / 2^31 - 1 in [-1, 1). */
void oracle_random_f32(float* out, int64_t n, uint32_t seed) {
  uint32_t s = seed;
  for (int64_t i = 0; i < n; i++) {
    s = s * 1664525u + 1013904223u;
    out[i] = (float)((double)s / 2147483648.0 - 1.0);
  }
}

/* Round-to-nearest-even to f16 and back. */
void oracle_round_f16(float* x, int64_t n) {
  for (int64_t i = 0; i < n; i++) x[i] = (float)(_Float16)x[i];
}

int oracle_num_threads(void) {
  int n = 1;
#ifdef _OPENMP
#pragma omp parallel
  {
#pragma omp master
    n = omp_get_num_threads();
  }
#endif
  return n;
}

/* Number of host threads the parallel loops use from now on (a launcher may have set
 * OMP_NUM_THREADS=1 for its worker processes before this library was loaded). */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
