// General prefill attention on the FP32 pipes: every option of the 'attn' op,
// f32 or f16 storage, any head size up to 512.  It is the kernel for fp32
// inputs (tensor cores would not hold the 1e-4 tolerance in one pass) and for
// shapes the tensor-core kernel does not take.
//
// A CTA owns 16 query rows of one query head and walks the key tiles of the
// union of its rows' bands.  K and V tiles of 32 keys are staged in shared
// memory as f32; each warp owns 4 rows: lane j scores key j of the tile for
// the 4 rows, the online softmax reduces across the warp, then lane x
// accumulates output columns x, x+32, ... with the probabilities broadcast by
// shuffles.  Replaces the reference's prefill routes
// (packages/runntime/src/core/kernels/attention/attn.ts:105-199,327-649 and
// attnFlash.ts:93-276) with one kernel; math and masking rules are theirs.
#include "common.cuh"

namespace rt {
namespace {

constexpr int BQ = 16;      // query rows per CTA
constexpr int BK = 32;      // keys per tile (one per lane)
constexpr int WARPS = 4;
constexpr int RPW = BQ / WARPS;  // rows per warp

template <typename T, int NC>  // NC = ceil(hd / 32) output columns per lane
__global__ void __launch_bounds__(WARPS * 32)
prefill_simt_kernel(const AttnParams p) {
  extern __shared__ __align__(16) float smem[];
  const int hd = p.hd;
  const int ks = hd | 1;          // odd row stride: lanes read distinct banks
  const int vs = NC * 32;         // V rows padded to whole lanes, pad = 0
  float* sQ = smem;               // [hd][BQ], transposed so 4 rows load as one float4
  float* sK = sQ + hd * BQ;       // [BK][ks]
  float* sV = sK + BK * ks;       // [BK][vs]
  __shared__ int64_t sLo[BQ], sEnd[BQ];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t row0 = (int64_t)blockIdx.x * BQ;
  const int h = blockIdx.y;
  const int kvh = h / (p.qHeads / p.kvHeads);
  const T* __restrict__ q = static_cast<const T*>(p.q);
  const T* __restrict__ k = static_cast<const T*>(p.k) + (int64_t)kvh * hd;
  const T* __restrict__ v = static_cast<const T*>(p.v) + (int64_t)kvh * hd;

  if (tid < BQ) {
    int64_t lo = 1, end = 0;
    if (row0 + tid < p.qLen) row_band(p, row0 + tid, lo, end);
    sLo[tid] = lo;
    sEnd[tid] = end;
  }
  for (int idx = tid; idx < BQ * hd; idx += WARPS * 32) {
    const int r = idx / hd, x = idx - r * hd;
    const int64_t row = row0 + r;
    sQ[x * BQ + r] = row < p.qLen ? to_f32<T>(q[row * p.qStride + (int64_t)h * hd + x]) : 0.f;
  }
  // V pad columns stay zero for the whole kernel.
  if (vs != hd) {
    for (int idx = tid; idx < BK * (vs - hd); idx += WARPS * 32) {
      const int jj = idx / (vs - hd), x = hd + idx % (vs - hd);
      sV[jj * vs + x] = 0.f;
    }
  }
  __syncthreads();

  int64_t tileLo = INT64_MAX, tileEnd = -1;
#pragma unroll
  for (int r = 0; r < BQ; r++) {
    if (sLo[r] <= sEnd[r]) {
      tileLo = sLo[r] < tileLo ? sLo[r] : tileLo;
      tileEnd = sEnd[r] > tileEnd ? sEnd[r] : tileEnd;
    }
  }
  int64_t lo[RPW], end[RPW];
  float m[RPW], l[RPW], acc[RPW][NC];
#pragma unroll
  for (int r = 0; r < RPW; r++) {
    lo[r] = sLo[warp * RPW + r];
    end[r] = sEnd[warp * RPW + r];
    m[r] = kNegSeed;
    l[r] = 0.f;
    if (p.sinks) {
      m[r] = p.sinks[h] * 0.6931471805599453f;
      l[r] = 1.f;
    }
#pragma unroll
    for (int c = 0; c < NC; c++) acc[r][c] = 0.f;
  }

  for (int64_t k0 = tileLo; k0 <= tileEnd; k0 += BK) {
    const int nk = (int)((tileEnd - k0 + 1) < BK ? (tileEnd - k0 + 1) : BK);
    __syncthreads();  // previous tile fully consumed
    for (int idx = tid; idx < BK * hd; idx += WARPS * 32) {
      const int jj = idx / hd, x = idx - jj * hd;
      float kv = 0.f, vv = 0.f;
      if (jj < nk) {
        const int64_t off = (k0 + jj) * p.kvStride + x;
        kv = to_f32<T>(k[off]);
        vv = to_f32<T>(v[off]);
      }
      sK[jj * ks + x] = kv;
      sV[jj * vs + x] = vv;
    }
    __syncthreads();

    // Does any of this warp's rows see any key of the tile?
    bool warpLive = false;
#pragma unroll
    for (int r = 0; r < RPW; r++) warpLive |= (lo[r] <= k0 + nk - 1) && (end[r] >= k0);
    if (!warpLive) continue;

    float s[RPW];
#pragma unroll
    for (int r = 0; r < RPW; r++) s[r] = 0.f;
    const float* kr = sK + lane * ks;
    const float4* q4 = reinterpret_cast<const float4*>(sQ) + warp;
    for (int x = 0; x < hd; x++) {
      const float kx = kr[x];
      const float4 qq = q4[x * (BQ / 4)];
      s[0] = fmaf(qq.x, kx, s[0]);
      s[1] = fmaf(qq.y, kx, s[1]);
      s[2] = fmaf(qq.z, kx, s[2]);
      s[3] = fmaf(qq.w, kx, s[3]);
    }
    const int64_t j = k0 + lane;
    const float bias = (p.hasKeyBias && j >= p.biasStart && j < p.biasEnd) ? p.biasValue : 0.f;
    float pr[RPW];
#pragma unroll
    for (int r = 0; r < RPW; r++) {
      const bool vis = j >= lo[r] && j <= end[r];
      const float sc = vis ? s[r] + bias : -INFINITY;
      const float mNew = fmaxf(m[r], warp_max(sc));
      const float corr = __expf(m[r] - mNew);
      const float pe = vis ? __expf(sc - mNew) : 0.f;
      l[r] = l[r] * corr + warp_sum(pe);
      m[r] = mNew;
      pr[r] = pe;
#pragma unroll
      for (int c = 0; c < NC; c++) acc[r][c] *= corr;
    }
    for (int jj = 0; jj < nk; jj++) {
      float pj[RPW];
#pragma unroll
      for (int r = 0; r < RPW; r++) pj[r] = __shfl_sync(0xffffffffu, pr[r], jj);
#pragma unroll
      for (int c = 0; c < NC; c++) {
        const float vv = sV[jj * vs + lane + 32 * c];
#pragma unroll
        for (int r = 0; r < RPW; r++) acc[r][c] = fmaf(pj[r], vv, acc[r][c]);
      }
    }
  }

  T* __restrict__ out = static_cast<T*>(p.out);
  const int64_t qw = (int64_t)p.qHeads * hd;
#pragma unroll
  for (int r = 0; r < RPW; r++) {
    const int64_t row = row0 + warp * RPW + r;
    if (row >= p.qLen) continue;
    const float invL = l[r] > 0.f ? 1.f / l[r] : 0.f;  // empty band -> zeros
#pragma unroll
    for (int c = 0; c < NC; c++) {
      const int x = lane + 32 * c;
      if (x < hd) out[row * qw + (int64_t)h * hd + x] = from_f32<T>(acc[r][c] * invL);
    }
  }
}

template <typename T, int NC>
cudaError_t launch(const AttnParams& p, cudaStream_t s) {
  const int hd = p.hd;
  const size_t smem = sizeof(float) * ((size_t)hd * BQ + (size_t)BK * (hd | 1) + (size_t)BK * NC * 32);
  auto kern = prefill_simt_kernel<T, NC>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  const int64_t tiles = (p.qLen + BQ - 1) / BQ;
  dim3 grid((unsigned)tiles, (unsigned)p.qHeads);
  kern<<<grid, WARPS * 32, smem, s>>>(p);
  return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch_nc(const AttnParams& p, cudaStream_t s) {
  const int nc = (p.hd + 31) / 32;
  if (nc <= 1) return launch<T, 1>(p, s);
  if (nc <= 2) return launch<T, 2>(p, s);
  if (nc <= 4) return launch<T, 4>(p, s);
  if (nc <= 8) return launch<T, 8>(p, s);
  return launch<T, 16>(p, s);
}

}  // namespace

cudaError_t launch_prefill_simt(const AttnParams& p, int dtype, cudaStream_t s) {
  return dtype == RT_F16 ? dispatch_nc<__half>(p, s) : dispatch_nc<float>(p, s);
}

}  // namespace rt
