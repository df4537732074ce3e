// LayerNorm and RMSNorm, forward and backward, bf16 in/out with fp32 statistics.
// Optional fused residual add in forward: s = x + res is written back as the new residual stream
// and normalised in the same pass.
//
// Math follows the reference's CPU layers (reference: src/nn/layers.zig:60-81 RMSNorm forward,
// :101-135 RMSNorm backward, :180-206 LayerNorm forward, :228-271 LayerNorm backward; CUDA
// counterparts kernels/cuda/layernorm.cu:91-254, kernels/cuda/normalization.cu:27-120). The
// reference has no LayerNorm backward kernel and reduces weight gradients with atomics; here the
// weight/bias gradients are reduced in two deterministic passes through a [blocks, D] fp32
// scratch buffer supplied by the caller.
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

constexpr int NORM_MAX_VEC = 16;  // uint4 (8 x bf16) per thread held in registers

// TPR = threads per row (32: one warp per row; 256: one CTA per row).
template <int TPR, bool RMS, bool HAS_RES>
__global__ void __launch_bounds__(256) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                       const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                                                       __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out,
                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                                       int D, float eps) {
  constexpr int ROWS_PER_BLOCK = 256 / TPR;
  __shared__ float red[2][8];
  const int t = threadIdx.x % TPR;
  const int row = blockIdx.x * ROWS_PER_BLOCK + threadIdx.x / TPR;
  if (TPR == 32 && row >= rows) return;
  const int nvec = D / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * D);
  const uint4* rr = HAS_RES ? reinterpret_cast<const uint4*>(res + (long long)row * D) : nullptr;
  uint4 buf[NORM_MAX_VEC];
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int vi = t + i * TPR;
    if (vi < nvec) {
      uint4 v = xr[vi];
      uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
      if (HAS_RES) {
        uint4 r = rr[vi];
        const uint32_t* pr = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) pv[j] = pack_bf16(bf16_lo(pv[j]) + bf16_lo(pr[j]), bf16_hi(pv[j]) + bf16_hi(pr[j]));
        reinterpret_cast<uint4*>(sum_out + (long long)row * D)[vi] = v;
      }
      buf[i] = v;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float a = bf16_lo(pv[j]), c = bf16_hi(pv[j]);
        s1 += a + c;
        s2 += a * a + c * c;
      }
    }
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if (TPR > 32) {
    const int wid = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) { red[0][wid] = s1; red[1][wid] = s2; }
    __syncthreads();
    s1 = 0.f; s2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { s1 += red[0][i]; s2 += red[1][i]; }
  }
  const float inv_d = 1.0f / (float)D;
  float mean = RMS ? 0.f : s1 * inv_d;
  float var = s2 * inv_d - mean * mean;
  var = fmaxf(var, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (t == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  const uint4* bv = reinterpret_cast<const uint4*>(b);
  uint4* yr = reinterpret_cast<uint4*>(y + (long long)row * D);
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int vi = t + i * TPR;
    if (vi < nvec) {
      const uint32_t* pv = reinterpret_cast<const uint32_t*>(&buf[i]);
      uint4 wq = wv[vi];
      const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wq);
      uint4 bq = make_uint4(0, 0, 0, 0);
      if (!RMS && b) bq = bv[vi];
      const uint32_t* pb = reinterpret_cast<const uint32_t*>(&bq);
      uint4 o;
      uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = (bf16_lo(pv[j]) - mean) * rstd * bf16_lo(pw[j]) + bf16_lo(pb[j]);
        const float hi = (bf16_hi(pv[j]) - mean) * rstd * bf16_hi(pw[j]) + bf16_hi(pb[j]);
        po[j] = pack_bf16(lo, hi);
      }
      yr[vi] = o;
    }
  }
}

// Backward. One CTA works on one row at a time (rows strided over the grid); thread t owns the 8
// columns of vector t (+ i*blockDim for D > 8192), so its share of dw/db lives in registers for
// the whole kernel and is written once, as row blockIdx.x of the [gridDim.x, D] partial buffers.
// The two per-row scalars are reduced across warps through a double-buffered shared array.
template <bool RMS, int V>
__global__ void __launch_bounds__(1024) norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                                                        const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dres,
                                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                                                        float* __restrict__ db_part, int rows, int D) {
  __shared__ float red[2][2][32];
  const int t = threadIdx.x, lane = t & 31, wid = t >> 5, nt = blockDim.x, nwarps = nt >> 5;
  const int nvec = D / 8;
  float accw[V][8], accb[V][8], wf[V][8];
  const uint4* wv = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int vi = t + i * nt;
    uint4 wq = make_uint4(0, 0, 0, 0);
    if (vi < nvec) wq = wv[vi];
    const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wq);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wf[i][2 * j] = bf16_lo(pw[j]);
      wf[i][2 * j + 1] = bf16_hi(pw[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) { accw[i][j] = 0.f; accb[i][j] = 0.f; }
  }
  const float inv_d = 1.0f / (float)D;
  int iter = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, ++iter) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (long long)row * D);
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * D);
    const float mu = RMS ? 0.f : mean[row];
    const float rs = rstd[row];
    float g[V][8], xh[V][8];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * nt;
      if (vi < nvec) {
        const uint4 dq = dyr[vi], xq = xr[vi];
        const uint32_t* pd = reinterpret_cast<const uint32_t*>(&dq);
        const uint32_t* px = reinterpret_cast<const uint32_t*>(&xq);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float d0 = bf16_lo(pd[j]), d1 = bf16_hi(pd[j]);
          const float x0 = (bf16_lo(px[j]) - mu) * rs, x1 = (bf16_hi(px[j]) - mu) * rs;
          accw[i][2 * j] += d0 * x0;
          accw[i][2 * j + 1] += d1 * x1;
          accb[i][2 * j] += d0;
          accb[i][2 * j + 1] += d1;
          const float g0 = d0 * wf[i][2 * j], g1 = d1 * wf[i][2 * j + 1];
          g[i][2 * j] = g0; g[i][2 * j + 1] = g1;
          xh[i][2 * j] = x0; xh[i][2 * j + 1] = x1;
          c1 += g0 + g1;
          c2 += g0 * x0 + g1 * x1;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) { g[i][j] = 0.f; xh[i][j] = 0.f; }
      }
    }
    c1 = warp_sum(c1);
    c2 = warp_sum(c2);
    if (lane == 0) { red[iter & 1][0][wid] = c1; red[iter & 1][1][wid] = c2; }
    __syncthreads();
    c1 = 0.f; c2 = 0.f;
    for (int k = 0; k < nwarps; ++k) { c1 += red[iter & 1][0][k]; c2 += red[iter & 1][1][k]; }
    c1 = RMS ? 0.f : c1 * inv_d;
    c2 *= inv_d;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (long long)row * D);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + (long long)row * D) : nullptr;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * nt;
      if (vi < nvec) {
        uint4 rq = make_uint4(0, 0, 0, 0);
        if (drr) rq = drr[vi];
        const uint32_t* pr = reinterpret_cast<const uint32_t*>(&rq);
        uint4 o;
        uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = rs * (g[i][2 * j] - c1 - xh[i][2 * j] * c2) + bf16_lo(pr[j]);
          const float hi = rs * (g[i][2 * j + 1] - c1 - xh[i][2 * j + 1] * c2) + bf16_hi(pr[j]);
          po[j] = pack_bf16(lo, hi);
        }
        dxr[vi] = o;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int vi = t + i * nt;
    if (vi < nvec) {
      float4* pw = reinterpret_cast<float4*>(dw_part + (long long)blockIdx.x * D + vi * 8);
      pw[0] = make_float4(accw[i][0], accw[i][1], accw[i][2], accw[i][3]);
      pw[1] = make_float4(accw[i][4], accw[i][5], accw[i][6], accw[i][7]);
      if (!RMS) {
        float4* pb = reinterpret_cast<float4*>(db_part + (long long)blockIdx.x * D + vi * 8);
        pb[0] = make_float4(accb[i][0], accb[i][1], accb[i][2], accb[i][3]);
        pb[1] = make_float4(accb[i][4], accb[i][5], accb[i][6], accb[i][7]);
      }
    }
  }
}

// out[c] (+)= sum_p part[p, c]; out is bf16 or fp32.
template <typename OutT>
__global__ void reduce_partials_kernel(const float* __restrict__ part, OutT* __restrict__ out, int P, int D, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += part[(long long)p * D + c];
  if (accumulate) s += (float)out[c];
  out[c] = (OutT)s;
}

}  // namespace
}  // namespace elfa

using namespace elfa;

static int norm_check(int rows, int D) {
  ELFA_REQUIRE(rows > 0 && D > 0, "norm: empty input");
  ELFA_REQUIRE(D % 8 == 0, "norm: D must be a multiple of 8");
  ELFA_REQUIRE(D <= 256 * NORM_MAX_VEC * 8, "norm: D too large (max 32768)");
  return ELFA_OK;
}

// y = norm(x [+ res]) * w [+ b]; kind: 0 = LayerNorm, 1 = RMSNorm. `res`/`sum_out` may be null
// (no residual). mean_out may be null for RMSNorm.
ELFA_API int elfa_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* sum_out, float* mean_out,
                           float* rstd_out, int rows, int D, float eps, int kind, void* stream) {
  int rc = norm_check(rows, D);
  if (rc) return rc;
  ELFA_REQUIRE(x && w && y, "norm_fwd: null pointer");
  ELFA_REQUIRE(!res || sum_out, "norm_fwd: residual given without sum_out");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* X = static_cast<const __nv_bfloat16*>(x);
  const auto* R = static_cast<const __nv_bfloat16*>(res);
  const auto* W = static_cast<const __nv_bfloat16*>(w);
  const auto* B = static_cast<const __nv_bfloat16*>(b);
  auto* Y = static_cast<__nv_bfloat16*>(y);
  auto* S = static_cast<__nv_bfloat16*>(sum_out);
  const bool warp_row = D <= 32 * NORM_MAX_VEC * 8;  // <= 4096: one warp per row, 16 independent 16-byte loads per lane
  const bool rms = kind == 1, has_res = res != nullptr;
#define LAUNCH_FWD(TPR, RMS_, RES_)                                                                                     \
  norm_fwd_kernel<TPR, RMS_, RES_><<<(rows + (256 / TPR) - 1) / (256 / TPR), 256, 0, s>>>(X, R, W, B, Y, S, mean_out, rstd_out, \
                                                                                           rows, D, eps)
  if (warp_row) {
    if (rms) { if (has_res) LAUNCH_FWD(32, true, true); else LAUNCH_FWD(32, true, false); }
    else { if (has_res) LAUNCH_FWD(32, false, true); else LAUNCH_FWD(32, false, false); }
  } else {
    if (rms) { if (has_res) LAUNCH_FWD(256, true, true); else LAUNCH_FWD(256, true, false); }
    else { if (has_res) LAUNCH_FWD(256, false, true); else LAUNCH_FWD(256, false, false); }
  }
#undef LAUNCH_FWD
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Number of partial rows the backward kernel writes for a given problem (scratch = 2 * P * D floats).
ELFA_API int elfa_norm_bwd_partials(int rows, int D) {
  (void)D;
  return rows < 592 ? rows : 592;
}

// dx = norm backward (+ dres); dw/db (bf16 or fp32 per `grads_f32`) are accumulated when
// `accumulate` is set. scratch: 2 * elfa_norm_bwd_partials(rows, D) * D floats.
ELFA_API int elfa_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, const void* dres,
                           void* dx, void* dw, void* db, float* scratch, int rows, int D, int kind, int grads_f32,
                           int accumulate, void* stream) {
  int rc = norm_check(rows, D);
  if (rc) return rc;
  ELFA_REQUIRE(dy && x && w && rstd && dx && dw && scratch, "norm_bwd: null pointer");
  ELFA_REQUIRE(D <= 16384, "norm_bwd: D too large (max 16384)");
  ELFA_REQUIRE(kind == 1 || mean, "norm_bwd: LayerNorm needs the saved mean");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int P = elfa_norm_bwd_partials(rows, D);
  float* dw_part = scratch;
  float* db_part = scratch + (long long)P * D;
  const bool rms = kind == 1;
  const int nvec = D / 8;
  const int V = nvec > 1024 ? 2 : 1;
  int threads = ((nvec + V - 1) / V + 31) / 32 * 32;
#define LAUNCH_BWD(RMS_, V_)                                                                                                    norm_bwd_kernel<RMS_, V_><<<P, threads, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),                                                   static_cast<const __nv_bfloat16*>(w), mean, rstd,                                                                             static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx),                                                     dw_part, db_part, rows, D)
  if (V == 1) { if (rms) LAUNCH_BWD(true, 1); else LAUNCH_BWD(false, 1); }
  else { if (rms) LAUNCH_BWD(true, 2); else LAUNCH_BWD(false, 2); }
#undef LAUNCH_BWD
  ELFA_CUDA(cudaGetLastError());
  const int blocks = (D + 255) / 256;
  if (grads_f32) {
    reduce_partials_kernel<float><<<blocks, 256, 0, s>>>(dw_part, static_cast<float*>(dw), P, D, accumulate);
    if (!rms && db) reduce_partials_kernel<float><<<blocks, 256, 0, s>>>(db_part, static_cast<float*>(db), P, D, accumulate);
  } else {
    reduce_partials_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(dw_part, static_cast<__nv_bfloat16*>(dw), P, D, accumulate);
    if (!rms && db)
      reduce_partials_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(db_part, static_cast<__nv_bfloat16*>(db), P, D, accumulate);
  }
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(3);
  return ELFA_OK;
}
