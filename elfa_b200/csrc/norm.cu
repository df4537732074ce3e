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

__device__ __forceinline__ uint4 ld_or_zero(const uint4* p, bool ok) {
  uint4 v = make_uint4(0, 0, 0, 0);
  if (ok) v = *p;
  return v;
}

// TPR = threads per row (32 ... 256, a CTA of 256 threads holds 256 / TPR rows), NV = 16-byte vectors per
// thread. Every load of a row is issued before the first use (NV independent loads per thread in
// flight), then the statistics, then the output pass from registers: x is read once.
template <int TPR, int NV, bool RMS, bool HAS_RES>
__global__ void __launch_bounds__(256, NV <= 8 ? (HAS_RES ? 2 : 3) : 1) norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                                       const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                                                       __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out,
                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows,
                                                       int D, float eps) {
  constexpr int ROWS_PER_BLOCK = 256 / TPR;
  constexpr int ROW_WARPS = TPR / 32;
  __shared__ float red[2][8];
  const int t = threadIdx.x % TPR;
  const int row = blockIdx.x * ROWS_PER_BLOCK + threadIdx.x / TPR;
  const bool valid = row < rows;
  const int nvec = D / 8;
  const long long off = (long long)(valid ? row : 0) * D;
  const uint4* xr = reinterpret_cast<const uint4*>(x + off);
  uint4 buf[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) buf[i] = ld_or_zero(xr + t + i * TPR, valid && t + i * TPR < nvec);
  if (HAS_RES) {
    const uint4* rr = reinterpret_cast<const uint4*>(res + off);
    uint4 rb[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) rb[i] = ld_or_zero(rr + t + i * TPR, valid && t + i * TPR < nvec);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      uint32_t* pv = reinterpret_cast<uint32_t*>(&buf[i]);
      const uint32_t* pr = reinterpret_cast<const uint32_t*>(&rb[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) pv[j] = pack_bf16(bf16_lo(pv[j]) + bf16_lo(pr[j]), bf16_hi(pv[j]) + bf16_hi(pr[j]));
      if (valid && t + i * TPR < nvec) reinterpret_cast<uint4*>(sum_out + off)[t + i * TPR] = buf[i];
    }
  }
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const uint32_t* pv = reinterpret_cast<const uint32_t*>(&buf[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = bf16_lo(pv[j]), c = bf16_hi(pv[j]);
      s1 += a + c;
      s2 += a * a + c * c;
    }
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if (ROW_WARPS > 1) {
    const int wid = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) { red[0][wid] = s1; red[1][wid] = s2; }
    __syncthreads();
    const int w0 = (threadIdx.x / TPR) * ROW_WARPS;
    s1 = 0.f; s2 = 0.f;
#pragma unroll
    for (int i = 0; i < ROW_WARPS; ++i) { s1 += red[0][w0 + i]; s2 += red[1][w0 + i]; }
  }
  const float inv_d = 1.0f / (float)D;
  float mean = RMS ? 0.f : s1 * inv_d;
  float var = s2 * inv_d - mean * mean;
  var = fmaxf(var, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (t == 0 && valid) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  const uint4* bv = reinterpret_cast<const uint4*>(b);
  uint4* yr = reinterpret_cast<uint4*>(y + off);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = t + i * TPR;
    if (valid && vi < nvec) {
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

// two bf16 values of one 32-bit word as a packed fp32 pair
__device__ __forceinline__ uint64_t bf16x2_to_f32x2(uint32_t u) { return pack_f32x2(bf16_lo(u), bf16_hi(u)); }

// Backward. One CTA works on one row at a time (rows strided over the grid); thread t owns the 8
// columns of vector t (+ i*blockDim for D > 8192), so its share of dw/db lives in registers for
// the whole kernel and is written once, as row blockIdx.x of the [gridDim.x, D] partial buffers.
// The two per-row scalars are reduced across warps through a double-buffered shared array (one
// value per warp, summed again by a warp reduction). The next row's dy / x / residual gradient are
// requested before the reduction of the current row (V == 1), so the loads overlap the barrier and
// the output pass. The kernel is bound by instruction issue, not by memory, so the arithmetic runs
// on packed fp32 pairs and dy / x stay packed in registers (unpacked twice, never kept as fp32).
template <bool RMS, int V>
__global__ void __launch_bounds__(1024) norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean,
                                                        const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dres,
                                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_part,
                                                        float* __restrict__ db_part, int rows, int D) {
  constexpr bool PREFETCH = V == 1;
  __shared__ float red[2][2][32];
  const int t = threadIdx.x, lane = t & 31, wid = t >> 5, nt = blockDim.x, nwarps = nt >> 5;
  const int nvec = D / 8;
  uint64_t accw[V][4], accb[V][4], wf[V][4];
  const uint4* wv = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const uint4 wq = ld_or_zero(wv + t + i * nt, t + i * nt < nvec);
    const uint32_t* pw = reinterpret_cast<const uint32_t*>(&wq);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wf[i][j] = bf16x2_to_f32x2(pw[j]);
      accw[i][j] = 0ull;
      accb[i][j] = 0ull;
    }
  }
  const float inv_d = 1.0f / (float)D;
  uint4 dn[V], xn[V], rn[V];
  float mu_n = 0.f, rs_n = 0.f;
  auto fetch = [&](int row) {
    const bool ok = row < rows;
    const long long off = (long long)(ok ? row : 0) * D;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * nt;
      dn[i] = ld_or_zero(reinterpret_cast<const uint4*>(dy + off) + vi, ok && vi < nvec);
      xn[i] = ld_or_zero(reinterpret_cast<const uint4*>(x + off) + vi, ok && vi < nvec);
      rn[i] = ld_or_zero(reinterpret_cast<const uint4*>(dres + off) + vi, ok && dres != nullptr && vi < nvec);
    }
    if (ok) {
      mu_n = RMS ? 0.f : mean[row];
      rs_n = rstd[row];
    }
  };
  if (PREFETCH) fetch(blockIdx.x);
  int iter = 0;
  for (int row = blockIdx.x; row < rows; row += gridDim.x, ++iter) {
    if (!PREFETCH) fetch(row);
    uint4 dq[V], xq[V], rq[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { dq[i] = dn[i]; xq[i] = xn[i]; rq[i] = rn[i]; }
    const float rs = rs_n;
    const uint64_t rs2 = pack_f32x2(rs, rs), nmurs2 = pack_f32x2(-mu_n * rs, -mu_n * rs);
    if (PREFETCH) fetch(row + gridDim.x);
    // a zero-filled vector (beyond D) has dy = 0, so every product below is 0 whatever its x-hat is
    uint64_t s1 = 0ull, s2 = 0ull;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const uint32_t* pd = reinterpret_cast<const uint32_t*>(&dq[i]);
      const uint32_t* px = reinterpret_cast<const uint32_t*>(&xq[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint64_t d2 = bf16x2_to_f32x2(pd[j]);
        const uint64_t xh2 = fma_f32x2(bf16x2_to_f32x2(px[j]), rs2, nmurs2);
        accw[i][j] = fma_f32x2(d2, xh2, accw[i][j]);
        accb[i][j] = add_f32x2(accb[i][j], d2);
        const uint64_t g2 = mul_f32x2(d2, wf[i][j]);
        s1 = add_f32x2(s1, g2);
        s2 = fma_f32x2(g2, xh2, s2);
      }
    }
    float c1, c2, hi1, hi2;
    unpack_f32x2(s1, c1, hi1);
    unpack_f32x2(s2, c2, hi2);
    c1 = warp_sum(c1 + hi1);
    c2 = warp_sum(c2 + hi2);
    if (lane == 0) { red[iter & 1][0][wid] = c1; red[iter & 1][1][wid] = c2; }
    __syncthreads();
    c1 = warp_sum(lane < nwarps ? red[iter & 1][0][lane] : 0.f);
    c2 = warp_sum(lane < nwarps ? red[iter & 1][1][lane] : 0.f);
    c1 = RMS ? 0.f : c1 * inv_d;
    c2 *= inv_d;
    const uint64_t nc1 = pack_f32x2(-c1, -c1), nc2 = pack_f32x2(-c2, -c2);
    uint4* dxr = reinterpret_cast<uint4*>(dx + (long long)row * D);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const int vi = t + i * nt;
      if (vi < nvec) {
        const uint32_t* pd = reinterpret_cast<const uint32_t*>(&dq[i]);
        const uint32_t* px = reinterpret_cast<const uint32_t*>(&xq[i]);
        const uint32_t* pr = reinterpret_cast<const uint32_t*>(&rq[i]);
        uint4 o;
        uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint64_t g2 = mul_f32x2(bf16x2_to_f32x2(pd[j]), wf[i][j]);
          const uint64_t xh2 = fma_f32x2(bf16x2_to_f32x2(px[j]), rs2, nmurs2);
          // dx = rs * (g - c1 - xhat * c2) + dres
          const uint64_t o2 = fma_f32x2(fma_f32x2(xh2, nc2, add_f32x2(g2, nc1)), rs2, bf16x2_to_f32x2(pr[j]));
          float lo, hi;
          unpack_f32x2(o2, lo, hi);
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
      float a[8], c[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        unpack_f32x2(accw[i][j], a[2 * j], a[2 * j + 1]);
        unpack_f32x2(accb[i][j], c[2 * j], c[2 * j + 1]);
      }
      float4* pw = reinterpret_cast<float4*>(dw_part + (long long)blockIdx.x * D + vi * 8);
      pw[0] = make_float4(a[0], a[1], a[2], a[3]);
      pw[1] = make_float4(a[4], a[5], a[6], a[7]);
      if (!RMS) {
        float4* pb = reinterpret_cast<float4*>(db_part + (long long)blockIdx.x * D + vi * 8);
        pb[0] = make_float4(c[0], c[1], c[2], c[3]);
        pb[1] = make_float4(c[4], c[5], c[6], c[7]);
      }
    }
  }
}

// out[c] (+)= sum_p part[p, c] in a fixed order; out is bf16 or fp32. grid (ceil(D / 32), 1 or 2): blockIdx.y
// selects (part0, out0) or (part1, out1); block (32, 16): thread (c, r) adds rows r, r + 16, ... of column c.
template <typename OutT>
__global__ void __launch_bounds__(512) reduce_partials_kernel(const float* __restrict__ part0, const float* __restrict__ part1,
                                                              OutT* __restrict__ out0, OutT* __restrict__ out1, int P, int D,
                                                              int accumulate) {
  __shared__ float red[16][33];
  const float* part = blockIdx.y ? part1 : part0;
  OutT* out = blockIdx.y ? out1 : out0;
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < D)
    for (int p = threadIdx.y; p < P; p += 16) s += part[(long long)p * D + c];
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < D) {
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) tot += red[k][threadIdx.x];
    if (accumulate) tot += (float)out[c];
    out[c] = (OutT)tot;
  }
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
  const bool rms = kind == 1, has_res = res != nullptr;
#define LAUNCH_FWD(TPR, NV)                                                                                                  \
  do {                                                                                                                       \
    const int grid = (rows + (256 / TPR) - 1) / (256 / TPR);                                                                 \
    if (rms) {                                                                                                               \
      if (has_res) norm_fwd_kernel<TPR, NV, true, true><<<grid, 256, 0, s>>>(X, R, W, B, Y, S, mean_out, rstd_out, rows, D, eps);  \
      else norm_fwd_kernel<TPR, NV, true, false><<<grid, 256, 0, s>>>(X, R, W, B, Y, S, mean_out, rstd_out, rows, D, eps);    \
    } else {                                                                                                                 \
      if (has_res) norm_fwd_kernel<TPR, NV, false, true><<<grid, 256, 0, s>>>(X, R, W, B, Y, S, mean_out, rstd_out, rows, D, eps); \
      else norm_fwd_kernel<TPR, NV, false, false><<<grid, 256, 0, s>>>(X, R, W, B, Y, S, mean_out, rstd_out, rows, D, eps);   \
    }                                                                                                                        \
  } while (0)
  // at most 8 vectors (128 bytes) per thread up to D = 16384, so that several rows per SM are in flight
  if (D <= 1024) LAUNCH_FWD(32, 4);
  else if (D <= 2048) LAUNCH_FWD(32, 8);
  else if (D <= 4096) LAUNCH_FWD(64, 8);
  else if (D <= 8192) LAUNCH_FWD(128, 8);
  else if (D <= 16384) LAUNCH_FWD(256, 8);
  else LAUNCH_FWD(256, 16);
#undef LAUNCH_FWD
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Number of partial rows the backward kernel writes for a given problem (scratch = 2 * P * D floats).
static int norm_bwd_threads(int D) {
  const int nvec = D / 8;
  const int V = nvec > 1024 ? 2 : 1;
  return ((nvec + V - 1) / V + 31) / 32 * 32;
}

ELFA_API int elfa_norm_bwd_partials(int rows, int D) {
  int per_sm = 1024 / norm_bwd_threads(D > 0 ? D : 8);   // 64 registers per thread: 1024 threads resident per SM
  per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
  const int P = device_sm_count() * per_sm;
  return rows < P ? rows : P;
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
  const int V = D / 8 > 1024 ? 2 : 1;
  const int threads = norm_bwd_threads(D);
#define LAUNCH_BWD(RMS_, V_)                                                                                                     \
  norm_bwd_kernel<RMS_, V_><<<P, threads, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),   \
                                                  static_cast<const __nv_bfloat16*>(w), mean, rstd,                              \
                                                  static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx),      \
                                                  dw_part, db_part, rows, D)
  if (V == 1) { if (rms) LAUNCH_BWD(true, 1); else LAUNCH_BWD(false, 1); }
  else { if (rms) LAUNCH_BWD(true, 2); else LAUNCH_BWD(false, 2); }
#undef LAUNCH_BWD
  ELFA_CUDA(cudaGetLastError());
  const dim3 rgrid((D + 31) / 32, (!rms && db) ? 2 : 1), rblock(32, 16);
  if (grads_f32)
    reduce_partials_kernel<float><<<rgrid, rblock, 0, s>>>(dw_part, db_part, static_cast<float*>(dw), static_cast<float*>(db), P, D,
                                                           accumulate);
  else
    reduce_partials_kernel<__nv_bfloat16><<<rgrid, rblock, 0, s>>>(dw_part, db_part, static_cast<__nv_bfloat16*>(dw),
                                                                   static_cast<__nv_bfloat16*>(db), P, D, accumulate);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
  return ELFA_OK;
}
