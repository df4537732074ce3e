// EFLA recurrence (forward and backward) and the causal depthwise ShortConv (forward and backward).
//
// EFLA, per (batch, head), state S [d, d] fp32 (row = key index i, column = value index j):
//   lam = |k|^2, c = (1 - exp(-beta lam)) / lam, p = S^T k, e = v - p, S += c k e^T, o = p + c lam e
// (o equals S_new^T k). One CTA per (batch, head); thread j keeps column j of S in registers for the
// whole sequence (forward) so the state never leaves the chip and is never rounded to bf16 - the
// reference rounds the bf16 state in global memory on every token and launches once per chunk
// (reference: kernels/cuda/efla.cu:121-197 forward, :199-271 state history, :273-401 backward
// without the beta gradient; fp32 variant kernels/cuda/efla_scan.cu:99-260 with grad_beta via
// atomics; CPU math src/model/efla.zig:27-49,275-329,509-588).
// Backward walks the chunks in reverse: the states inside a chunk are recomputed from the chunk's
// saved boundary state into a global workspace ([chunk, d, d] per CTA), then the reverse-time
// recursion runs with S and dS in shared memory (padded rows, so both column and row sweeps are
// conflict free). beta gets its gradient; reductions are fixed-order (deterministic).
//
// ShortConv: y[b,t,c] = bias[c] + sum_w x[b,t-w,c] weight[c,w] (reference:
// kernels/cuda/convolution.cu:4-57,126-189; src/model/prism.zig:948-973). The weight gradient is a
// per-(channel, tap) reduction without atomics.
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

__device__ __forceinline__ void efla_coeff(float beta, float lam, float& c, float& dc_dbeta, float& dc_dlam) {
  if (lam < 1e-6f) {
    c = beta - 0.5f * beta * beta * lam + beta * beta * beta * lam * lam / 6.f;
    dc_dbeta = 1.f - beta * lam + 0.5f * beta * beta * lam * lam;
    dc_dlam = -0.5f * beta * beta + beta * beta * beta * lam / 3.f;
  } else {
    const float ex = __expf(-beta * lam);
    c = (1.f - ex) / lam;
    dc_dbeta = ex;
    dc_dlam = (beta * lam * ex - (1.f - ex)) / (lam * lam);
  }
}

// block-wide sum of one float per thread (blockDim.x = d <= 128), result broadcast
__device__ __forceinline__ float block_sum(float v, float* red, int nwarps) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
  for (int i = 0; i < nwarps; ++i) s += red[i];
  return s;
}

// k, v, o: [B, T, H, D] bf16. state0 / state_out: [B, H, D, D] fp32. ckpt: [B, H, nchunks, D, D] holds the
// state at the START of every chunk.
template <int D>
__global__ void __launch_bounds__(D) efla_scan_fwd_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                          const float* __restrict__ beta_ptr, const float* __restrict__ state0,
                                                          __nv_bfloat16* __restrict__ o, float* __restrict__ state_out,
                                                          float* __restrict__ ckpt, int T, int H, int chunk) {
  __shared__ float sk[D];
  __shared__ float red[4];
  const int bh = blockIdx.x, b = bh / H, h = bh % H, j = threadIdx.x;
  const float beta = *beta_ptr;
  float S[D];
  if (state0) {
#pragma unroll
    for (int i = 0; i < D; ++i) S[i] = state0[((long long)bh * D + i) * D + j];
  } else {
#pragma unroll
    for (int i = 0; i < D; ++i) S[i] = 0.f;
  }
  const int nchunks = (T + chunk - 1) / chunk;
  for (int t = 0; t < T; ++t) {
    if (ckpt && t % chunk == 0) {
      float* dst = ckpt + ((long long)bh * nchunks + t / chunk) * D * D;
#pragma unroll
      for (int i = 0; i < D; ++i) dst[i * D + j] = S[i];
    }
    const long long off = (((long long)b * T + t) * H + h) * D + j;
    const float kj = __bfloat162float(k[off]), vj = __bfloat162float(v[off]);
    __syncthreads();
    sk[j] = kj;
    const float lam = block_sum(kj * kj, red, D / 32);   // contains the barrier that publishes sk
    float c, d1, d2;
    efla_coeff(beta, lam, c, d1, d2);
    float p = 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) p += sk[i] * S[i];
    const float e = vj - p;
    const float ce = c * e;
#pragma unroll
    for (int i = 0; i < D; ++i) S[i] += sk[i] * ce;
    o[off] = __float2bfloat16(p + c * lam * e);
  }
  if (state_out) {
#pragma unroll
    for (int i = 0; i < D; ++i) state_out[((long long)bh * D + i) * D + j] = S[i];
  }
}

// Backward. Shared memory: S and dS as [D][D+1] fp32, vectors of D floats.
// work: [B*H][chunk][D][D] fp32 scratch (state BEFORE each token of the current chunk).
template <int D>
__global__ void __launch_bounds__(D) efla_scan_bwd_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                          const float* __restrict__ beta_ptr, const float* __restrict__ ckpt,
                                                          const __nv_bfloat16* __restrict__ dout, const float* __restrict__ dstate_out,
                                                          __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                                                          float* __restrict__ dbeta, float* __restrict__ dstate0,
                                                          float* __restrict__ work, int T, int H, int chunk) {
  extern __shared__ float sm[];
  constexpr int LD = D + 1;
  float* sS = sm;                 // [D][LD]  state before the current token
  float* sG = sS + D * LD;        // [D][LD]  gradient w.r.t. the state after the current token
  float* sk = sG + D * LD;        // [D]
  float* se = sk + D;             // [D] e = v - p
  float* sdo = se + D;            // [D]
  float* sde = sdo + D;           // [D]
  float* sdp = sde + D;           // [D]
  float* red = sdp + D;           // [4]
  const int bh = blockIdx.x, b = bh / H, h = bh % H, x = threadIdx.x;
  const float beta = *beta_ptr;
  const int nchunks = (T + chunk - 1) / chunk;
  float* wk = work + (long long)bh * chunk * D * D;
  for (int i = 0; i < D; ++i) sG[i * LD + x] = dstate_out ? dstate_out[((long long)bh * D + i) * D + x] : 0.f;
  float dbeta_acc = 0.f;
  for (int ch = nchunks - 1; ch >= 0; --ch) {
    const int t0 = ch * chunk, t1 = min(T, t0 + chunk);
    // ---- recompute the states of this chunk (column x in registers), store S_before per token
    {
      float S[D];
      const float* src = ckpt + ((long long)bh * nchunks + ch) * D * D;
#pragma unroll
      for (int i = 0; i < D; ++i) S[i] = src[i * D + x];
      for (int t = t0; t < t1; ++t) {
        float* dst = wk + (long long)(t - t0) * D * D;
#pragma unroll
        for (int i = 0; i < D; ++i) dst[i * D + x] = S[i];
        const long long off = (((long long)b * T + t) * H + h) * D + x;
        const float kx = __bfloat162float(k[off]), vx = __bfloat162float(v[off]);
        __syncthreads();
        sk[x] = kx;
        const float lam = block_sum(kx * kx, red, D / 32);
        float c, d1, d2;
        efla_coeff(beta, lam, c, d1, d2);
        float p = 0.f;
#pragma unroll
        for (int i = 0; i < D; ++i) p += sk[i] * S[i];
        const float ce = c * (vx - p);
#pragma unroll
        for (int i = 0; i < D; ++i) S[i] += sk[i] * ce;
      }
    }
    __syncthreads();
    // ---- reverse-time recursion over the chunk
    for (int t = t1 - 1; t >= t0; --t) {
      const long long off = (((long long)b * T + t) * H + h) * D + x;
      const float kx = __bfloat162float(k[off]), vx = __bfloat162float(v[off]);
      const float gox = __bfloat162float(dout[off]);
      const float* src = wk + (long long)(t - t0) * D * D;
      __syncthreads();
      for (int i = 0; i < D; ++i) sS[i * LD + x] = src[i * D + x];   // S before token t
      sk[x] = kx;
      sdo[x] = gox;
      const float lam = block_sum(kx * kx, red, D / 32);
      float c, dc_db, dc_dl;
      efla_coeff(beta, lam, c, dc_db, dc_dl);
      // column sweep (x = value index j): p_j, e_j
      float p = 0.f;
      for (int i = 0; i < D; ++i) p += sk[i] * sS[i * LD + x];
      const float e = vx - p;
      se[x] = e;
      __syncthreads();
      // o = S'^T k: dS' += k do^T (column x gets k_i * do_x)
      for (int i = 0; i < D; ++i) sG[i * LD + x] += sk[i] * gox;
      __syncthreads();
      // row sweep (x = key index i): a_i = sum_j S'_ij do_j, b_i = sum_j dS'_ij e_j
      float a = 0.f, bsum = 0.f;
      const float ck = c * kx;
      for (int jj = 0; jj < D; ++jj) {
        const float sp = sS[x * LD + jj] + ck * se[jj];     // S'_ij
        a += sp * sdo[jj];
        bsum += sG[x * LD + jj] * se[jj];
      }
      // dc = sum_i k_i b_i
      const float dc = block_sum(kx * bsum, red, D / 32);
      // column sweep: de_j = c * sum_i dS'_ij k_i ; dp = -de
      float de = 0.f;
      for (int i = 0; i < D; ++i) de += sG[i * LD + x] * sk[i];
      de *= c;
      sde[x] = de;
      sdp[x] = -de;
      __syncthreads();
      // row sweep: g_i = sum_j S_ij dp_j  (p = S^T k -> dk += S dp)
      float g = 0.f;
      for (int jj = 0; jj < D; ++jj) g += sS[x * LD + jj] * sdp[jj];
      const float dlam = dc * dc_dl;
      const float dkx = a + c * bsum + g + 2.f * kx * dlam;
      dbeta_acc += (x == 0) ? dc * dc_db : 0.f;
      dk[off] = __float2bfloat16(dkx);
      dv[off] = __float2bfloat16(de);
      // dS (before token) = dS' + k dp^T
      for (int i = 0; i < D; ++i) sG[i * LD + x] += sk[i] * sdp[x];
    }
  }
  __syncthreads();
  if (dstate0)
    for (int i = 0; i < D; ++i) dstate0[((long long)bh * D + i) * D + x] = sG[i * LD + x];
  if (x == 0) dbeta[bh] = dbeta_acc;
}

// ------------------------------------------------------------------------------------ ShortConv
__global__ void __launch_bounds__(256) shortconv_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                            const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int B,
                                                            int T, int C, int W) {
  const long long n = (long long)B * T * C;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int c = (int)(i % C);
    const int t = (int)((i / C) % T);
    float acc = bias ? __bfloat162float(bias[c]) : 0.f;
    const int wmax = min(W, t + 1);
    for (int j = 0; j < wmax; ++j) acc += __bfloat162float(x[i - (long long)j * C]) * __bfloat162float(w[c * W + j]);
    y[i] = __float2bfloat16(acc);
  }
}

// dx[b,t,c] = sum_w dy[b,t+w,c] weight[c,w]
__global__ void __launch_bounds__(256) shortconv_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ dx, int B, int T, int C, int W) {
  const long long n = (long long)B * T * C;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int c = (int)(i % C);
    const int t = (int)((i / C) % T);
    float acc = 0.f;
    const int wmax = min(W, T - t);
    for (int j = 0; j < wmax; ++j) acc += __bfloat162float(dy[i + (long long)j * C]) * __bfloat162float(w[c * W + j]);
    dx[i] = __float2bfloat16(acc);
  }
}

// dw[c,w] = sum_{b,t>=w} dy[b,t,c] x[b,t-w,c]; db[c] = sum dy. grid (ceil(C/32), W + 1), block (32, 8):
// blockIdx.y == W computes the bias gradient.
__global__ void __launch_bounds__(256) shortconv_bwd_dw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                               float* __restrict__ dw, float* __restrict__ db, int B, int T, int C,
                                                               int W) {
  __shared__ float sm[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int wj = blockIdx.y;
  float acc = 0.f;
  if (c < C) {
    const long long rows = (long long)B * T;
    for (long long r = threadIdx.y; r < rows; r += 8) {
      const int t = (int)(r % T);
      const float g = __bfloat162float(dy[r * C + c]);
      if (wj == W) acc += g;
      else if (t >= wj) acc += g * __bfloat162float(x[(r - wj) * C + c]);
    }
  }
  sm[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < C) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += sm[i][threadIdx.x];
    if (wj == W) { if (db) db[c] = s; }
    else dw[c * W + wj] = s;
  }
}

template <int D>
int launch_efla_fwd(const void* k, const void* v, const float* beta, const float* state0, void* o, float* state_out, float* ckpt, int B,
                    int T, int H, int chunk, cudaStream_t s) {
  efla_scan_fwd_kernel<D><<<B * H, D, 0, s>>>(static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), beta, state0,
                                              static_cast<__nv_bfloat16*>(o), state_out, ckpt, T, H, chunk);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

template <int D>
int launch_efla_bwd(const void* k, const void* v, const float* beta, const float* ckpt, const void* dout, const float* dstate_out,
                    void* dk, void* dv, float* dbeta, float* dstate0, float* work, int B, int T, int H, int chunk, cudaStream_t s) {
  const size_t smem = (size_t)(2 * D * (D + 1) + 5 * D + 8) * sizeof(float);
  auto kern = efla_scan_bwd_kernel<D>;
  if (smem > 48 * 1024) ELFA_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<B * H, D, smem, s>>>(static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), beta, ckpt,
                              static_cast<const __nv_bfloat16*>(dout), dstate_out, static_cast<__nv_bfloat16*>(dk),
                              static_cast<__nv_bfloat16*>(dv), dbeta, dstate0, work, T, H, chunk);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// k, v, o: [B, T, H, d] bf16; beta: 1 float; state0 (optional) / state_out: [B, H, d, d] fp32;
// ckpt: [B, H, ceil(T/chunk), d, d] fp32 (chunk-start states, needed by backward) or null.
ELFA_API int elfa_efla_scan_fwd(const void* k, const void* v, const float* beta, const float* state0, void* o, float* state_out,
                                float* ckpt, int B, int T, int H, int d, int chunk, void* stream) {
  ELFA_REQUIRE(k && v && beta && o && B > 0 && T > 0 && H > 0 && chunk > 0, "efla_scan_fwd: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (d) {
    case 32: return launch_efla_fwd<32>(k, v, beta, state0, o, state_out, ckpt, B, T, H, chunk, s);
    case 64: return launch_efla_fwd<64>(k, v, beta, state0, o, state_out, ckpt, B, T, H, chunk, s);
    case 96: return launch_efla_fwd<96>(k, v, beta, state0, o, state_out, ckpt, B, T, H, chunk, s);
    case 128: return launch_efla_fwd<128>(k, v, beta, state0, o, state_out, ckpt, B, T, H, chunk, s);
    default: set_last_error("efla_scan_fwd: head dimension must be 32, 64, 96 or 128"); return ELFA_ERR_UNSUPPORTED;
  }
}

// Gradients of elfa_efla_scan_fwd. dbeta: [B*H] partial sums (add them up); work: [B*H, chunk, d, d] fp32.
ELFA_API int elfa_efla_scan_bwd(const void* k, const void* v, const float* beta, const float* ckpt, const void* dout,
                                const float* dstate_out, void* dk, void* dv, float* dbeta, float* dstate0, float* work, int B, int T,
                                int H, int d, int chunk, void* stream) {
  ELFA_REQUIRE(k && v && beta && ckpt && dout && dk && dv && dbeta && work && B > 0 && T > 0 && H > 0 && chunk > 0,
               "efla_scan_bwd: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (d) {
    case 32: return launch_efla_bwd<32>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta, dstate0, work, B, T, H, chunk, s);
    case 64: return launch_efla_bwd<64>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta, dstate0, work, B, T, H, chunk, s);
    case 96: return launch_efla_bwd<96>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta, dstate0, work, B, T, H, chunk, s);
    case 128: return launch_efla_bwd<128>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta, dstate0, work, B, T, H, chunk, s);
    default: set_last_error("efla_scan_bwd: head dimension must be 32, 64, 96 or 128"); return ELFA_ERR_UNSUPPORTED;
  }
}

ELFA_API int elfa_shortconv_fwd(const void* x, const void* w, const void* bias, void* y, int B, int T, int C, int W, void* stream) {
  ELFA_REQUIRE(x && w && y && B > 0 && T > 0 && C > 0 && W > 0, "shortconv_fwd: bad arguments");
  const long long n = (long long)B * T * C;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  shortconv_fwd_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(bias),
      static_cast<__nv_bfloat16*>(y), B, T, C, W);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// dx bf16 [B,T,C]; dw fp32 [C,W]; db fp32 [C] or null.
ELFA_API int elfa_shortconv_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, float* db, int B, int T, int C, int W,
                                void* stream) {
  ELFA_REQUIRE(x && w && dy && dx && dw && B > 0 && T > 0 && C > 0 && W > 0, "shortconv_bwd: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long n = (long long)B * T * C;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  shortconv_bwd_dx_kernel<<<(int)blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(w),
                                                      static_cast<__nv_bfloat16*>(dx), B, T, C, W);
  dim3 grid((C + 31) / 32, W + 1), block(32, 8);
  shortconv_bwd_dw_kernel<<<grid, block, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), dw, db, B,
                                                 T, C, W);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
  return ELFA_OK;
}
