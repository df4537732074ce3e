// EFLA recurrence (forward and backward) and the causal depthwise ShortConv (forward and backward).
//
// EFLA, per (batch, head), state S [d, d] fp32 (row = key index i, column = value index j):
//   lam = |k|^2, c = (1 - exp(-beta lam)) / lam, p = S^T k, e = v - p, S += c k e^T, o = p + c lam e
// (o equals S_new^T k). Forward: one CTA of four warps per (batch, head, 32 value columns); its threads keep the
// state in registers for the whole sequence so it never leaves the chip and is never rounded to bf16 - the
// reference rounds the bf16 state in global memory on every token and launches once per chunk
// (reference: kernels/cuda/efla.cu:121-197 forward, :199-271 state history, :273-401 backward
// without the beta gradient; fp32 variant kernels/cuda/efla_scan.cu:99-260 with grad_beta via
// atomics; CPU math src/model/efla.zig:27-49,275-329,509-588).
// Backward walks the chunks in reverse with the same thread layout: the states inside a chunk are
// recomputed from the chunk's saved boundary state into a global workspace ([chunk, d, d] per (batch,
// head)), then the reverse-time recursion keeps the state gradient in registers and sums the key-gradient
// rows through a per-warp shared-memory transpose. beta gets its gradient; reductions are fixed-order
// (deterministic).
//
// ShortConv: y[b,t,c] = bias[c] + sum_w x[b,t-w,c] weight[c,w] (reference:
// kernels/cuda/convolution.cu:4-57,126-189; src/model/prism.zig:948-973). The weight gradient is one
// pass over the rows per (32 channels, 4 taps) without atomics.
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

// k, v, o: [B, T, H, D] bf16. state0 / state_out: [B, H, D, D] fp32. ckpt: [B, H, nchunks, D, D] holds the
// state at the START of every chunk.
// The columns of S evolve independently (column j needs k_t, c_t and v_t[j] only), so a CTA owns 32 value columns:
// grid (B*H, D/32). Its four warps split the D key rows: warp w keeps rows [w D/4, (w+1) D/4) of the 32 columns in
// registers (lane = column), so the dependent instruction chain of a step is a quarter as long and the four
// schedulers of the SM all have a warp. A step costs one block barrier: the warps exchange their partial dot
// products through a parity-double-buffered shared array. Time is walked in tiles of EFLA_TT tokens: every warp
// fetches eight of the tile's rows with all loads in flight together (keys as fp32, the CTA's 32 value columns),
// warp 0 computes lam / c for the whole tile (lane r owns token r), and the sequential part touches global memory
// only for the output.
constexpr int EFLA_TT = 32;
constexpr int EFLA_W = 4;

template <int D>
__device__ __forceinline__ void efla_load_tile(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                               const __nv_bfloat16* __restrict__ dout, float (*sk)[D], float (*sv)[32], float (*sdo)[32],
                                               float* sc, float* slam, float beta, long long row0, long long row_stride, int col,
                                               int n, int warp, int lane) {
  __syncthreads();                                       // the previous tile has been consumed
  const int r0 = warp * (EFLA_TT / EFLA_W);
  if (r0 < n) {
    __nv_bfloat16 kq[8][D / 32], vq[8], dq[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const long long row = row0 + (long long)min(r0 + u, n - 1) * row_stride;      // clamped: rows past the end re-read the last one
#pragma unroll
      for (int c = 0; c < D / 32; ++c) kq[u][c] = k[row + c * 32 + lane];
      vq[u] = v[row + col];
      if (dout) dq[u] = dout[row + col];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) sk[r0 + u][c * 32 + lane] = __bfloat162float(kq[u][c]);
      sv[r0 + u][lane] = __bfloat162float(vq[u]);
      if (dout) sdo[r0 + u][lane] = __bfloat162float(dq[u]);
    }
  }
  __syncthreads();
  if (warp == 0 && lane < n) {                           // the rotated index keeps the banks apart
    float lam = 0.f;
#pragma unroll 8
    for (int c = 0; c < D; ++c) {
      const float x = sk[lane][(c + lane) % D];
      lam += x * x;
    }
    float c_, d1, d2;
    efla_coeff(beta, lam, c_, d1, d2);
    sc[lane] = c_;
    if (slam) slam[lane] = lam;
  }
  __syncthreads();
}

// One step of the recurrence for this warp's R rows: returns p (complete, after the exchange) and applies the update.
template <int R>
__device__ __forceinline__ float efla_step(float (&S)[R], const float* __restrict__ krow, float c_, float vj, float* part, int warp,
                                           int lane) {
  const float4* kr = reinterpret_cast<const float4*>(krow);
  float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
  for (int i = 0; i < R / 4; ++i) {
    const float4 kk = kr[i];
    p0 += kk.x * S[4 * i];
    p1 += kk.y * S[4 * i + 1];
    p2 += kk.z * S[4 * i + 2];
    p3 += kk.w * S[4 * i + 3];
  }
  part[warp * 32 + lane] = (p0 + p1) + (p2 + p3);
  __syncthreads();
  const float p = (part[lane] + part[32 + lane]) + (part[64 + lane] + part[96 + lane]);
  const float ce = c_ * (vj - p);
#pragma unroll
  for (int i = 0; i < R / 4; ++i) {
    const float4 kk = kr[i];
    S[4 * i] += kk.x * ce;
    S[4 * i + 1] += kk.y * ce;
    S[4 * i + 2] += kk.z * ce;
    S[4 * i + 3] += kk.w * ce;
  }
  return p;
}

template <int D>
__global__ void __launch_bounds__(32 * EFLA_W) efla_scan_fwd_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                                    const float* __restrict__ beta_ptr, const float* __restrict__ state0,
                                                                    __nv_bfloat16* __restrict__ o, float* __restrict__ state_out,
                                                                    float* __restrict__ ckpt, int T, int H, int chunk) {
  constexpr int R = D / EFLA_W;
  __shared__ __align__(16) float sk[EFLA_TT][D];
  __shared__ float sv[EFLA_TT][32];
  __shared__ float sc[EFLA_TT], slam[EFLA_TT];
  __shared__ float spart[2][EFLA_W * 32];
  const int bh = blockIdx.x, b = bh / H, h = bh % H, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.y * 32 + lane, i0 = warp * R;
  const float beta = *beta_ptr;
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i) S[i] = state0 ? state0[((long long)bh * D + i0 + i) * D + col] : 0.f;
  const int nchunks = (T + chunk - 1) / chunk;
  for (int t0 = 0; t0 < T; t0 += EFLA_TT) {
    const int n = min(EFLA_TT, T - t0);
    efla_load_tile<D>(k, v, nullptr, sk, sv, nullptr, sc, slam, beta, (((long long)b * T + t0) * H + h) * D, (long long)H * D, col, n,
                      warp, lane);
    for (int r = 0; r < n; ++r) {
      const int t = t0 + r;
      if (ckpt && t % chunk == 0) {
        float* dst = ckpt + ((long long)bh * nchunks + t / chunk) * D * D;
#pragma unroll
        for (int i = 0; i < R; ++i) dst[(i0 + i) * D + col] = S[i];
      }
      const float c_ = sc[r], vj = sv[r][lane];
      const float p = efla_step<R>(S, sk[r] + i0, c_, vj, spart[r & 1], warp, lane);
      if (warp == 0) o[(((long long)b * T + t) * H + h) * D + col] = __float2bfloat16(p + c_ * slam[r] * (vj - p));
    }
  }
  if (state_out) {
#pragma unroll
    for (int i = 0; i < R; ++i) state_out[((long long)bh * D + i0 + i) * D + col] = S[i];
  }
}

// Backward: the same layout (CTA = 32 value columns, warp w = key rows [w D/4, (w+1) D/4), lane = column). Every warp
// keeps its rows of G = dL/dS (the gradient with respect to the state AFTER the current token) in registers for
// the whole sequence. Chunks are walked in reverse; inside a chunk the states are recomputed from the chunk's saved
// boundary state and the state BEFORE every token goes to a global workspace ([chunk, D, D] per (batch, head); a
// thread reads back only what it wrote), then the reverse-time recursion streams each of them twice:
//   pass 1: p_j = sum_i k_i S_ij ;  G_ij += k_i do_j ;  w_j = sum_i G_ij k_i   (partial over the warp's rows; ONE block
//           barrier per step exchanges both partial sums) ;  e_j = v_j - p_j ;  dv_j = de_j = c w_j ;  dp_j = -de_j ;
//           dc = sum_j e_j w_j (over the lanes here, over the column blocks in the finishing kernel)
//   pass 2: r_ij = (S_ij + c k_i e_j) do_j + c G_ij e_j + S_ij dp_j ;  G_ij += k_i dp_j
// dk_i = sum_j r_ij + 2 k_i dc dc/dlam needs a sum over ALL value columns: within the warp it goes through a
// padded shared-memory transpose private to the warp (lane j writes r_.j, lane i adds up row i), across the D/32
// column blocks through fp32 partial buffers that efla_bwd_finish_kernel adds up (fixed order: deterministic)
// together with the lam term and the per-token beta gradient.
// work: [B*H][chunk][D][D] fp32. dk_part: [D/32][rows][D] fp32, dc_part: [D/32][rows] fp32, rows = B*T*H.
template <int D>
__global__ void __launch_bounds__(32 * EFLA_W) efla_scan_bwd_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                                                    const float* __restrict__ beta_ptr, const float* __restrict__ ckpt,
                                                                    const __nv_bfloat16* __restrict__ dout,
                                                                    const float* __restrict__ dstate_out, float* __restrict__ dk_part,
                                                                    __nv_bfloat16* __restrict__ dv, float* __restrict__ dc_part,
                                                                    float* __restrict__ dstate0, float* __restrict__ work, int B, int T,
                                                                    int H, int chunk) {
  constexpr int R = D / EFLA_W;
  __shared__ __align__(16) float sk[EFLA_TT][D];
  __shared__ float sv[EFLA_TT][32], sdo[EFLA_TT][32];
  __shared__ float sc[EFLA_TT];
  __shared__ float spart[2][2 * EFLA_W * 32];            // [parity][p partials | w partials]
  __shared__ float sred[EFLA_W][R][33];
  const int bh = blockIdx.x, b = bh / H, h = bh % H, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col = blockIdx.y * 32 + lane, i0 = warp * R;
  const long long rows = (long long)B * T * H;
  const float beta = *beta_ptr;
  const int nchunks = (T + chunk - 1) / chunk;
  float* wk = work + (long long)bh * chunk * D * D + (long long)i0 * D + col;     // this thread's first element of a token's state
  float* dkp = dk_part + (long long)blockIdx.y * rows * D;
  float* dcp = dc_part + (long long)blockIdx.y * rows;
  float G[R];
#pragma unroll
  for (int i = 0; i < R; ++i) G[i] = dstate_out ? dstate_out[((long long)bh * D + i0 + i) * D + col] : 0.f;

  for (int ch = nchunks - 1; ch >= 0; --ch) {
    const int t0 = ch * chunk, t1 = min(T, t0 + chunk);
    // ---- recompute the states of this chunk, store the state BEFORE every token
    {
      float S[R];
      const float* src = ckpt + ((long long)bh * nchunks + ch) * D * D;
#pragma unroll
      for (int i = 0; i < R; ++i) S[i] = src[(i0 + i) * D + col];
      for (int s0 = t0; s0 < t1; s0 += EFLA_TT) {
        const int n = min(EFLA_TT, t1 - s0);
        efla_load_tile<D>(k, v, nullptr, sk, sv, nullptr, sc, nullptr, beta, (((long long)b * T + s0) * H + h) * D, (long long)H * D,
                          col, n, warp, lane);
        for (int r = 0; r < n; ++r) {
          float* dst = wk + (long long)(s0 + r - t0) * D * D;
#pragma unroll
          for (int i = 0; i < R; ++i) dst[i * D] = S[i];
          efla_step<R>(S, sk[r] + i0, sc[r], sv[r][lane], spart[r & 1], warp, lane);
        }
      }
    }
    // ---- reverse-time recursion over the chunk (sub-tiles of EFLA_TT tokens, last one first)
    const int ntiles = (t1 - t0 + EFLA_TT - 1) / EFLA_TT;
    for (int ti = ntiles - 1; ti >= 0; --ti) {
      const int s0 = t0 + ti * EFLA_TT, n = min(EFLA_TT, t1 - s0);
      efla_load_tile<D>(k, v, dout, sk, sv, sdo, sc, nullptr, beta, (((long long)b * T + s0) * H + h) * D, (long long)H * D, col, n,
                        warp, lane);
      for (int r = n - 1; r >= 0; --r) {
        const int t = s0 + r;
        const float* Sb = wk + (long long)(t - t0) * D * D;            // S before token t: element (i0 + i, col) at Sb[i * D]
        const float4* kr = reinterpret_cast<const float4*>(sk[r] + i0);
        const float c_ = sc[r], go = sdo[r][lane];
        // pass 1
        float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f, w0 = 0.f, w1 = 0.f, w2 = 0.f, w3 = 0.f;
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 kk = kr[i];
          p0 += kk.x * Sb[(4 * i) * D];
          p1 += kk.y * Sb[(4 * i + 1) * D];
          p2 += kk.z * Sb[(4 * i + 2) * D];
          p3 += kk.w * Sb[(4 * i + 3) * D];
          G[4 * i] += kk.x * go;
          G[4 * i + 1] += kk.y * go;
          G[4 * i + 2] += kk.z * go;
          G[4 * i + 3] += kk.w * go;
          w0 += G[4 * i] * kk.x;
          w1 += G[4 * i + 1] * kk.y;
          w2 += G[4 * i + 2] * kk.z;
          w3 += G[4 * i + 3] * kk.w;
        }
        float* part = spart[r & 1];
        part[warp * 32 + lane] = (p0 + p1) + (p2 + p3);
        part[EFLA_W * 32 + warp * 32 + lane] = (w0 + w1) + (w2 + w3);
        __syncthreads();
        const float p = (part[lane] + part[32 + lane]) + (part[64 + lane] + part[96 + lane]);
        const float w = (part[128 + lane] + part[160 + lane]) + (part[192 + lane] + part[224 + lane]);
        const float e = sv[r][lane] - p;
        const float de = c_ * w, dp = -de;
        const long long row = ((long long)b * T + t) * H + h;
        const float dc = warp_sum(e * w);
        if (warp == 0) {
          dv[row * D + col] = __float2bfloat16(de);
          if (lane == 0) dcp[row] = dc;
        }
        // pass 2
        const float ce = c_ * e;
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          const float4 kk = kr[i];
          const float kv[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int ii = 4 * i + u;
            const float sb = Sb[ii * D];
            sred[warp][ii][lane] = (sb + kv[u] * ce) * go + ce * G[ii] + sb * dp;
            G[ii] += kv[u] * dp;
          }
        }
        __syncwarp();
        if (lane < R) {
          float acc = 0.f;
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) acc += sred[warp][lane][jj];
          dkp[row * D + i0 + lane] = acc;
        }
        __syncwarp();
      }
    }
  }
  if (dstate0) {
#pragma unroll
    for (int i = 0; i < R; ++i) dstate0[((long long)bh * D + i0 + i) * D + col] = G[i];
  }
}

// dk = sum of the column blocks' partial rows + 2 k dc dc/dlam (bf16); dbeta_tok[row] = dc dc/dbeta. One warp per row.
__global__ void __launch_bounds__(256) efla_bwd_finish_kernel(const __nv_bfloat16* __restrict__ k, const float* __restrict__ beta_ptr,
                                                              const float* __restrict__ dk_part, const float* __restrict__ dc_part,
                                                              __nv_bfloat16* __restrict__ dk, float* __restrict__ dbeta_tok,
                                                              long long rows, int D, int nb) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float beta = *beta_ptr;
  float kx[4], lam = 0.f;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const int c = m * 32 + lane;
    kx[m] = c < D ? __bfloat162float(k[row * D + c]) : 0.f;
    lam += kx[m] * kx[m];
  }
  lam = warp_sum(lam);
  float dc = 0.f;
  for (int q = 0; q < nb; ++q) dc += dc_part[q * rows + row];
  float c_, dc_db, dc_dl;
  efla_coeff(beta, lam, c_, dc_db, dc_dl);
  const float dlam = dc * dc_dl;
#pragma unroll
  for (int m = 0; m < 4; ++m) {
    const int c = m * 32 + lane;
    if (c < D) {
      float acc = 0.f;
      for (int q = 0; q < nb; ++q) acc += dk_part[((long long)q * rows + row) * D + c];
      dk[row * D + c] = __float2bfloat16(acc + 2.f * kx[m] * dlam);
    }
  }
  if (lane == 0) dbeta_tok[row] = dc * dc_db;
}


// ------------------------------------------------------------------------------------ ShortConv
// Forward and input gradient share one kernel (DX = false: y[t] = bias + sum_j x[t - j] w[j]; DX = true:
// dx[t] = sum_j dy[t + j] w[j]). A lane owns a PAIR of adjacent channels (4-byte loads, 128 bytes per warp); the
// CTA's 64 channels x W weights sit transposed in shared memory (the [C, W] layout read directly would touch a
// different cache line in every lane); a warp walks SC_ROWS / 8 consecutive time steps, so the W - 1 re-reads of an
// input element come from L1. grid (ceil(B T / SC_ROWS), ceil(C / 64)), block (32, 8), dynamic smem W * 64 floats.
constexpr int SC_ROWS = 64;

template <bool DX>
__global__ void __launch_bounds__(256) shortconv_apply_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ w,
                                                              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                                              int B, int T, int C, int W) {
  extern __shared__ float sw[];                          // [W][64]
  const int lane = threadIdx.x, warp = threadIdx.y;
  const int c0 = blockIdx.y * 64;
  for (int i = warp * 32 + lane; i < W * 64; i += 256) {
    const int cl = i / W, j = i % W;                     // consecutive threads read consecutive weights of a channel
    sw[j * 64 + cl] = c0 + cl < C ? __bfloat162float(w[(long long)(c0 + cl) * W + j]) : 0.f;
  }
  __syncthreads();
  const int c = c0 + 2 * lane;
  if (c >= C) return;
  const long long rows = (long long)B * T;
  const long long r0 = (long long)blockIdx.x * SC_ROWS + warp * (SC_ROWS / 8);
  float b0 = 0.f, b1 = 0.f;
  if (!DX && bias) {
    b0 = __bfloat162float(bias[c]);
    b1 = __bfloat162float(bias[c + 1]);
  }
  for (long long r = r0; r < min(rows, r0 + SC_ROWS / 8); ++r) {
    const int t = (int)(r % T);
    const int taps = DX ? min(W, T - t) : min(W, t + 1);
    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(in + r * C + c);
    const long long step = DX ? (long long)(C / 2) : -(long long)(C / 2);
    float a0 = b0, a1 = b1;
#pragma unroll 4
    for (int j = 0; j < taps; ++j) {
      const float2 xv = __bfloat1622float2(src[j * step]);
      const float2 wv = *reinterpret_cast<const float2*>(sw + j * 64 + 2 * lane);
      a0 += xv.x * wv.x;
      a1 += xv.y * wv.y;
    }
    *reinterpret_cast<__nv_bfloat162*>(out + r * C + c) = __floats2bfloat162_rn(a0, a1);
  }
}

// dw[c,w] = sum_{b,t>=w} dy[b,t,c] x[b,t-w,c]; db[c] = sum dy. A CTA owns 32 channels (lane = channel) and SC_TAPS taps;
// its 32 warps stride over all B T rows (four rows in flight per warp), every row's dy is read once and multiplied with
// the SC_TAPS shifted inputs; the warps' partial sums are added in warp order (no atomics). grid (ceil(C / 32),
// ceil(W / SC_TAPS)), block (32, 32); the CTAs with blockIdx.y == 0 also produce the bias gradient.
constexpr int SC_TAPS = 4;

__global__ void __launch_bounds__(1024) shortconv_bwd_dw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                                                float* __restrict__ dw, float* __restrict__ db, int B, int T, int C,
                                                                int W) {
  __shared__ float sm[32][SC_TAPS + 1][33];
  const int lane = threadIdx.x, warp = threadIdx.y;
  const int c = blockIdx.x * 32 + lane;
  const int w0 = blockIdx.y * SC_TAPS;
  float acc[SC_TAPS], accb = 0.f;
#pragma unroll
  for (int u = 0; u < SC_TAPS; ++u) acc[u] = 0.f;
  if (c < C) {
    const long long rows = (long long)B * T;
#pragma unroll 4
    for (long long r = warp; r < rows; r += 32) {
      const int t = (int)(r % T);
      const float g = __bfloat162float(dy[r * C + c]);
      accb += g;
#pragma unroll
      for (int u = 0; u < SC_TAPS; ++u) {
        const int wj = w0 + u;
        if (wj < W && t >= wj) acc[u] += g * __bfloat162float(x[(r - wj) * C + c]);
      }
    }
  }
#pragma unroll
  for (int u = 0; u < SC_TAPS; ++u) sm[warp][u][lane] = acc[u];
  sm[warp][SC_TAPS][lane] = accb;
  __syncthreads();
  if (warp <= SC_TAPS && c < C) {                        // warp u adds up tap u, warp SC_TAPS the bias column
    float s = 0.f;
    for (int i = 0; i < 32; ++i) s += sm[i][warp][lane];
    if (warp == SC_TAPS) {
      if (db && blockIdx.y == 0) db[c] = s;
    } else if (w0 + warp < W) {
      dw[(long long)c * W + w0 + warp] = s;
    }
  }
}

template <int D>
int launch_efla_fwd(const void* k, const void* v, const float* beta, const float* state0, void* o, float* state_out, float* ckpt, int B,
                    int T, int H, int chunk, cudaStream_t s) {
  efla_scan_fwd_kernel<D><<<dim3(B * H, D / 32), 32 * EFLA_W, 0, s>>>(static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), beta, state0,
                                              static_cast<__nv_bfloat16*>(o), state_out, ckpt, T, H, chunk);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

template <int D>
int launch_efla_bwd(const void* k, const void* v, const float* beta, const float* ckpt, const void* dout, const float* dstate_out,
                    void* dk, void* dv, float* dbeta_tok, float* dstate0, float* work, float* dk_part, float* dc_part, int B, int T,
                    int H, int chunk, cudaStream_t s) {
  efla_scan_bwd_kernel<D><<<dim3(B * H, D / 32), 32 * EFLA_W, 0, s>>>(
      static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), beta, ckpt, static_cast<const __nv_bfloat16*>(dout),
      dstate_out, dk_part, static_cast<__nv_bfloat16*>(dv), dc_part, dstate0, work, B, T, H, chunk);
  ELFA_CUDA(cudaGetLastError());
  const long long rows = (long long)B * T * H;
  efla_bwd_finish_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(k), beta, dk_part, dc_part,
                                                                    static_cast<__nv_bfloat16*>(dk), dbeta_tok, rows, D, D / 32);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
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

// Gradients of elfa_efla_scan_fwd. dbeta_tok: [B*T*H] per-token terms (add them up); work: [B*H, chunk, d, d] fp32;
// dk_part: [d/32, B*T*H, d] fp32 and dc_part: [d/32, B*T*H] fp32 are scratch (one slice per block of 32 value columns).
ELFA_API int elfa_efla_scan_bwd(const void* k, const void* v, const float* beta, const float* ckpt, const void* dout,
                                const float* dstate_out, void* dk, void* dv, float* dbeta_tok, float* dstate0, float* work,
                                float* dk_part, float* dc_part, int B, int T, int H, int d, int chunk, void* stream) {
  ELFA_REQUIRE(k && v && beta && ckpt && dout && dk && dv && dbeta_tok && work && dk_part && dc_part && B > 0 && T > 0 && H > 0 &&
                   chunk > 0,
               "efla_scan_bwd: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (d) {
    case 32: return launch_efla_bwd<32>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta_tok, dstate0, work, dk_part, dc_part, B, T, H, chunk, s);
    case 64: return launch_efla_bwd<64>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta_tok, dstate0, work, dk_part, dc_part, B, T, H, chunk, s);
    case 96: return launch_efla_bwd<96>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta_tok, dstate0, work, dk_part, dc_part, B, T, H, chunk, s);
    case 128: return launch_efla_bwd<128>(k, v, beta, ckpt, dout, dstate_out, dk, dv, dbeta_tok, dstate0, work, dk_part, dc_part, B, T, H, chunk, s);
    default: set_last_error("efla_scan_bwd: head dimension must be 32, 64, 96 or 128"); return ELFA_ERR_UNSUPPORTED;
  }
}

ELFA_API int elfa_shortconv_fwd(const void* x, const void* w, const void* bias, void* y, int B, int T, int C, int W, void* stream) {
  ELFA_REQUIRE(x && w && y && B > 0 && T > 0 && C > 0 && W > 0, "shortconv_fwd: bad arguments");
  ELFA_REQUIRE(C % 2 == 0 && W <= 128, "shortconv_fwd: the channel count must be even and the window at most 128");
  const long long rows = (long long)B * T;
  dim3 grid((unsigned)((rows + SC_ROWS - 1) / SC_ROWS), (C + 63) / 64), block(32, 8);
  shortconv_apply_kernel<false><<<grid, block, (size_t)W * 64 * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
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
  ELFA_REQUIRE(C % 2 == 0 && W <= 128, "shortconv_bwd: the channel count must be even and the window at most 128");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * T;
  dim3 grid((unsigned)((rows + SC_ROWS - 1) / SC_ROWS), (C + 63) / 64), block(32, 8);
  shortconv_apply_kernel<true><<<grid, block, (size_t)W * 64 * sizeof(float), s>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(w), nullptr, static_cast<__nv_bfloat16*>(dx), B, T, C, W);
  dim3 grid2((C + 31) / 32, (W + SC_TAPS - 1) / SC_TAPS), block2(32, 32);
  shortconv_bwd_dw_kernel<<<grid2, block2, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), dw, db, B,
                                                   T, C, W);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
  return ELFA_OK;
}
