// Vectorised bf16 elementwise kernels (8 elements per 128-bit access) and the embedding
// gather / scatter-add. GELU and its derivative normally run inside GEMM epilogues; these are
// the standalone forms.
//
// reference: kernels/cuda/activations.cu:22-45 (GELU fwd/bwd, SiLU), kernels/cuda/layernorm.cu:256-306
// (bf16 GELU), kernels/cuda/elementwise.cu:100-107 (multiply), kernels/cuda/init.cu:119-135 (fill, cast),
// src/nn/layers.zig:316-319 (GELU formulas), :459-501 (embedding forward / backward).
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

enum { OP_GELU = 0, OP_GELU_BWD = 1, OP_ADD = 2, OP_MUL = 3, OP_SILU = 4, OP_SILU_BWD = 5, OP_RELU = 6, OP_RELU_BWD = 7,
       OP_GELU_ERF = 8, OP_GELU_ERF_BWD = 9, OP_SCALE = 10 };

template <int OP>
__device__ __forceinline__ float apply(float a, float b, float alpha) {
  if (OP == OP_GELU) return gelu_tanh(a);
  if (OP == OP_GELU_BWD) return b * dgelu_tanh(a);  // a = pre-activation, b = upstream gradient
  if (OP == OP_ADD) return a + alpha * b;
  if (OP == OP_MUL) return a * b;
  if (OP == OP_SILU) return a / (1.f + __expf(-a));
  if (OP == OP_SILU_BWD) {
    const float s = 1.f / (1.f + __expf(-a));
    return b * s * (1.f + a * (1.f - s));
  }
  if (OP == OP_RELU) return fmaxf(a, 0.f);
  if (OP == OP_RELU_BWD) return a > 0.f ? b : 0.f;
  if (OP == OP_GELU_ERF) return 0.5f * a * (1.f + erff(a * 0.7071067811865476f));
  if (OP == OP_GELU_ERF_BWD) {
    const float cdf = 0.5f * (1.f + erff(a * 0.7071067811865476f));
    const float pdf = 0.3989422804014327f * __expf(-0.5f * a * a);
    return b * (cdf + a * pdf);
  }
  if (OP == OP_SCALE) return a * alpha;
  return a;
}

template <int OP, bool BINARY>
__global__ void __launch_bounds__(256) ew_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                                 __nv_bfloat16* __restrict__ out, long long n, float alpha) {
  const long long nvec = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  constexpr int U = 4;   // 16-byte loads in flight per thread and operand
  for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += U * stride) {
    uint4 av[U], bv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      av[u] = make_uint4(0, 0, 0, 0);
      bv[u] = make_uint4(0, 0, 0, 0);
      if (i < nvec) {
        av[u] = reinterpret_cast<const uint4*>(a)[i];
        if (BINARY) bv[u] = reinterpret_cast<const uint4*>(b)[i];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) {
        const uint32_t* pa = reinterpret_cast<const uint32_t*>(&av[u]);
        const uint32_t* pb = reinterpret_cast<const uint32_t*>(&bv[u]);
        uint4 o;
        uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          po[j] = pack_bf16(apply<OP>(bf16_lo(pa[j]), bf16_lo(pb[j]), alpha), apply<OP>(bf16_hi(pa[j]), bf16_hi(pb[j]), alpha));
        reinterpret_cast<uint4*>(out)[i] = o;
      }
    }
  }
  // tail (n not a multiple of 8)
  const long long tail0 = nvec * 8;
  for (long long i = tail0 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float bb = BINARY ? __bfloat162float(b[i]) : 0.f;
    out[i] = __float2bfloat16(apply<OP>(__bfloat162float(a[i]), bb, alpha));
  }
}

// out[t, :] = tok_emb[ids[t], :] (+ pos_emb[pos0 + (t / pos_div) % seq, :]); pos_div = 1 for [B, S] ids, B for [S, B] ids
__global__ void __launch_bounds__(256) embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ tok,
                                                            const __nv_bfloat16* __restrict__ pos, __nv_bfloat16* __restrict__ out,
                                                            int tokens, int D, int seq, int pos_div, int pos0, int vocab_lo, int vocab_hi,
                                                            int vocab_total, unsigned int* status) {
  const int nvec = D / 8;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const long long id = ids[t];
    const bool mine = id >= vocab_lo && id < vocab_hi;
    if (threadIdx.x == 0 && (id < 0 || id >= vocab_total)) atomicOr(status, (unsigned)ELFA_ST_BAD_TARGET);
    const uint4* tr = reinterpret_cast<const uint4*>(tok + (long long)(mine ? id - vocab_lo : 0) * D);
    const uint4* pr = pos ? reinterpret_cast<const uint4*>(pos + (long long)(pos0 + (t / pos_div) % seq) * D) : nullptr;
    uint4* orow = reinterpret_cast<uint4*>(out + (long long)t * D);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      uint4 a = mine ? tr[v] : make_uint4(0, 0, 0, 0);
      if (pr && (vocab_lo == 0)) {  // the rank that owns vocabulary slice 0 adds the positions
        const uint4 b = pr[v];
        uint32_t* pa = reinterpret_cast<uint32_t*>(&a);
        const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
        for (int j = 0; j < 4; ++j) pa[j] = pack_bf16(bf16_lo(pa[j]) + bf16_lo(pb[j]), bf16_hi(pa[j]) + bf16_hi(pb[j]));
      }
      orow[v] = a;
    }
  }
}

// dtok[ids[t], :] += dy[t, :] (atomics); dpos[pos0 + (t / pos_div) % seq, :] += dy[t, :]
template <typename GradT>
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                                            GradT* __restrict__ dtok, GradT* __restrict__ dpos, int tokens, int D,
                                                            int seq, int pos_div, int pos0, int vocab_lo, int vocab_hi) {
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    const long long id = ids[t];
    const bool mine = id >= vocab_lo && id < vocab_hi;
    const __nv_bfloat16* g = dy + (long long)t * D;
    GradT* tr = dtok + (long long)(mine ? id - vocab_lo : 0) * D;
    GradT* pr = (dpos && vocab_lo == 0) ? dpos + (long long)(pos0 + (t / pos_div) % seq) * D : nullptr;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const float v = __bfloat162float(g[c]);
      if (mine) atomicAdd(tr + c, (GradT)v);
      if (pr) atomicAdd(pr + c, (GradT)v);
    }
  }
}

template <typename SrcT, typename DstT>
__global__ void __launch_bounds__(256) cast_kernel(const SrcT* __restrict__ src, DstT* __restrict__ dst, long long n, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = (DstT)((float)src[i] * scale);
}

inline int ew_grid(long long n) {
  long long b = (n / 8 + 255) / 256;
  if (b < 1) b = 1;
  return (int)(b > 148 * 8 ? 148 * 8 : b);
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// op: 0 gelu(a) | 1 b*gelu'(a) | 2 a+alpha*b | 3 a*b | 4 silu(a) | 5 b*silu'(a) | 6 relu | 7 relu' | 8 gelu_erf | 9 gelu_erf' | 10 a*alpha
ELFA_API int elfa_elementwise(int op, const void* a, const void* b, void* out, long long n, float alpha, void* stream) {
  ELFA_REQUIRE(a && out && n > 0, "elementwise: null pointer or empty");
  const bool binary = (op == OP_GELU_BWD || op == OP_ADD || op == OP_MUL || op == OP_SILU_BWD || op == OP_RELU_BWD || op == OP_GELU_ERF_BWD);
  ELFA_REQUIRE(!binary || b, "elementwise: binary op needs b");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto* A = static_cast<const __nv_bfloat16*>(a);
  const auto* B = static_cast<const __nv_bfloat16*>(b);
  auto* O = static_cast<__nv_bfloat16*>(out);
  const int g = ew_grid(n);
  switch (op) {
    case OP_GELU: ew_kernel<OP_GELU, false><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_GELU_BWD: ew_kernel<OP_GELU_BWD, true><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_ADD: ew_kernel<OP_ADD, true><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_MUL: ew_kernel<OP_MUL, true><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_SILU: ew_kernel<OP_SILU, false><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_SILU_BWD: ew_kernel<OP_SILU_BWD, true><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_RELU: ew_kernel<OP_RELU, false><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_RELU_BWD: ew_kernel<OP_RELU_BWD, true><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_GELU_ERF: ew_kernel<OP_GELU_ERF, false><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_GELU_ERF_BWD: ew_kernel<OP_GELU_ERF_BWD, true><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    case OP_SCALE: ew_kernel<OP_SCALE, false><<<g, 256, 0, s>>>(A, B, O, n, alpha); break;
    default: set_last_error("elementwise: unknown op"); return ELFA_ERR_ARG;
  }
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Token (+ learned position) embedding. Only ids in [vocab_lo, vocab_hi) are looked up (rows of
// `tok` are local to that slice); other tokens give zeros, so a sum over vocabulary-parallel ranks
// rebuilds the full embedding. Positions are added by the rank with vocab_lo == 0.
ELFA_API int elfa_embedding_fwd(const long long* ids, const void* tok, const void* pos, void* out, int tokens, int D, int seq,
                                int pos_div, int pos0, int vocab_lo, int vocab_hi, int vocab_total, void* stream) {
  ELFA_REQUIRE(ids && tok && out && tokens > 0 && D % 8 == 0 && seq > 0 && pos_div > 0, "embedding_fwd: bad arguments");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "embedding_fwd: no status word");
  const int grid = tokens < 148 * 16 ? tokens : 148 * 16;
  const int threads = D / 8 >= 256 ? 256 : (D / 8 >= 128 ? 128 : 64);
  embedding_fwd_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(tok), static_cast<const __nv_bfloat16*>(pos), static_cast<__nv_bfloat16*>(out), tokens,
      D, seq, pos_div, pos0, vocab_lo, vocab_hi, vocab_total, st);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Scatter-add of dy into fp32 (grads_f32 = 1) or bf16 gradient tables.
ELFA_API int elfa_embedding_bwd(const long long* ids, const void* dy, void* dtok, void* dpos, int tokens, int D, int seq, int pos_div, int pos0,
                                int vocab_lo, int vocab_hi, int grads_f32, void* stream) {
  ELFA_REQUIRE(ids && dy && dtok && tokens > 0 && seq > 0 && pos_div > 0, "embedding_bwd: bad arguments");
  const int grid = tokens < 148 * 16 ? tokens : 148 * 16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (grads_f32)
    embedding_bwd_kernel<float><<<grid, 256, 0, s>>>(ids, static_cast<const __nv_bfloat16*>(dy), static_cast<float*>(dtok),
                                                     static_cast<float*>(dpos), tokens, D, seq, pos_div, pos0, vocab_lo, vocab_hi);
  else
    embedding_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(ids, static_cast<const __nv_bfloat16*>(dy),
                                                             static_cast<__nv_bfloat16*>(dtok), static_cast<__nv_bfloat16*>(dpos),
                                                             tokens, D, seq, pos_div, pos0, vocab_lo, vocab_hi);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// dst = (dst_type) (src * scale); types: 0 = fp32, 1 = bf16.
ELFA_API int elfa_cast(const void* src, int src_type, void* dst, int dst_type, long long n, float scale, void* stream) {
  ELFA_REQUIRE(src && dst && n > 0, "cast: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long b = (n + 255) / 256;
  const int g = (int)(b > 148 * 16 ? 148 * 16 : b);
  if (src_type == 0 && dst_type == 1)
    cast_kernel<float, __nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const float*>(src), static_cast<__nv_bfloat16*>(dst), n, scale);
  else if (src_type == 1 && dst_type == 0)
    cast_kernel<__nv_bfloat16, float><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), static_cast<float*>(dst), n, scale);
  else if (src_type == 0 && dst_type == 0)
    cast_kernel<float, float><<<g, 256, 0, s>>>(static_cast<const float*>(src), static_cast<float*>(dst), n, scale);
  else if (src_type == 1 && dst_type == 1)
    cast_kernel<__nv_bfloat16, __nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), n, scale);
  else {
    set_last_error("cast: unknown type");
    return ELFA_ERR_ARG;
  }
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// ---- row softmax ------------------------------------------------------------------------------------
// reference: kernels/cuda/layernorm.cu softmax kernel and src/nn/nn_kernels.zig:226-267 (host loop).
// One warp per row, two passes over the row held in registers when it fits (<= 4096 columns), else
// three passes over global memory. out = softmax(x * scale) in bf16.
namespace elfa {
namespace {

__global__ void __launch_bounds__(256) softmax_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                           long long rows, int cols, long long ldx, long long ldo, float scale) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + row * ldx;
  __nv_bfloat16* orow = out + row * ldo;
  const float s2 = scale * 1.4426950408889634f;
  float mx = -INFINITY;
  for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, __bfloat162float(xr[c]));
  mx = warp_max(mx);
  const float m2 = mx == -INFINITY ? 0.f : mx * s2;
  float sum = 0.f;
  for (int c = lane; c < cols; c += 32) sum += fast_exp2(__bfloat162float(xr[c]) * s2 - m2);
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  for (int c = lane; c < cols; c += 32) orow[c] = __float2bfloat16(fast_exp2(__bfloat162float(xr[c]) * s2 - m2) * inv);
}

}  // namespace
}  // namespace elfa

ELFA_API int elfa_softmax_rows(const void* x, void* out, long long rows, int cols, long long ldx, long long ldo, float scale,
                               void* stream) {
  ELFA_REQUIRE(x && out && rows > 0 && cols > 0 && scale > 0.f, "softmax_rows: bad arguments");
  const long long blocks = (rows + 7) / 8;
  ELFA_REQUIRE(blocks < (1ll << 31), "softmax_rows: too many rows");
  elfa::softmax_rows_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), rows, cols, ldx, ldo, scale);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}
