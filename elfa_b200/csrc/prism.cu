// PRISM iterative refinement, forward and backward, one kernel each.
//
// reference: src/model/prism.zig:318-421 (host loops over tokens, groups and iterations) and
// :488-871 (backward); kernels/cuda/include/kernels.h declares prism_forward_cuda but no source defines it.
//
//   r_0 = v - u                                   per group g of d channels
//   delta_l = gelu(p_l * r_l),  r_{l+1} = r_l - delta_l,  l = 0 .. L-1      (p_l [B,T,d] is shared by all groups)
//   y = u + sum_l delta_l
//
// One thread owns one (token, channel-in-group) pair and walks over the G groups, so the gradient of
// p_l (a sum over groups) is accumulated in registers: no atomics, deterministic. Consecutive
// threads touch consecutive channels: every access is coalesced. The backward recomputes r_l.
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

constexpr int PRISM_MAX_L = 8;

struct PrismPtrs {
  const __nv_bfloat16* p[PRISM_MAX_L];   // [tokens, d] each
  float* dp[PRISM_MAX_L];                // [tokens, d] fp32 each (backward)
};

__global__ void __launch_bounds__(256) prism_fwd_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ v,
                                                        PrismPtrs pp, __nv_bfloat16* __restrict__ y, long long tokens, int G, int d,
                                                        int L) {
  const long long n = tokens * d;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long t = i / d;
    const int c = (int)(i - t * d);
    float pl[PRISM_MAX_L];
    for (int l = 0; l < L; ++l) pl[l] = __bfloat162float(pp.p[l][t * d + c]);
    const long long base = t * (long long)G * d + c;
    for (int g = 0; g < G; ++g) {
      const float uu = __bfloat162float(u[base + (long long)g * d]);
      float r = __bfloat162float(v[base + (long long)g * d]) - uu;
      float refined = 0.f;
      for (int l = 0; l < L; ++l) {
        const float delta = gelu_tanh(pl[l] * r);
        r -= delta;
        refined += delta;
      }
      y[base + (long long)g * d] = __float2bfloat16(uu + refined);
    }
  }
}

__global__ void __launch_bounds__(256) prism_bwd_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ v,
                                                        PrismPtrs pp, const __nv_bfloat16* __restrict__ dy,
                                                        __nv_bfloat16* __restrict__ du, __nv_bfloat16* __restrict__ dv, long long tokens,
                                                        int G, int d, int L) {
  const long long n = tokens * d;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long t = i / d;
    const int c = (int)(i - t * d);
    float pl[PRISM_MAX_L], dpl[PRISM_MAX_L];
    for (int l = 0; l < L; ++l) {
      pl[l] = __bfloat162float(pp.p[l][t * d + c]);
      dpl[l] = 0.f;
    }
    const long long base = t * (long long)G * d + c;
    for (int g = 0; g < G; ++g) {
      const long long idx = base + (long long)g * d;
      const float uu = __bfloat162float(u[idx]);
      const float go = __bfloat162float(dy[idx]);
      float rl[PRISM_MAX_L];
      float r = __bfloat162float(v[idx]) - uu;
      for (int l = 0; l < L; ++l) {      // forward again: r_l
        rl[l] = r;
        r -= gelu_tanh(pl[l] * r);
      }
      float dr = 0.f;                    // gradient with respect to r_{l+1}
      for (int l = L - 1; l >= 0; --l) {
        const float z = pl[l] * rl[l];
        const float dz = (go - dr) * dgelu_tanh(z);
        dpl[l] += dz * rl[l];
        dr += dz * pl[l];
      }
      du[idx] = __float2bfloat16(go - dr);
      dv[idx] = __float2bfloat16(dr);
    }
    for (int l = 0; l < L; ++l) pp.dp[l][t * d + c] = dpl[l];
  }
}

int prism_grid(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b < 148 * 8 ? b : 148 * 8);
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// u, v, y: [tokens, G * d] bf16; p: host array of L device pointers to [tokens, d] bf16 (already sigmoid-ed).
ELFA_API int elfa_prism_fwd(const void* u, const void* v, const unsigned long long* p, void* y, long long tokens, int G, int d, int L,
                            void* stream) {
  ELFA_REQUIRE(u && v && p && y && tokens > 0 && G > 0 && d > 0 && L >= 1 && L <= PRISM_MAX_L, "prism_fwd: bad arguments");
  PrismPtrs pp{};
  for (int l = 0; l < L; ++l) pp.p[l] = reinterpret_cast<const __nv_bfloat16*>(p[l]);
  prism_fwd_kernel<<<prism_grid(tokens * d), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(u), static_cast<const __nv_bfloat16*>(v), pp, static_cast<__nv_bfloat16*>(y), tokens, G, d, L);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}

// du, dv: [tokens, G * d] bf16; dp: host array of L device pointers to [tokens, d] fp32.
ELFA_API int elfa_prism_bwd(const void* u, const void* v, const unsigned long long* p, const void* dy, void* du, void* dv,
                            const unsigned long long* dp, long long tokens, int G, int d, int L, void* stream) {
  ELFA_REQUIRE(u && v && p && dy && du && dv && dp && tokens > 0 && G > 0 && d > 0 && L >= 1 && L <= PRISM_MAX_L,
               "prism_bwd: bad arguments");
  PrismPtrs pp{};
  for (int l = 0; l < L; ++l) {
    pp.p[l] = reinterpret_cast<const __nv_bfloat16*>(p[l]);
    pp.dp[l] = reinterpret_cast<float*>(dp[l]);
  }
  prism_bwd_kernel<<<prism_grid(tokens * d), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(u), static_cast<const __nv_bfloat16*>(v), pp, static_cast<const __nv_bfloat16*>(dy),
      static_cast<__nv_bfloat16*>(du), static_cast<__nv_bfloat16*>(dv), tokens, G, d, L);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}
