// Optimizer kernels over flat parameter buffers: AdamW and Lion with fp32 master weights and
// moments and a bf16 (or fp32) working copy written in the same pass, the global gradient-norm
// reduction, the clip coefficient / non-finite guard computed on the device (no host sync in the
// step), and the Muon helpers (momentum, Frobenius normalisation, 3I - G, apply).
//
// reference: src/kernels/optim_kernels.zig:102-167 (Lion, AdamW math), :214-250 (norm, clip);
// src/optim/optimizer.zig:111-143 (Lion), :246-320 (Muon + Newton-Schulz), :547-593 (clipping);
// kernels/cuda/optim.cu:125-177 (bf16 Lion / AdamW kernels), :187-216 (sum of squares, clip),
// :218-290 (Gram / update kernels of Newton-Schulz, here done by the tcgen05 GEMM).
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

struct StepScalars {   // device-resident scalars shared by the kernels of one optimizer step
  float sumsq;         // accumulated by sumsq kernels
  float clip_coef;     // min(1, max_norm / norm) * inv_loss_scale
  float grad_norm;     // unscaled global gradient norm (for telemetry)
  int skip;            // 1 if the norm is not finite -> every update kernel leaves state untouched
  float lr;            // learning rate of this step, read by the Lion / Muon kernels when their `lr` argument is negative:
                       // a captured CUDA graph of the update then follows the schedule without being captured again
};

__device__ __forceinline__ float sumsq16(const uint4& v, float) {
  const float4 f = *reinterpret_cast<const float4*>(&v);
  return f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
}
__device__ __forceinline__ float sumsq16(const uint4& v, __nv_bfloat16) {
  const uint32_t* p = reinterpret_cast<const uint32_t*>(&v);
  float a = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) a += bf16_lo(p[j]) * bf16_lo(p[j]) + bf16_hi(p[j]) * bf16_hi(p[j]);
  return a;
}

// part[block] = sum of squares of this block's share. The 16-byte aligned body is read as vectors, four
// loads in flight per thread; the unaligned head and the tail are read element by element.
template <typename GradT>
__global__ void __launch_bounds__(256) sumsq_kernel(const GradT* __restrict__ g, long long n, float* __restrict__ part) {
  __shared__ float sm[8];
  constexpr int E = 16 / (int)sizeof(GradT);
  long long head = (long long)(((16 - (reinterpret_cast<uintptr_t>(g) & 15)) & 15) / sizeof(GradT));
  if (head > n) head = n;
  const long long nvec = (n - head) / E;
  const uint4* gv = reinterpret_cast<const uint4*>(g + head);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float acc = 0.f;
  for (long long i0 = tid; i0 < nvec; i0 += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      v[u] = make_uint4(0, 0, 0, 0);
      if (i0 + u * stride < nvec) v[u] = gv[i0 + u * stride];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) acc += sumsq16(v[u], GradT());
  }
  for (long long i = tid; i < head; i += stride) {
    const float v = (float)g[i];
    acc += v * v;
  }
  for (long long i = head + nvec * E + tid; i < n; i += stride) {
    const float v = (float)g[i];
    acc += v * v;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += sm[i];
    part[blockIdx.x] = s;
  }
}

// scal->sumsq (+)= sum(part[0..P)) in a fixed order.
__global__ void sumsq_finish_kernel(const float* __restrict__ part, int P, StepScalars* scal, int accumulate) {
  __shared__ float sm[256];
  float a = 0.f;
  for (int i = threadIdx.x; i < P; i += 256) a += part[i];
  sm[threadIdx.x] = a;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) scal->sumsq = (accumulate ? scal->sumsq : 0.f) + sm[0];
}

// Turns sumsq into the clip coefficient. inv_scale = 1 / loss_scale.
__global__ void clip_coef_kernel(StepScalars* scal, float max_norm, float inv_scale, unsigned int* status) {
  const float norm = sqrtf(scal->sumsq) * inv_scale;
  scal->grad_norm = norm;
  if (!isfinite(norm)) {
    scal->skip = 1;
    scal->clip_coef = 0.f;
    atomicOr(status, (unsigned)ELFA_ST_NONFINITE);
    return;
  }
  scal->skip = 0;
  float c = 1.f;
  if (max_norm > 0.f && norm > max_norm && norm > 1e-8f) c = max_norm / norm;
  scal->clip_coef = c * inv_scale;
}

__device__ __forceinline__ void load4(const float* p, float (&o)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&o)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  o[0] = bf16_lo(v.x); o[1] = bf16_hi(v.x); o[2] = bf16_lo(v.y); o[3] = bf16_hi(v.y);
}
__device__ __forceinline__ void store4(float* p, const float (&o)[4]) { *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]); }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&o)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]));
}

__device__ __forceinline__ void adamw_update(float& p, float& mi, float& vi, float g, float lr, float beta1, float beta2, float eps,
                                             float wd, float inv_bc1, float inv_bc2) {
  mi = beta1 * mi + (1.f - beta1) * g;
  vi = beta2 * vi + (1.f - beta2) * g * g;
  const float mh = mi * inv_bc1, vh = vi * inv_bc2;
  p -= lr * (mh / (sqrtf(vh) + eps) + wd * p);
}

// VEC = 4: every pointer is aligned for 4-element accesses and `n` counts groups of four; VEC = 1: element by element.
template <typename GradT, typename ParamT, int VEC>
__global__ void __launch_bounds__(256) adamw_kernel(ParamT* __restrict__ param, float* __restrict__ master, float* __restrict__ m,
                                                    float* __restrict__ v, const GradT* __restrict__ grad, long long n, float lr,
                                                    float beta1, float beta2, float eps, float wd, float inv_bc1, float inv_bc2,
                                                    const StepScalars* __restrict__ scal) {
  float gscale = 1.f;
  if (scal) {
    if (scal->skip) return;
    gscale = scal->clip_coef;
  }
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (VEC == 4) {
      float g[4], p[4], mm[4], vv[4];
      load4(grad + 4 * i, g);
      load4(master + 4 * i, p);
      load4(m + 4 * i, mm);
      load4(v + 4 * i, vv);
#pragma unroll
      for (int j = 0; j < 4; ++j) adamw_update(p[j], mm[j], vv[j], g[j] * gscale, lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2);
      store4(m + 4 * i, mm);
      store4(v + 4 * i, vv);
      store4(master + 4 * i, p);
      if (param) store4(param + 4 * i, p);
    } else {
      float p = master[i], mi = m[i], vi = v[i];
      adamw_update(p, mi, vi, (float)grad[i] * gscale, lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2);
      m[i] = mi;
      v[i] = vi;
      master[i] = p;
      if (param) param[i] = (ParamT)p;
    }
  }
}

template <typename GradT, typename ParamT>
__global__ void __launch_bounds__(256) lion_kernel(ParamT* __restrict__ param, float* __restrict__ master, float* __restrict__ m,
                                                   const GradT* __restrict__ grad, long long n, float lr, float beta1, float beta2,
                                                   float wd, const StepScalars* __restrict__ scal) {
  float gscale = 1.f;
  if (scal) {
    if (scal->skip) return;
    gscale = scal->clip_coef;
    if (lr < 0.f) lr = scal->lr;
  }
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float g = (float)grad[i] * gscale;
    float p = master[i];
    const float mi = m[i];
    const float u = beta1 * mi + (1.f - beta1) * g;
    const float sgn = u > 0.f ? 1.f : (u < 0.f ? -1.f : 0.f);
    p = p * (1.f - lr * wd) - lr * sgn;
    m[i] = beta2 * mi + (1.f - beta2) * g;
    master[i] = p;
    if (param) param[i] = (ParamT)p;
  }
}

// Muon: m = beta * m + g * gscale (fp32), y = bf16(m) and the partial sums of m^2.
template <typename GradT>
__global__ void __launch_bounds__(256) muon_momentum_kernel(float* __restrict__ m, const GradT* __restrict__ grad,
                                                            __nv_bfloat16* __restrict__ y, long long n, float beta,
                                                            const StepScalars* __restrict__ scal, float* __restrict__ part) {
  __shared__ float sm[8];
  float gscale = 1.f;
  bool skip = false;
  if (scal) { skip = scal->skip != 0; gscale = scal->clip_coef; }
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float mi = m[i];
    if (!skip) {
      mi = beta * mi + (float)grad[i] * gscale;
      m[i] = mi;
    }
    y[i] = __float2bfloat16(mi);
    acc += mi * mi;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += sm[i];
    part[blockIdx.x] = s;
  }
}

// y *= 1 / max(||m||_F, tiny) where ||m||^2 = sum(part[0..P)); norm_out[0] = ||m||_F.
__global__ void __launch_bounds__(256) muon_normalize_kernel(__nv_bfloat16* __restrict__ y, long long n, const float* __restrict__ part,
                                                             int P, float* __restrict__ norm_out) {
  __shared__ float s_inv;
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < P; ++i) s += part[i];
    const float nrm = sqrtf(s);
    if (blockIdx.x == 0 && norm_out) norm_out[0] = nrm;
    s_inv = nrm > 1e-8f ? 1.f / nrm : 1.f;
  }
  __syncthreads();
  const float inv = s_inv;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16(__bfloat162float(y[i]) * inv);
}

// G <- 3I - G for a square bf16 matrix [d, d].
__global__ void three_i_minus_kernel(__nv_bfloat16* __restrict__ g, int d) {
  const long long n = (long long)d * d;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int r = (int)(i / d), c = (int)(i % d);
    g[i] = __float2bfloat16((r == c ? 3.f : 0.f) - __bfloat162float(g[i]));
  }
}

// master -= lr * y ; param = cast(master)
template <typename ParamT>
__global__ void __launch_bounds__(256) muon_apply_kernel(ParamT* __restrict__ param, float* __restrict__ master,
                                                         const __nv_bfloat16* __restrict__ y, long long n, float lr,
                                                         const StepScalars* __restrict__ scal) {
  if (scal && scal->skip) return;
  if (scal && lr < 0.f) lr = scal->lr;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float p = master[i] - lr * __bfloat162float(y[i]);
    master[i] = p;
    if (param) param[i] = (ParamT)p;
  }
}

inline int flat_grid(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b > 148 * 8 ? 148 * 8 : (b < 1 ? 1 : b));
}

}  // namespace
}  // namespace elfa

using namespace elfa;

#define ELFA_SUMSQ_MAX_PART 1184

// scalars: 4 x 4 bytes {sumsq, clip_coef, grad_norm, skip}. part: >= 1184 floats of scratch.
// grad_type: 0 fp32, 1 bf16. accumulate: add to scalars->sumsq instead of overwriting it.
ELFA_API int elfa_sumsq(const void* grad, int grad_type, long long n, float* part, void* scalars, int accumulate, void* stream) {
  ELFA_REQUIRE(grad && part && scalars && n > 0, "sumsq: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = flat_grid(n);
  if (grad_type == 0) sumsq_kernel<float><<<g, 256, 0, s>>>(static_cast<const float*>(grad), n, part);
  else sumsq_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(grad), n, part);
  sumsq_finish_kernel<<<1, 256, 0, s>>>(part, g, static_cast<StepScalars*>(scalars), accumulate);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
  return ELFA_OK;
}

ELFA_API int elfa_clip_coef(void* scalars, float max_norm, float inv_loss_scale, void* stream) {
  ELFA_REQUIRE(scalars, "clip_coef: null scalars");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "clip_coef: no status word");
  clip_coef_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<StepScalars*>(scalars), max_norm, inv_loss_scale, st);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// param (bf16 if param_type == 1, fp32 if 0, may be null) / master, m, v fp32 / grad per grad_type.
// step >= 1. scalars may be null (no clipping, never skipped).
ELFA_API int elfa_adamw(void* param, int param_type, float* master, float* m, float* v, const void* grad, int grad_type, long long n,
                        float lr, float beta1, float beta2, float eps, float wd, int step, const void* scalars, void* stream) {
  ELFA_REQUIRE(master && m && v && grad && n > 0 && step >= 1, "adamw: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float inv_bc1 = 1.f / (1.f - powf(beta1, (float)step)), inv_bc2 = 1.f / (1.f - powf(beta2, (float)step));
  const auto* sc = static_cast<const StepScalars*>(scalars);
  const size_t gsz = grad_type == 0 ? 4 : 2, psz = param_type == 0 ? 4 : 2;
  auto aligned = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
  const bool vec = n >= 4 && aligned(master, 16) && aligned(m, 16) && aligned(v, 16) && aligned(grad, 4 * gsz) &&
                   (!param || aligned(param, 4 * psz));
  const long long body = vec ? n / 4 * 4 : 0, tail = n - body;
#define ADAMW(GT, PT)                                                                                                            \
  do {                                                                                                                           \
    if (body)                                                                                                                    \
      adamw_kernel<GT, PT, 4><<<flat_grid(body / 4), 256, 0, s>>>(static_cast<PT*>(param), master, m, v,                          \
                                                                  static_cast<const GT*>(grad), body / 4, lr, beta1, beta2, eps, \
                                                                  wd, inv_bc1, inv_bc2, sc);                                     \
    if (tail)                                                                                                                    \
      adamw_kernel<GT, PT, 1><<<flat_grid(tail), 256, 0, s>>>(param ? static_cast<PT*>(param) + body : nullptr, master + body,   \
                                                              m + body, v + body, static_cast<const GT*>(grad) + body, tail, lr, \
                                                              beta1, beta2, eps, wd, inv_bc1, inv_bc2, sc);                      \
  } while (0)
  if (grad_type == 0 && param_type == 0) ADAMW(float, float);
  else if (grad_type == 0) ADAMW(float, __nv_bfloat16);
  else if (param_type == 0) ADAMW(__nv_bfloat16, float);
  else ADAMW(__nv_bfloat16, __nv_bfloat16);
#undef ADAMW
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

ELFA_API int elfa_lion(void* param, int param_type, float* master, float* m, const void* grad, int grad_type, long long n, float lr,
                       float beta1, float beta2, float wd, const void* scalars, void* stream) {
  ELFA_REQUIRE(master && m && grad && n > 0, "lion: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = flat_grid(n);
  const auto* sc = static_cast<const StepScalars*>(scalars);
#define LION(GT, PT) lion_kernel<GT, PT><<<g, 256, 0, s>>>(static_cast<PT*>(param), master, m, static_cast<const GT*>(grad), n, lr, beta1, beta2, wd, sc)
  if (grad_type == 0 && param_type == 0) LION(float, float);
  else if (grad_type == 0) LION(float, __nv_bfloat16);
  else if (param_type == 0) LION(__nv_bfloat16, float);
  else LION(__nv_bfloat16, __nv_bfloat16);
#undef LION
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Muon step 1: m = beta*m + g; y = bf16(m) / ||m||_F. part: >= 1184 floats. norm_out: 1 float.
ELFA_API int elfa_muon_momentum(float* m, const void* grad, int grad_type, void* y, long long n, float beta, const void* scalars,
                                float* part, float* norm_out, void* stream) {
  ELFA_REQUIRE(m && grad && y && part && n > 0, "muon_momentum: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = flat_grid(n);
  const auto* sc = static_cast<const StepScalars*>(scalars);
  if (grad_type == 0) muon_momentum_kernel<float><<<g, 256, 0, s>>>(m, static_cast<const float*>(grad), static_cast<__nv_bfloat16*>(y), n, beta, sc, part);
  else muon_momentum_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(m, static_cast<const __nv_bfloat16*>(grad), static_cast<__nv_bfloat16*>(y), n, beta, sc, part);
  muon_normalize_kernel<<<g, 256, 0, s>>>(static_cast<__nv_bfloat16*>(y), n, part, g, norm_out);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
  return ELFA_OK;
}

ELFA_API int elfa_three_i_minus(void* g, int d, void* stream) {
  ELFA_REQUIRE(g && d > 0, "three_i_minus: bad arguments");
  three_i_minus_kernel<<<flat_grid((long long)d * d), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(g), d);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

ELFA_API int elfa_muon_apply(void* param, int param_type, float* master, const void* y, long long n, float lr, const void* scalars,
                             void* stream) {
  ELFA_REQUIRE(master && y && n > 0, "muon_apply: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = flat_grid(n);
  const auto* sc = static_cast<const StepScalars*>(scalars);
  if (param_type == 0) muon_apply_kernel<float><<<g, 256, 0, s>>>(static_cast<float*>(param), master, static_cast<const __nv_bfloat16*>(y), n, lr, sc);
  else muon_apply_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<__nv_bfloat16*>(param), master, static_cast<const __nv_bfloat16*>(y), n, lr, sc);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}
