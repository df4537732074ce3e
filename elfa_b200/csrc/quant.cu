// Quantisation kernels: block-scaled MXFP8 (e4m3 values, one ue8m0 scale per 32 elements) and
// NVFP4 (e2m1 values, one e4m3 scale per 16 elements plus an fp32 tensor scale), per-tensor FP8
// with a caller-owned scale, integer affine fake-quant with surrogate gradients, and abs-max.
// "Fake-quant" kernels write the dequantised value back in bf16 (quantisation-aware training);
// the "quantize" kernels emit the packed payload + scales for block-scaled tensor-core GEMMs.
//
// reference: src/tensor/dtype.zig:85-190 (ScaleFactor with amax history, BlockScale), :192-303 (e4m3
// codec, saturating), :587-642 (e2m1 codec); src/quantization/stable_qat.zig:52-130 (affine
// fake-quant and its surrogate gradients); kernels/cuda/elementwise.cu:303-319,457-488 (per-tensor
// fp8 quant / dequant and CUB abs-max); src/ptx/tcgen05_kernels.ptx:183,482 (the quantize_mxfp8 and
// stable_qat stubs these kernels make real).
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

__device__ __forceinline__ float e4m3_rt(float x) {  // round-trip through e4m3 (RNE, saturating)
  const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E4M3)));
}
__device__ __forceinline__ float e5m2_rt(float x) {
  const __nv_fp8_storage_t q = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E5M2);
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(q, __NV_E5M2)));
}
__device__ __forceinline__ float e2m1_rt(float x) {
  const __nv_fp4_storage_t q = __nv_cvt_float_to_fp4(x, __NV_E2M1, cudaRoundNearest);
  return __half2float(__half(__nv_cvt_fp4_to_halfraw(q, __NV_E2M1)));
}

// MX shared exponent for a block with abs-max `amax`: floor(log2(amax)) - emax(e4m3 = 8),
// clamped to the ue8m0 range. Returns the biased byte; *scale = 2^e, *inv = 2^-e.
__device__ __forceinline__ uint8_t mx_scale(float amax, float* scale, float* inv) {
  int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 - 8;
  if (amax == 0.f) e = -127;
  e = max(-127, min(127, e));
  *scale = __uint_as_float((uint32_t)(e + 127) << 23);
  if (e == -127) *scale = 5.877471754111438e-39f;  // 2^-127 (subnormal fp32)
  *inv = e == -127 ? 1.7014118346046923e38f : __uint_as_float((uint32_t)(127 - e) << 23);
  return (uint8_t)(e + 127);
}

// ---- blocks along the contiguous dimension -------------------------------------------------------
// One thread per 32-element block (64 bytes). fake: out bf16. real: payload e4m3 + scales [rows, cols/32].
template <bool FAKE>
__global__ void __launch_bounds__(256) mxfp8_rowwise_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                            uint8_t* __restrict__ payload, uint8_t* __restrict__ scales,
                                                            long long nblocks) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long blk = (long long)blockIdx.x * blockDim.x + threadIdx.x; blk < nblocks; blk += stride) {
    const uint4* src = reinterpret_cast<const uint4*>(x + blk * 32);
    uint4 v[4];
    float f[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = src[i];
      const uint32_t* pv = reinterpret_cast<const uint32_t*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[i * 8 + 2 * j] = bf16_lo(pv[j]);
        f[i * 8 + 2 * j + 1] = bf16_hi(pv[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f[i * 8 + 2 * j]), fabsf(f[i * 8 + 2 * j + 1])));
      }
    }
    float sc, inv;
    const uint8_t sb = mx_scale(amax, &sc, &inv);
    if (FAKE) {
      uint4* dst = reinterpret_cast<uint4*>(out + blk * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint4 o;
        uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) po[j] = pack_bf16(e4m3_rt(f[i * 8 + 2 * j] * inv) * sc, e4m3_rt(f[i * 8 + 2 * j + 1] * inv) * sc);
        dst[i] = o;
      }
    } else {
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t acc = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc |= (uint32_t)__nv_cvt_float_to_fp8(f[i * 4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
        w[i] = acc;
      }
      uint4* dst = reinterpret_cast<uint4*>(payload + blk * 32);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
      scales[blk] = sb;
    }
  }
}

// ---- blocks along dim 0 (the contraction dimension of an [in, out] weight) ---------------------------
// thread = one column of one 32-row group; a warp covers 32 adjacent columns (coalesced).
__global__ void __launch_bounds__(256) mxfp8_colwise_fake_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                 int rows, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r0 = blockIdx.y * 32;
  if (c >= cols) return;
  float f[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    f[i] = r0 + i < rows ? __bfloat162float(x[(long long)(r0 + i) * cols + c]) : 0.f;
    amax = fmaxf(amax, fabsf(f[i]));
  }
  float sc, inv;
  mx_scale(amax, &sc, &inv);
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (r0 + i < rows) out[(long long)(r0 + i) * cols + c] = __float2bfloat16(e4m3_rt(f[i] * inv) * sc);
}

// NVFP4 fake-quant, 16-element blocks along the contiguous dim. tensor_scale = amax_tensor / (448 * 6).
__global__ void __launch_bounds__(256) nvfp4_rowwise_fake_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                 long long nblocks, const float* __restrict__ tensor_amax) {
  const float ta = *tensor_amax;
  const float ts = ta > 0.f ? ta / (448.f * 6.f) : 1.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long blk = (long long)blockIdx.x * blockDim.x + threadIdx.x; blk < nblocks; blk += stride) {
    const uint4* src = reinterpret_cast<const uint4*>(x + blk * 16);
    float f[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 v = src[i];
      const uint32_t* pv = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[i * 8 + 2 * j] = bf16_lo(pv[j]);
        f[i * 8 + 2 * j + 1] = bf16_hi(pv[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f[i * 8 + 2 * j]), fabsf(f[i * 8 + 2 * j + 1])));
      }
    }
    const float sb = e4m3_rt(amax / (6.f * ts));   // block scale in e4m3 (non-negative)
    const float full = sb * ts;
    const float inv = full > 0.f ? 1.f / full : 0.f;
    uint4* dst = reinterpret_cast<uint4*>(out + blk * 16);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 o;
      uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) po[j] = pack_bf16(e2m1_rt(f[i * 8 + 2 * j] * inv) * full, e2m1_rt(f[i * 8 + 2 * j + 1] * inv) * full);
      dst[i] = o;
    }
  }
}

__global__ void __launch_bounds__(256) nvfp4_colwise_fake_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                 int rows, int cols, const float* __restrict__ tensor_amax) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r0 = blockIdx.y * 16;
  if (c >= cols) return;
  const float ta = *tensor_amax;
  const float ts = ta > 0.f ? ta / (448.f * 6.f) : 1.f;
  float f[16];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    f[i] = r0 + i < rows ? __bfloat162float(x[(long long)(r0 + i) * cols + c]) : 0.f;
    amax = fmaxf(amax, fabsf(f[i]));
  }
  const float sb = e4m3_rt(amax / (6.f * ts));
  const float full = sb * ts;
  const float inv = full > 0.f ? 1.f / full : 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    if (r0 + i < rows) out[(long long)(r0 + i) * cols + c] = __float2bfloat16(e2m1_rt(f[i] * inv) * full);
}

// abs-max of a bf16 tensor into *out (float, must be >= 0 before the call; bitwise max is valid for
// non-negative floats).
__global__ void __launch_bounds__(256) amax_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float sm[8];
  float a = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) a = fmaxf(a, fabsf(__bfloat162float(x[i])));
  a = warp_max(a);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) a = fmaxf(a, sm[i]);
    atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(a));
  }
}

// Per-tensor FP8 fake-quant with a caller-owned scale: out = rt(x * scale) / scale. fmt 0 = e4m3, 1 = e5m2.
__global__ void __launch_bounds__(256) fp8_tensor_fake_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                              long long n, const float* __restrict__ scale_ptr, int fmt) {
  const float sc = *scale_ptr;
  const float inv = sc != 0.f ? 1.f / sc : 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = __bfloat162float(x[i]) * sc;
    out[i] = __float2bfloat16((fmt == 0 ? e4m3_rt(v) : e5m2_rt(v)) * inv);
  }
}

// Integer affine fake-quant: scale = (max-min)/(2^b-1), zp = -min/scale, q = clamp(round(x/scale+zp)).
__global__ void __launch_bounds__(256) int_affine_fake_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                              long long n, const float* __restrict__ minmax, int bits) {
  const float lo = minmax[0], hi = minmax[1];
  const float qmax = (float)((1 << bits) - 1);
  float sc = (hi - lo) / qmax;
  if (!(sc > 0.f)) sc = 1.f;
  const float zp = -lo / sc;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = __bfloat162float(x[i]);
    const float q = fminf(fmaxf(rintf(v / sc + zp), 0.f), qmax);
    out[i] = __float2bfloat16((q - zp) * sc);
  }
}

__global__ void __launch_bounds__(256) minmax_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ part) {
  __shared__ float smin[8], smax[8];
  float lo = INFINITY, hi = -INFINITY;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = __bfloat162float(x[i]);
    lo = fminf(lo, v);
    hi = fmaxf(hi, v);
  }
  hi = warp_max(hi);
  lo = -warp_max(-lo);
  if ((threadIdx.x & 31) == 0) { smin[threadIdx.x >> 5] = lo; smax[threadIdx.x >> 5] = hi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) { lo = fminf(lo, smin[i]); hi = fmaxf(hi, smax[i]); }
    part[2 * blockIdx.x] = lo;
    part[2 * blockIdx.x + 1] = hi;
  }
}
__global__ void minmax_finish_kernel(const float* __restrict__ part, int P, float* __restrict__ out) {
  float lo = INFINITY, hi = -INFINITY;
  for (int i = 0; i < P; ++i) { lo = fminf(lo, part[2 * i]); hi = fmaxf(hi, part[2 * i + 1]); }
  out[0] = lo;
  out[1] = hi;
}

// Surrogate gradients of the quantiser: 0 straight-through, 1 sigmoid-tempered (T), 2 piecewise linear.
__global__ void __launch_bounds__(256) qat_surrogate_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                                                                __nv_bfloat16* __restrict__ out, long long n, int mode, float p0,
                                                                float p1) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float xv = __bfloat162float(x[i]), gv = __bfloat162float(g[i]);
    float r = gv;
    if (mode == 1) {
      const float s = 1.f / (1.f + __expf(-xv / p0));
      r = gv * s * (1.f - s) / p0;
    } else if (mode == 2) {
      r = fabsf(xv) <= p0 ? gv : gv * p1;
    }
    out[i] = __float2bfloat16(r);
  }
}

inline int qgrid(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b > 148 * 16 ? 148 * 16 : (b < 1 ? 1 : b));
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// MXFP8 fake-quant of a [rows, cols] bf16 matrix. axis 1: 32-element blocks along cols (cols % 32 == 0);
// axis 0: blocks of 32 rows (any rows; a short last block is allowed).
ELFA_API int elfa_mxfp8_fake_quant(const void* x, void* out, int rows, int cols, int axis, void* stream) {
  ELFA_REQUIRE(x && out && rows > 0 && cols > 0, "mxfp8_fake_quant: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (axis == 1) {
    ELFA_REQUIRE(cols % 32 == 0, "mxfp8_fake_quant: cols must be a multiple of 32");
    const long long nb = (long long)rows * cols / 32;
    mxfp8_rowwise_kernel<true><<<qgrid(nb), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), nullptr, nullptr, nb);
  } else {
    dim3 grid((cols + 255) / 256, (rows + 31) / 32);
    mxfp8_colwise_fake_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), rows, cols);
  }
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// MXFP8 quantise (row-wise blocks): payload [rows, cols] e4m3 bytes, scales [rows, cols/32] ue8m0 bytes.
ELFA_API int elfa_mxfp8_quantize(const void* x, void* payload, void* scales, int rows, int cols, void* stream) {
  ELFA_REQUIRE(x && payload && scales && rows > 0 && cols > 0 && cols % 32 == 0, "mxfp8_quantize: bad arguments");
  const long long nb = (long long)rows * cols / 32;
  mxfp8_rowwise_kernel<false><<<qgrid(nb), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), nullptr, static_cast<uint8_t*>(payload), static_cast<uint8_t*>(scales), nb);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// NVFP4 fake-quant; tensor_amax: device float holding max|x| of the whole tensor (see elfa_amax).
ELFA_API int elfa_nvfp4_fake_quant(const void* x, void* out, int rows, int cols, int axis, const float* tensor_amax, void* stream) {
  ELFA_REQUIRE(x && out && tensor_amax && rows > 0 && cols > 0, "nvfp4_fake_quant: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (axis == 1) {
    ELFA_REQUIRE(cols % 16 == 0, "nvfp4_fake_quant: cols must be a multiple of 16");
    const long long nb = (long long)rows * cols / 16;
    nvfp4_rowwise_fake_kernel<<<qgrid(nb), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), nb, tensor_amax);
  } else {
    dim3 grid((cols + 255) / 256, (rows + 15) / 16);
    nvfp4_colwise_fake_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), rows, cols, tensor_amax);
  }
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// *out = max(*out, max|x|). Zero *out first for a fresh reduction.
ELFA_API int elfa_amax(const void* x, long long n, float* out, void* stream) {
  ELFA_REQUIRE(x && out && n > 0, "amax: bad arguments");
  amax_kernel<<<qgrid(n / 4 + 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x), n, out);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

ELFA_API int elfa_fp8_tensor_fake_quant(const void* x, void* out, long long n, const float* scale, int fmt, void* stream) {
  ELFA_REQUIRE(x && out && scale && n > 0 && (fmt == 0 || fmt == 1), "fp8_tensor_fake_quant: bad arguments");
  fp8_tensor_fake_kernel<<<qgrid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                                                  static_cast<__nv_bfloat16*>(out), n, scale, fmt);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// minmax: 2 device floats (written here); part: >= 2 * 2368 floats of scratch.
ELFA_API int elfa_int_affine_fake_quant(const void* x, void* out, long long n, int bits, float* minmax, float* part, void* stream) {
  ELFA_REQUIRE(x && out && minmax && part && n > 0 && bits >= 2 && bits <= 16, "int_affine_fake_quant: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = qgrid(n / 4 + 1);
  minmax_kernel<<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, part);
  minmax_finish_kernel<<<1, 1, 0, s>>>(part, g, minmax);
  int_affine_fake_kernel<<<qgrid(n), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), n, minmax, bits);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(3);
  return ELFA_OK;
}

ELFA_API int elfa_qat_surrogate_bwd(const void* x, const void* g, void* out, long long n, int mode, float p0, float p1, void* stream) {
  ELFA_REQUIRE(x && g && out && n > 0 && mode >= 0 && mode <= 2, "qat_surrogate_bwd: bad arguments");
  qat_surrogate_bwd_kernel<<<qgrid(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g), static_cast<__nv_bfloat16*>(out), n, mode, p0, p1);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}
