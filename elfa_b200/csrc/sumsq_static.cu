// Sum of squares without any allocation: the variant of elfa_sumsq() for callers that may not
// allocate device memory (see elfa_static.h). The per-block partial sums live in a file-scope
// device array instead of a caller-provided scratch buffer.
#include <mutex>

#include "common.cuh"
#include "elfa_static.h"

namespace {

constexpr int kMaxBlocks = 1024;

// Scratch shared by every call on this device. In host code this name is only a handle for the
// runtime, not a device address: the address is obtained once per device with
// cudaGetSymbolAddress() below and passed to the kernels as an ordinary pointer.
static __device__ __align__(256) float g_static_partials[kMaxBlocks];

template <typename T>
__global__ void __launch_bounds__(256) sumsq_static_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ part) {
  __shared__ float sm[8];
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = (float)x[i];
    acc += v * v;
  }
  acc = elfa::warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += sm[i];
    part[blockIdx.x] = s;   // every slot the second kernel reads is written here first
  }
}

__global__ void sumsq_static_finish_kernel(const float* __restrict__ part, int nblocks, float* __restrict__ out) {
  __shared__ float sm[256];
  float a = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += 256) a += part[i];
  sm[threadIdx.x] = a;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = sm[0];
}

std::mutex g_mu;
float* g_scratch_addr[64] = {nullptr};   // device address of g_static_partials, per device

// Device address of the scratch array on the current device (looked up on first use).
int scratch_for_current_device(float** out) {
  int dev = 0;
  ELFA_CUDA(cudaGetDevice(&dev));
  ELFA_REQUIRE(dev >= 0 && dev < 64, "sumsq_static: device index out of range");
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    ELFA_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_partials));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return ELFA_OK;
}

}  // namespace

ELFA_API int elfa_sumsq_static(const void* x, int grad_type, long long n, float* out, void* stream) {
  ELFA_REQUIRE(x && out, "sumsq_static: null pointer");
  ELFA_REQUIRE(grad_type == 0 || grad_type == 1, "sumsq_static: grad_type must be 0 (fp32) or 1 (bf16)");
  ELFA_REQUIRE(n >= 1, "sumsq_static: empty input");
  ELFA_REQUIRE(n <= ELFA_SUMSQ_STATIC_MAX_ELEMS,
               "sumsq_static: input larger than ELFA_SUMSQ_STATIC_MAX_ELEMS (the static scratch holds 1024 partial sums of at most 2^24 "
               "elements); use elfa_sumsq with a caller-provided scratch buffer");
  float* part = nullptr;
  int rc = scratch_for_current_device(&part);
  if (rc != ELFA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long blocks = (n + 255) / 256;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  const int g = (int)blocks;
  if (grad_type == 0) sumsq_static_partial_kernel<float><<<g, 256, 0, s>>>(static_cast<const float*>(x), n, part);
  else sumsq_static_partial_kernel<__nv_bfloat16><<<g, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, part);
  sumsq_static_finish_kernel<<<1, 256, 0, s>>>(part, g, out);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
  return ELFA_OK;
}
