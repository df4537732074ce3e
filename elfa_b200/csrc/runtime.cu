// Host runtime of the native library: error reporting, the per-device status word, device
// queries, TMA tensor-map creation, peer access, pinned host memory.
// Native counterpart of the reference's CUDA runtime shim (reference: src/runtime/cuda.zig:283-507,
// src/cuda_bindings.zig:14-135): PyTorch owns contexts and streams, this file adds what the
// kernels need beyond that.
#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>

#include "common.cuh"

namespace elfa {

static thread_local std::string g_last_error;
void set_last_error(const char* msg) { g_last_error = msg ? msg : ""; }
int cuda_fail(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return ELFA_ERR_CUDA;
}

static std::atomic<long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static std::atomic<int> g_deterministic{0};
bool deterministic_mode() { return g_deterministic.load(std::memory_order_relaxed) != 0; }

static std::mutex g_mu;
static unsigned int* g_status[64] = {nullptr};

unsigned int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static EncodeTiledFn get_encode() {
  // The driver call needs a current context on the calling thread; autograd worker threads may
  // not have bound the primary context yet. cudaFree(0) binds it (once per thread).
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(0);
    ctx_bound = true;
  }
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return nullptr;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld_bytes,
                 uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    set_last_error("cuTensorMapEncodeTiled is not available (no driver?)");
    return ELFA_ERR_CUDA;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld_bytes & 15)) {
    set_last_error("tensor map: base address and row pitch must be multiples of 16 bytes");
    return ELFA_ERR_ARG;
  }
  CUtensorMapDataType dt = elem_bytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_error = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r);
    return ELFA_ERR_CUDA;
  }
  return ELFA_OK;
}

// General N-d (<= 5) tiled map, 16-bit elements, 128-byte swizzle. dims/box innermost first;
// strides_bytes has ndim-1 entries (dims 1..).
int make_tmap_nd_bf16(CUtensorMap* out, const void* base, int ndim, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box) {
  EncodeTiledFn enc = get_encode();
  if (!enc) {
    set_last_error("cuTensorMapEncodeTiled is not available (no driver?)");
    return ELFA_ERR_CUDA;
  }
  if (reinterpret_cast<uintptr_t>(base) & 15) {
    set_last_error("tensor map: base address must be a multiple of 16 bytes");
    return ELFA_ERR_ARG;
  }
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < ndim; ++i) { d[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < ndim; ++i) {
    if (strides_bytes[i] & 15) {
      set_last_error("tensor map: strides must be multiples of 16 bytes");
      return ELFA_ERR_ARG;
    }
    st[i] = strides_bytes[i];
  }
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ndim, const_cast<void*>(base), d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_error = "cuTensorMapEncodeTiled (nd) failed with code " + std::to_string((int)r);
    return ELFA_ERR_CUDA;
  }
  return ELFA_OK;
}

}  // namespace elfa

using namespace elfa;

ELFA_API const char* elfa_last_error() { return g_last_error.c_str(); }

ELFA_API int elfa_version() { return 100; }

// runtime.deterministic: kernels choose a fixed summation order (the GEMM does not split the contraction across CTAs)
ELFA_API int elfa_set_deterministic(int on) {
  elfa::g_deterministic.store(on ? 1 : 0, std::memory_order_relaxed);
  return ELFA_OK;
}

#ifndef ELFA_SOURCE_HASH
#define ELFA_SOURCE_HASH "unknown"
#endif
ELFA_API const char* elfa_source_hash() { return ELFA_SOURCE_HASH; }

// Number of kernels this library has launched in this process (optionally reset).
ELFA_API long long elfa_launch_count(int reset) {
  long long v = g_launches.load();
  if (reset) g_launches.store(0);
  return v;
}

// Reads and clears the status word of the current device (synchronises the device).
namespace {
__global__ void bounds_selftest_kernel(unsigned int* status) {
  // no memory is touched: an index one past a four-element extent goes through the same test the kernels use
  if (threadIdx.x == 0 && !elfa::bounds_ok(4, 4, status)) return;
}
}  // namespace

// 1 when this library is the checked variant (-DELFA_BOUNDS), else 0.
ELFA_API int elfa_bounds_enabled() {
#ifdef ELFA_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// Runs the index test of the checked build on an out-of-range index (no access follows): afterwards the status word carries
// ELFA_ST_BOUNDS in the checked variant and stays clear in the normal one.
ELFA_API int elfa_bounds_selftest(void* stream) {
  unsigned int* st = elfa::status_word();
  ELFA_REQUIRE(st != nullptr, "bounds_selftest: no status word");
  bounds_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(st);
  ELFA_CUDA(cudaGetLastError());
  return ELFA_OK;
}

ELFA_API int elfa_status(unsigned int* out) {
  unsigned int* p = status_word();
  ELFA_REQUIRE(p != nullptr, "no status word (no device?)");
  ELFA_CUDA(cudaDeviceSynchronize());
  ELFA_CUDA(cudaMemcpy(out, p, sizeof(unsigned int), cudaMemcpyDeviceToHost));
  ELFA_CUDA(cudaMemset(p, 0, sizeof(unsigned int)));
  return ELFA_OK;
}

// out[0]=major out[1]=minor out[2]=SM count out[3]=max opt-in shared memory per block out[4]=L2 bytes
ELFA_API int elfa_device_info(int device, long long* out) {
  cudaDeviceProp p;
  ELFA_CUDA(cudaGetDeviceProperties(&p, device));
  out[0] = p.major;
  out[1] = p.minor;
  out[2] = p.multiProcessorCount;
  out[3] = (long long)p.sharedMemPerBlockOptin;
  out[4] = p.l2CacheSize;
  out[5] = (long long)p.totalGlobalMem;
  return ELFA_OK;
}

ELFA_API int elfa_is_blackwell(int device) {
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) return 0;
  return p.major >= 10 ? 1 : 0;
}

// Enables peer access from the current device to every other visible device that supports it.
// Returns the number of peers enabled in *n_enabled.
ELFA_API int elfa_enable_peer_access(int* n_enabled) {
  int cur = 0, n = 0, cnt = 0;
  ELFA_CUDA(cudaGetDevice(&cur));
  ELFA_CUDA(cudaGetDeviceCount(&n));
  for (int d = 0; d < n; ++d) {
    if (d == cur) continue;
    int can = 0;
    ELFA_CUDA(cudaDeviceCanAccessPeer(&can, cur, d));
    if (!can) continue;
    cudaError_t e = cudaDeviceEnablePeerAccess(d, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      cudaGetLastError();
      e = cudaSuccess;
    }
    ELFA_CUDA(e);
    ++cnt;
  }
  if (n_enabled) *n_enabled = cnt;
  return ELFA_OK;
}

ELFA_API int elfa_pinned_alloc(void** out, size_t bytes) {
  ELFA_CUDA(cudaHostAlloc(out, bytes, cudaHostAllocPortable));
  return ELFA_OK;
}
ELFA_API int elfa_pinned_free(void* p) {
  ELFA_CUDA(cudaFreeHost(p));
  return ELFA_OK;
}
