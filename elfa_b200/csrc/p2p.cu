// Write-then-flag hand-off between neighbouring ranks over NVLink peer memory: the sender copies a
// small buffer (a ShortConv halo, an EFLA / PRISM state or affine map) into the receiver's symmetric
// buffer with plain peer stores and then raises the receiver's arrival counter with a release; the
// receiver waits for the counter with a bounded spin.
//
// reference: src/distributed/sequence_parallel.zig:130-159 (ringExchange: grouped ncclSend / ncclRecv of
// one activation block per step) and :202-240 (syncCrossBoundary: a halo of boundary x hidden values to
// the neighbour). The reference has no consumer for either; here they carry the ShortConv halo and the
// EFLA state between sequence-parallel ranks.
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

// Every block copies its slice, then bumps the receiver's counter once; the receiver expects `gridDim.x`
// more arrivals per hand-off.
__global__ void __launch_bounds__(256) p2p_send_kernel(const uint4* __restrict__ src, uint4* __restrict__ peer_dst, long long nvec,
                                                       unsigned int* peer_counter) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) peer_dst[v] = src[v];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(peer_counter) : "memory");
}

// Bounded wait until *counter >= target (wrap-safe). On expiry sets the status word and returns.
__global__ void p2p_wait_kernel(const unsigned int* counter, unsigned int target, long long limit_cycles, unsigned int* status) {
  if (threadIdx.x != 0) return;
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if ((int)(v - target) >= 0) return;
    if (clock64() - t0 > limit_cycles) {
      atomicOr(status, (unsigned)ELFA_ST_FLAG_TIMEOUT);
      return;
    }
    __nanosleep(200);
  }
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// Copies `bytes` (a multiple of 16) from `src` to `peer_dst` (an address inside a peer's symmetric arena) and adds
// `*blocks_out` arrivals to `peer_counter` (a u32 in the peer's arena). The receiver passes the running total of
// expected arrivals to elfa_p2p_wait.
ELFA_API int elfa_p2p_send(const void* src, unsigned long long peer_dst, long long bytes, unsigned long long peer_counter,
                           int* blocks_out, void* stream) {
  ELFA_REQUIRE(src && peer_dst && peer_counter && blocks_out && bytes > 0 && bytes % 16 == 0, "p2p_send: bad arguments");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (peer_dst & 15) == 0, "p2p_send: buffers must be 16-byte aligned");
  const long long nvec = bytes / 16;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 64) blocks = 64;
  p2p_send_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), reinterpret_cast<uint4*>(peer_dst), nvec, reinterpret_cast<unsigned int*>(peer_counter));
  ELFA_CUDA(cudaGetLastError());
  *blocks_out = (int)blocks;
  count_launches(1);
  return ELFA_OK;
}

// Stream-ordered bounded wait for `target` arrivals on this rank's counter.
ELFA_API int elfa_p2p_wait(const void* counter, unsigned int target, int wait_ms, void* stream) {
  ELFA_REQUIRE(counter != nullptr, "p2p_wait: null counter");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "p2p_wait: no status word");
  p2p_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned int*>(counter), target,
                                                                   (long long)(wait_ms > 0 ? wait_ms : 10000) * 1900000LL, st);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}
