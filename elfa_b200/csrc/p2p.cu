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

// Link probe: copies `bytes` from local memory to `dst` (normally a peer's arena) with one of the mechanisms the fused
// kernels can use, so that their ceilings can be measured apart from any GEMM.
//   mode 0: every thread loads 16 bytes and stores them (grid-stride)
//   mode 1: one lane per warp drives a ring of `depth` shared-memory buffers of `piece` bytes: bulk load global -> shared,
//           bulk store shared -> dst; a buffer is reused once its store has read it (cp.async.bulk.wait_group.read)
// Every wait on a load is bounded (status word), like everywhere else.
__global__ void __launch_bounds__(256) p2p_probe_kernel(const char* __restrict__ src, char* __restrict__ dst, long long bytes, int mode,
                                                        int piece, int depth, unsigned int* status) {
  extern __shared__ __align__(128) uint8_t probe_smem[];
  if (mode == 0) {
    const long long nvec = bytes / 16, stride = (long long)gridDim.x * blockDim.x;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) d4[v] = s4[v];
    return;
  }
  __shared__ uint64_t bars[8 * 4];
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) {
    for (int i = 0; i < nwarps * depth; ++i) mbar_init(smem_u32(&bars[i]), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (lane != 0) return;
  const uint32_t buf0 = smem_u32(probe_smem) + (uint32_t)warp * depth * piece;
  const long long npieces = (bytes + piece - 1) / piece;
  const long long first = (long long)blockIdx.x * nwarps + warp, step = (long long)gridDim.x * nwarps;
  uint32_t n_issued = 0, n_done = 0;
  auto nbytes_of = [&](long long c) { const long long rem = bytes - c * piece; return (uint32_t)(rem < piece ? rem : piece); };
  auto issue_load = [&](long long c) {
    const int b = n_issued % depth;
    const uint32_t bar = smem_u32(&bars[warp * depth + b]);
    mbar_expect_tx(bar, nbytes_of(c));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(buf0 + b * piece), "l"(src + c * piece), "r"(nbytes_of(c)), "r"(bar) : "memory");
    ++n_issued;
  };
  // prologue: depth - 1 loads ahead
  long long c_load = first;
  for (int i = 0; i < depth - 1 && c_load < npieces; ++i, c_load += step) issue_load(c_load);
  for (long long c = first; c < npieces; c += step) {
    if (c_load < npieces) {
      // the buffer about to be refilled was last read by the store issued `depth - 1` pieces ago... wait until at most
      // depth - 2 stores still read their buffers (depth is 2, 3 or 4)
      if (depth == 2) tma_store_wait_read<0>(); else if (depth == 3) tma_store_wait_read<1>(); else tma_store_wait_read<2>();
      issue_load(c_load);
      c_load += step;
    }
    const int b = n_done % depth;
    if (!mbar_wait(smem_u32(&bars[warp * depth + b]), (n_done / depth) & 1, &abort_flag, status)) break;
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst + c * piece), "r"(buf0 + b * piece), "r"(nbytes_of(c)) : "memory");
    tma_store_commit();
    ++n_done;
  }
  tma_store_wait<0>();
  for (uint32_t j = n_done; j < n_issued; ++j) {   // after a timeout: a bounded chance for loads in flight to land
    const long long t0 = clock64();
    while (!mbar_try(smem_u32(&bars[warp * depth + j % depth]), (j / depth) & 1) && clock64() - t0 < 4000000) {}
  }
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// Link probe (see p2p_probe_kernel). `piece` a multiple of 16 up to 16384, `depth` 2..4, `warps` 1..8 per CTA.
ELFA_API int elfa_p2p_probe(const void* src, unsigned long long dst, long long bytes, int mode, int ctas, int warps, int piece, int depth,
                            void* stream) {
  ELFA_REQUIRE(src && dst && bytes > 0 && bytes % 16 == 0 && ctas > 0, "p2p_probe: bad arguments");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (dst & 15) == 0, "p2p_probe: buffers must be 16-byte aligned");
  ELFA_REQUIRE(mode == 0 || (warps >= 1 && warps <= 8 && depth >= 2 && depth <= 4 && piece % 16 == 0 && piece > 0 && piece <= 16384),
               "p2p_probe: bad pipeline shape");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "p2p_probe: no status word");
  const int threads = mode == 0 ? 256 : warps * 32;
  const size_t smem = mode == 0 ? 0 : (size_t)warps * depth * piece;
  ELFA_REQUIRE(smem <= 200 * 1024, "p2p_probe: pipeline buffers exceed shared memory");
  static size_t configured = 0;
  if (smem > configured) {
    ELFA_CUDA(cudaFuncSetAttribute(p2p_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024)));
    configured = 200 * 1024;
  }
  p2p_probe_kernel<<<ctas, threads, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const char*>(src), reinterpret_cast<char*>(dst),
                                                                               bytes, mode, piece, depth, st);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}

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
