// Device-side building blocks of the fused compute + collective kernels: bounded waits on counters
// that peer GPUs increment, and the push role that sends byte ranges of this GPU's memory into the
// same offsets of every peer's buffer with bulk copies (local global -> shared -> peer global).
//
// Nothing here is a multicast and no bulk / tensor load ever reads another GPU's memory: remote data
// is written into the consumer's own memory and read from there.
//
// Reference call sites these kernels replace: src/distributed/tensor_parallel.zig:77-129 and
// src/distributed/sequence_parallel.zig:79-128 (ncclAllGather, then the consumer GEMM).
#pragma once
#include "common.cuh"

namespace elfa {

constexpr int MAX_RANKS = 8;

inline long long wait_cycles_of(int wait_ms) { return (long long)(wait_ms > 0 ? wait_ms : 10000) * 1900000LL; }

#ifdef __CUDACC__
// Bounded wait until *flag >= target (wrap-safe). The counter is written by other GPUs.
__device__ __forceinline__ bool flag_wait(const unsigned int* flag, unsigned int target, long long limit, volatile int* abort_flag,
                                          unsigned int* status) {
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int)(v - target) >= 0) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) {
      *abort_flag = 1;
      atomicOr(status, (unsigned)ELFA_ST_FLAG_TIMEOUT);
      return false;
    }
    __nanosleep(100);
  }
}

__device__ __forceinline__ void flag_bump(unsigned long long peer_flags_base, int slot) {
  unsigned int* cnt = reinterpret_cast<unsigned int*>(peer_flags_base) + slot;
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
}

// What one rank sends in a fused all-gather: up to two byte ranges of its own buffer (for a
// block-scaled operand: its rows of the payload and its scale atoms), copied to the same offsets of
// every peer's buffer.
struct PushPlan {
  long long off[2];      // byte offsets inside the buffer, 16-byte aligned
  long long bytes[2];    // sizes, multiples of 16 bytes (0 = unused)
  long long limit;       // size of the buffer the ranges lie in (checked build: a piece past it is recorded and not sent)
};

constexpr int PUSH_PIECE = 8192;   // bytes per bulk copy

// Push role, run by two warps (`w` = 0 / 1) of every CTA of the grid. Peer rank+1 first, then rank+2, ...
// so that at any time every GPU receives from one sender. Lane 0 of each warp drives a two-buffer
// pipeline of bulk copies; after a peer's last piece has landed (store groups complete, system fence)
// warp 0 increments that peer's arrival counter [rank] once: the counter reaches `gridDim.x` more
// than before when the whole range is there.
//   buf0        : shared memory of this warp, 2 x PUSH_PIECE bytes, 16-byte aligned
//   bar_a/bar_b : two mbarriers (initialised with count 1) for the loads of the two buffers
//   sync_id     : a named barrier the two push warps meet at
__device__ __forceinline__ void push_ranges(const char* local_base, const unsigned long long* peer_base, const unsigned long long* peer_flags,
                                            int rank, int world, const PushPlan& plan, uint32_t buf0, uint32_t bar_a, uint32_t bar_b,
                                            int sync_id, int w, int lane, volatile int* abort_flag, unsigned int* status) {
  const long long np0 = (plan.bytes[0] + PUSH_PIECE - 1) / PUSH_PIECE;
  const long long np1 = (plan.bytes[1] + PUSH_PIECE - 1) / PUSH_PIECE;
  const long long npieces = np0 + np1;
  const long long c_first = (long long)blockIdx.x * 2 + w, c_step = (long long)gridDim.x * 2;
  uint32_t n_issued = 0, n_done = 0;   // loads issued / consumed: buffer = index & 1, phase = (index >> 1) & 1
  bool ok = true;
  auto piece = [&](long long c, long long& off, uint32_t& nb) {
    const int r = c < np0 ? 0 : 1;
    const long long i = r == 0 ? c : c - np0;
    const long long rem = plan.bytes[r] - i * PUSH_PIECE;
    off = plan.off[r] + i * PUSH_PIECE;
    nb = (uint32_t)(rem < PUSH_PIECE ? rem : PUSH_PIECE);
  };
  auto issue_load = [&](long long c) {
    const int b = n_issued & 1;
    long long off;
    uint32_t nb;
    piece(c, off, nb);
    tma_store_wait_read<0>();                       // the store that last used this buffer has read it
    const uint32_t bar = b ? bar_b : bar_a;
    mbar_expect_tx(bar, nb);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(buf0 + b * PUSH_PIECE), "l"(local_base + off), "r"(nb), "r"(bar) : "memory");
    ++n_issued;
  };
  // Peers are served one after the other without draining the pipeline in between: a peer's counter is raised once the
  // NEXT peer's stores have been issued and this peer's (older) bulk groups are known to be complete, so the NVLink round
  // trip of one peer's last pieces overlaps the next peer's transfers.
  auto wait_all_but = [](uint32_t n) {     // completion of every bulk group except the `n` most recent ones
    switch (n) {
      case 0: tma_store_wait<0>(); break;
      case 1: tma_store_wait<1>(); break;
      case 2: tma_store_wait<2>(); break;
      case 3: tma_store_wait<3>(); break;
      case 4: tma_store_wait<4>(); break;
      case 5: tma_store_wait<5>(); break;
      case 6: tma_store_wait<6>(); break;
      case 7: tma_store_wait<7>(); break;
      default: tma_store_wait<8>(); break;   // more than asked for: still correct
    }
  };
  int prev_peer = -1;
  for (int i = 1; i < world; ++i) {
    const int peer = (rank + i) % world;
    if (lane == 0) {
      char* dst = reinterpret_cast<char*>(peer_base[peer]);
      uint32_t stores = 0;
      if (ok && c_first < npieces) issue_load(c_first);
      for (long long c = c_first; c < npieces && ok; c += c_step) {
        if (c + c_step < npieces) issue_load(c + c_step);
        const int b = n_done & 1;
        if (!mbar_wait(b ? bar_b : bar_a, (n_done >> 1) & 1, abort_flag, status)) { ok = false; break; }
        long long off;
        uint32_t nb;
        piece(c, off, nb);
        if (bounds_ok(off + nb - 1, plan.limit, status))
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                       ::"l"(dst + off), "r"(buf0 + b * PUSH_PIECE), "r"(nb) : "memory");
        tma_store_commit();
        ++n_done;
        ++stores;
      }
      if (prev_peer >= 0) {
        wait_all_but(ok ? stores : 0u);                 // every store to the previous peer has completed
        __threadfence_system();
      }
    }
    __syncwarp();
    if (prev_peer >= 0) {
      named_bar_sync(sync_id, 64);                      // both push warps are done with the previous peer
      if (w == 0 && lane == 0) flag_bump(peer_flags[prev_peer], rank);
    }
    prev_peer = peer;
  }
  if (prev_peer >= 0) {
    if (lane == 0) {
      tma_store_wait<0>();
      __threadfence_system();
    }
    __syncwarp();
    named_bar_sync(sync_id, 64);
    if (w == 0 && lane == 0) flag_bump(peer_flags[prev_peer], rank);
  }
  if (lane == 0 && !ok) {   // give a load that is still in flight a bounded chance to land before the CTA exits
    for (uint32_t j = n_done; j < n_issued; ++j) {
      const long long t0 = clock64();
      while (!mbar_try((j & 1) ? bar_b : bar_a, (j >> 1) & 1) && clock64() - t0 < 4000000) {}
    }
  }
}
#endif  // __CUDACC__

}  // namespace elfa
