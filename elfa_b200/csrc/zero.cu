// ZeRO data-parallel step over NVLink peer memory: gradient reduce-scatter fused with the 1/N
// scale and the gradient-norm partial sums, and the sharded AdamW update fused with the parameter
// all-gather (each updated bf16 value is stored straight into every rank's parameter buffer).
// Plus the signal-word barrier the two kernels are bracketed with.
//
// Replaces the reference's sequence  ncclReduceScatter -> stream sync -> host loop x(1/N) ->
// optimizer -> grouped ncclAllGather -> host concat
// (reference: src/distributed/zero_sharding.zig:159-181 reduceScatterGradients, :115-157
// allGatherParameters; barrier = 1-float all-reduce, src/runtime/main.zig:170-176).
//
// All gradient / parameter buffers are regions of a symmetric arena: `peers[r]` is rank r's copy
// of the same region. Rank r owns elements [r * shard, (r + 1) * shard). The reduction adds the
// ranks in a fixed order, so the result is deterministic. Waits are bounded (status word).
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

constexpr int ZMAX = 8;

struct PeerPtrs {
  unsigned long long p[ZMAX];
};

struct StepScalarsZ {   // same layout as the optimizer's scalars
  float sumsq, clip_coef, grad_norm;
  int skip;
  float lr;
};

// One thread per peer: announce arrival to the peer, then wait for the peer's announcement.
__global__ void symm_barrier_kernel(PeerPtrs peer_flags, const unsigned int* my_flags, int rank, int world, unsigned int target,
                                    long long wait_cycles, unsigned int* status) {
  const int p = threadIdx.x;
  if (p >= world || p == rank) return;
  __threadfence_system();
  unsigned int* dst = reinterpret_cast<unsigned int*>(peer_flags.p[p]) + rank;
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(dst) : "memory");
  const long long t0 = clock64();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(my_flags + p) : "memory");
    if ((int)(v - target) >= 0) break;
    if (clock64() - t0 > wait_cycles) {
      atomicOr(status, (unsigned)ELFA_ST_FLAG_TIMEOUT);
      break;
    }
    __nanosleep(200);
  }
}

// out[i] = scale * sum_r grads_r[lo + i]  (fp32, i in [0, n)); part[block] = sum of out^2.
__global__ void __launch_bounds__(256) zero_reduce_kernel(PeerPtrs grads, int rank, int world, long long lo, long long n,
                                                          float* __restrict__ out, float scale, float* __restrict__ part) {
  __shared__ float sm[8];
  float acc2 = 0.f;
  const long long nvec = n / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 g[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)          // every peer's load in flight before the first add
      if (r < world) g[r] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo + v * 4);
#pragma unroll
    for (int r = 0; r < 8; ++r)          // fixed order: deterministic sum
      if (r < world) { s.x += g[r].x; s.y += g[r].y; s.z += g[r].z; s.w += g[r].w; }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[v] = s;
    acc2 += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  acc2 = warp_sum(acc2);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc2;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += sm[i];
    part[blockIdx.x] = s;
  }
}

// ---- stage 3 -------------------------------------------------------------------------------------
// Parameter gather with peer loads: dst[r * shard .. (r+1) * shard) = shard of rank r (16-byte vectors).
__global__ void __launch_bounds__(256) zero3_gather_kernel(PeerPtrs shards, int world, long long src_off, long long shard_vecs,
                                                           uint4* __restrict__ dst) {
  const long long total = shard_vecs * world;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; v0 < total; v0 += 4 * stride) {
    uint4 q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {    // four independent peer loads in flight per thread
      const long long v = v0 + u * stride;
      if (v < total) {
        const int r = (int)(v / shard_vecs);
        const long long i = v - (long long)r * shard_vecs;
        q[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(shards.p[r]) + src_off + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long v = v0 + u * stride;
      if (v < total) dst[v] = q[u];
    }
  }
}

// The same for a window [v_lo, v_hi) (16-byte vectors) of the concatenation: the part of a bucket that no GEMM fetches itself.
__global__ void __launch_bounds__(256) zero3_gather_window_kernel(PeerPtrs shards, long long src_off, long long shard_vecs, long long v_lo,
                                                                  long long v_hi, uint4* __restrict__ dst) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = v_lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; v < v_hi; v += stride) {
    const int r = (int)(v / shard_vecs);
    const long long i = v - (long long)r * shard_vecs;
    dst[v] = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(shards.p[r]) + src_off + i * 16);
  }
}

// Gradient reduce-scatter with peer loads: acc[i] += scale * sum_r grads_r[lo + i] (fixed order).
__global__ void __launch_bounds__(256) zero3_reduce_acc_kernel(PeerPtrs grads, int world, long long lo, long long n,
                                                               float* __restrict__ acc, float scale) {
  const long long nvec = n / 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 g[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)          // every peer's load in flight before the first add
      if (r < world) g[r] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo + v * 4);
#pragma unroll
    for (int r = 0; r < 8; ++r)          // fixed order
      if (r < world) { s.x += g[r].x; s.y += g[r].y; s.z += g[r].z; s.w += g[r].w; }
    float4 a = reinterpret_cast<float4*>(acc)[v];
    a.x += s.x * scale; a.y += s.y * scale; a.z += s.z * scale; a.w += s.w * scale;
    reinterpret_cast<float4*>(acc)[v] = a;
  }
}

// bf16 on the wire: every rank first rounds its fp32 gradient bucket to bf16 into a peer-addressable staging region
// (fp32 -> bf16, 8 elements per thread); the owners then sum the peers' bf16 values in fp32, in fixed rank order.
// NVLink carries 2 bytes per element instead of 4.
__global__ void __launch_bounds__(256) zero_pack_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long nvec = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    const float4 a = reinterpret_cast<const float4*>(src)[2 * v], b = reinterpret_cast<const float4*>(src)[2 * v + 1];
    reinterpret_cast<uint4*>(dst)[v] = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
  }
}

__global__ void __launch_bounds__(256) zero3_reduce_acc_bf16_kernel(PeerPtrs staged, int world, long long lo, long long n,
                                                                    float* __restrict__ acc, float scale) {
  const long long nvec = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 q[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)          // every peer's load in flight before the first add
      if (r < world) q[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(staged.p[r]) + lo + v * 8);
#pragma unroll
    for (int r = 0; r < 8; ++r) {        // fixed rank order
      if (r < world) {
        const uint32_t w[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          s[2 * j] += bf16_lo(w[j]);
          s[2 * j + 1] += bf16_hi(w[j]);
        }
      }
    }
    float4 a0 = reinterpret_cast<float4*>(acc)[2 * v], a1 = reinterpret_cast<float4*>(acc)[2 * v + 1];
    a0.x += s[0] * scale; a0.y += s[1] * scale; a0.z += s[2] * scale; a0.w += s[3] * scale;
    a1.x += s[4] * scale; a1.y += s[5] * scale; a1.z += s[6] * scale; a1.w += s[7] * scale;
    reinterpret_cast<float4*>(acc)[2 * v] = a0;
    reinterpret_cast<float4*>(acc)[2 * v + 1] = a1;
  }
}

__global__ void zero_sumsq_finish_kernel(const float* __restrict__ part, int P, StepScalarsZ* scal) {
  __shared__ float sm[256];
  float a = 0.f;
  for (int i = threadIdx.x; i < P; i += 256) a += part[i];
  sm[threadIdx.x] = a;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sm[threadIdx.x] += sm[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) scal->sumsq = sm[0];
}

// AdamW on the owned shard; the new bf16 values go to every rank's parameter buffer.
// Eight elements per thread (one 16-byte store per peer).
__global__ void __launch_bounds__(256) zero_adamw_allgather_kernel(PeerPtrs params, int rank, int world, long long lo, long long n,
                                                                   float* __restrict__ master, float* __restrict__ m,
                                                                   float* __restrict__ v, const float* __restrict__ g, float lr,
                                                                   float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                                                   const StepScalarsZ* __restrict__ scal, long long wd_lo, long long wd_hi) {
  const bool skip = scal->skip != 0;
  const float gscale = scal->clip_coef;
  const long long nvec = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long vi = (long long)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += stride) {
    const long long i0 = vi * 8;
    float p[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 pm = *reinterpret_cast<const float4*>(master + i0 + 4 * h);
      p[4 * h] = pm.x; p[4 * h + 1] = pm.y; p[4 * h + 2] = pm.z; p[4 * h + 3] = pm.w;
    }
    if (!skip) {
      float gg[8], mm[8], vv[8];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float4 a = *reinterpret_cast<const float4*>(g + i0 + 4 * h);
        const float4 b = *reinterpret_cast<const float4*>(m + i0 + 4 * h);
        const float4 c = *reinterpret_cast<const float4*>(v + i0 + 4 * h);
        gg[4 * h] = a.x; gg[4 * h + 1] = a.y; gg[4 * h + 2] = a.z; gg[4 * h + 3] = a.w;
        mm[4 * h] = b.x; mm[4 * h + 1] = b.y; mm[4 * h + 2] = b.z; mm[4 * h + 3] = b.w;
        vv[4 * h] = c.x; vv[4 * h + 1] = c.y; vv[4 * h + 2] = c.z; vv[4 * h + 3] = c.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long gi = lo + i0 + j;            // global index: weight decay applies inside [wd_lo, wd_hi)
        const float w = (gi >= wd_lo && gi < wd_hi) ? wd : 0.f;
        const float gj = gg[j] * gscale;
        mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
        vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
        p[j] -= lr * ((mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps) + w * p[j]);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        *reinterpret_cast<float4*>(master + i0 + 4 * h) = make_float4(p[4 * h], p[4 * h + 1], p[4 * h + 2], p[4 * h + 3]);
        *reinterpret_cast<float4*>(m + i0 + 4 * h) = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
        *reinterpret_cast<float4*>(v + i0 + 4 * h) = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
      }
    }
    const uint4 o = make_uint4(pack_bf16(p[0], p[1]), pack_bf16(p[2], p[3]), pack_bf16(p[4], p[5]), pack_bf16(p[6], p[7]));
    for (int i = 0; i < world; ++i) {
      const int r = (rank + i) % world;   // own copy first, then the peers, staggered by rank
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo + i0) = o;
    }
  }
}

inline int zgrid(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b > 148 * 8 ? 148 * 8 : (b < 1 ? 1 : b));
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// Barrier over the ranks of a symmetric arena. peer_flags: `world` device addresses of the ranks'
// barrier words (u32 per source rank); epoch: number of this call (1, 2, ...), same on all ranks.
ELFA_API int elfa_symm_barrier(const unsigned long long* peer_flags, const void* my_flags, int rank, int world, unsigned int epoch,
                               int wait_ms, void* stream) {
  ELFA_REQUIRE(peer_flags && my_flags && world >= 1 && world <= ZMAX && rank >= 0 && rank < world, "symm_barrier: bad arguments");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "symm_barrier: no status word");
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = peer_flags[i];
  symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pp, static_cast<const unsigned int*>(my_flags), rank, world,
                                                                      epoch, (long long)(wait_ms > 0 ? wait_ms : 10000) * 1900000LL, st);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// reduced[0..n) = scale * sum over ranks of grads_r[lo .. lo+n) (fp32); scalars->sumsq = sum(reduced^2).
// part: >= 1184 floats of scratch. n must be a multiple of 8.
ELFA_API int elfa_zero_reduce(const unsigned long long* peer_grads, int rank, int world, long long lo, long long n, float* reduced,
                              float scale, float* part, void* scalars, void* stream) {
  ELFA_REQUIRE(peer_grads && reduced && part && scalars && n > 0 && n % 8 == 0 && lo % 4 == 0, "zero_reduce: bad arguments");
  ELFA_REQUIRE(world >= 1 && world <= ZMAX && rank >= 0 && rank < world, "zero_reduce: bad rank/world");
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = peer_grads[i];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int g = zgrid(n / 4);
  zero_reduce_kernel<<<g, 256, 0, s>>>(pp, rank, world, lo, n, reduced, scale, part);
  zero_sumsq_finish_kernel<<<1, 256, 0, s>>>(part, g, static_cast<StepScalarsZ*>(scalars));
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(2);
  return ELFA_OK;
}

// AdamW on [lo, lo+n) with fp32 master / m / v (local, indexed from 0) and the reduced gradient;
// bf16 results are written to every rank's parameter buffer. Weight decay applies to global
// indices in [wd_lo, wd_hi).
ELFA_API int elfa_zero_adamw_allgather(const unsigned long long* peer_params, int rank, int world, long long lo, long long n,
                                       float* master, float* m, float* v, const float* reduced, float lr, float beta1, float beta2,
                                       float eps, float wd, int step, const void* scalars, long long wd_lo, long long wd_hi,
                                       void* stream) {
  ELFA_REQUIRE(peer_params && master && m && v && reduced && scalars && n > 0 && n % 8 == 0 && lo % 8 == 0 && step >= 1,
               "zero_adamw_allgather: bad arguments");
  ELFA_REQUIRE(world >= 1 && world <= ZMAX && rank >= 0 && rank < world, "zero_adamw_allgather: bad rank/world");
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = peer_params[i];
  const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
  zero_adamw_allgather_kernel<<<zgrid(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, rank, world, lo, n, master, m, v, reduced, lr, beta1, beta2, eps, wd, bc1, bc2, static_cast<const StepScalarsZ*>(scalars),
      wd_lo, wd_hi);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Stage 3 parameter gather of bytes [lo_bytes, hi_bytes) of the concatenation only (see elfa_zero3_gather for the rest).
ELFA_API int elfa_zero3_gather_window(const unsigned long long* peer_shards, int world, long long src_off_bytes, long long shard_bytes,
                                      long long lo_bytes, long long hi_bytes, void* dst, void* stream) {
  ELFA_REQUIRE(peer_shards && dst && world >= 1 && world <= ZMAX, "zero3_gather_window: bad arguments");
  ELFA_REQUIRE(shard_bytes > 0 && shard_bytes % 16 == 0 && src_off_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0,
               "zero3_gather_window: sizes and offsets must be multiples of 16 bytes");
  ELFA_REQUIRE(lo_bytes >= 0 && lo_bytes % 16 == 0 && hi_bytes % 16 == 0 && lo_bytes <= hi_bytes && hi_bytes <= shard_bytes * world,
               "zero3_gather_window: the window must be 16-byte aligned and inside the bucket");
  if (lo_bytes == hi_bytes) return ELFA_OK;
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = peer_shards[i];
  zero3_gather_window_kernel<<<zgrid((hi_bytes - lo_bytes) / 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      pp, src_off_bytes, shard_bytes / 16, lo_bytes / 16, hi_bytes / 16, static_cast<uint4*>(dst));
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Stage 3 parameter gather: dst (this rank's full-size slot) = concatenation of every rank's shard, which
// starts `src_off_bytes` into the rank's shard buffer (peer_shards: `world` device addresses). Peer loads only.
ELFA_API int elfa_zero3_gather(const unsigned long long* peer_shards, int world, long long src_off_bytes, long long shard_bytes,
                               void* dst, void* stream) {
  ELFA_REQUIRE(peer_shards && dst && world >= 1 && world <= ZMAX, "zero3_gather: bad arguments");
  ELFA_REQUIRE(shard_bytes > 0 && shard_bytes % 16 == 0 && src_off_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0,
               "zero3_gather: sizes and offsets must be multiples of 16 bytes");
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = peer_shards[i];
  const long long vecs = shard_bytes / 16;
  zero3_gather_kernel<<<zgrid(vecs * world / 4 + 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(pp, world, src_off_bytes, vecs,
                                                                                                static_cast<uint4*>(dst));
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Stage 3 gradient reduce-scatter: acc[0..n) += scale * sum over ranks of grads_r[lo .. lo+n) (fp32 elements).
ELFA_API int elfa_zero3_reduce_acc(const unsigned long long* peer_grads, int world, long long lo, long long n, float* acc, float scale,
                                   void* stream) {
  ELFA_REQUIRE(peer_grads && acc && world >= 1 && world <= ZMAX && n > 0 && n % 4 == 0 && lo % 4 == 0, "zero3_reduce_acc: bad arguments");
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = peer_grads[i];
  zero3_reduce_acc_kernel<<<zgrid(n / 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(pp, world, lo, n, acc, scale);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// fp32 gradients -> bf16 staging region (what the peers read in elfa_zero3_reduce_acc_bf16). n: multiple of 8.
ELFA_API int elfa_zero_pack_bf16(const float* src, void* dst, long long n, void* stream) {
  ELFA_REQUIRE(src && dst && n > 0 && n % 8 == 0, "zero_pack_bf16: bad arguments");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0, "zero_pack_bf16: alignment");
  zero_pack_bf16_kernel<<<zgrid(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, static_cast<__nv_bfloat16*>(dst), n);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// acc[0..n) += scale * sum over ranks of staged_r[lo .. lo+n), staged = the ranks' bf16 staging regions; fp32 sums in rank order.
ELFA_API int elfa_zero3_reduce_acc_bf16(const unsigned long long* peer_staged, int world, long long lo, long long n, float* acc,
                                        float scale, void* stream) {
  ELFA_REQUIRE(peer_staged && acc && world >= 1 && world <= ZMAX && n > 0 && n % 8 == 0 && lo % 8 == 0, "zero3_reduce_acc_bf16: bad arguments");
  PeerPtrs pp{};
  for (int i = 0; i < world; ++i) pp.p[i] = peer_staged[i];
  zero3_reduce_acc_bf16_kernel<<<zgrid(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(pp, world, lo, n, acc, scale);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}
