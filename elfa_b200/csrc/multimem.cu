// Collectives through the NVSwitch multicast mapping of a symmetric arena (NVLS): `multimem.ld_reduce`
// returns the sum of one address over every GPU of the group, reduced inside the switch, and
// `multimem.st` stores one value to that address on every GPU. An all-reduce is therefore one load and
// one store per element of this rank's 1 / world slice, and a GPU's NVLink carries 1 / world of the
// bytes in each direction per phase instead of (world - 1) / world.
//
// The reference's collective set is NCCL's (reference: src/runtime/nccl.zig:222-333 allReduce /
// reduceScatter / allGather, src/runtime/main.zig:170-176 barrier = 1-float all-reduce); its wish-list
// entry `nccl_allreduce_sum_fp8` (src/ptx/tcgen05_kernels.ptx:228) holds a scalar loop.
//
// `mc` is the multicast address of the arena (the same offsets as in the unicast mapping), `local` this
// rank's own mapping. The caller brackets every call with signal-word barriers (elfa_symm_barrier): all
// ranks' data complete before, all stores landed after. Nothing here waits, so nothing can hang.
// The mapping exists only while every rank of the group is alive; jobs in which ranks may leave keep
// to the peer-pointer kernels (plain loads and stores).
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

__device__ __forceinline__ float4 mm_ld_reduce_f32(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_f32(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
// eight bf16 values per call, summed in fp32 inside the switch
__device__ __forceinline__ uint4 mm_ld_reduce_bf16(const __nv_bfloat16* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_b32x4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// mode 0: all-reduce in place (slice of this rank: reduce, scale, store to everyone)
// mode 1: reduce-scatter (slice of this rank: reduce, scale, store to `out` locally)
// mode 2: all-gather (slice of this rank: read locally, store to everyone)
template <bool BF16>
__global__ void __launch_bounds__(256) multimem_kernel(char* mc, const char* local, char* out, long long off_bytes, long long n_elems,
                                                       int rank, int world, float scale, int mode) {
  constexpr int ESZ = BF16 ? 2 : 4;
  constexpr int VEC = 16 / ESZ;                       // elements per 16-byte access
  const long long per = n_elems / world;              // elements of one rank's slice
  const long long nvec = per / VEC;
  const long long base = off_bytes + (long long)rank * per * ESZ;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    const long long b = base + v * 16;
    if (mode == 2) {
      const uint4 q = *reinterpret_cast<const uint4*>(local + b);
      mm_st_b32x4(mc + b, q);
      continue;
    }
    if (BF16) {
      uint4 q = mm_ld_reduce_bf16(reinterpret_cast<const __nv_bfloat16*>(mc + b));
      if (scale != 1.f) {
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = pack_bf16(bf16_lo(w[j]) * scale, bf16_hi(w[j]) * scale);
        q = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (mode == 0) mm_st_b32x4(mc + b, q);
      else *reinterpret_cast<uint4*>(out + v * 16) = q;
    } else {
      float4 s = mm_ld_reduce_f32(reinterpret_cast<const float*>(mc + b));
      s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
      if (mode == 0) mm_st_f32(reinterpret_cast<float*>(mc + b), s);
      else *reinterpret_cast<float4*>(out + v * 16) = s;
    }
  }
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// One collective over `n` elements (fp32: dtype 0, bf16: dtype 1) that start `off_bytes` into the arena.
//   mode 0 all-reduce in place (every rank ends with scale * sum); mode 1 reduce-scatter: `out` (local, n / world elements)
//   = scale * sum of this rank's slice; mode 2 all-gather: this rank's slice goes to every rank.
// n must be a multiple of world * (16 / element size); off_bytes a multiple of 16. `mc`: multicast address of the arena,
// `local`: this rank's own address of the arena. Bracket with elfa_symm_barrier on the same stream.
ELFA_API int elfa_multimem_collective(unsigned long long mc, const void* local, void* out, long long off_bytes, long long n,
                                      int dtype, int rank, int world, float scale, int mode, void* stream) {
  ELFA_REQUIRE(mc != 0 && local, "multimem: no multicast mapping (NVLS unavailable or not enabled for this arena)");
  ELFA_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world && mode >= 0 && mode <= 2, "multimem: bad rank / world / mode");
  const int esz = dtype == 1 ? 2 : 4;
  ELFA_REQUIRE(dtype == 0 || dtype == 1, "multimem: dtype must be 0 (fp32) or 1 (bf16)");
  ELFA_REQUIRE(n > 0 && n % ((long long)world * (16 / esz)) == 0 && off_bytes % 16 == 0, "multimem: size / offset alignment");
  ELFA_REQUIRE(mode != 1 || out, "multimem: reduce-scatter needs an output");
  const long long nvec = n / world / (16 / esz);
  long long blocks = (nvec + 255) / 256;
  const int grid = (int)(blocks > 148 * 4 ? 148 * 4 : (blocks < 1 ? 1 : blocks));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 1)
    multimem_kernel<true><<<grid, 256, 0, s>>>(reinterpret_cast<char*>(mc), static_cast<const char*>(local), static_cast<char*>(out),
                                               off_bytes, n, rank, world, scale, mode);
  else
    multimem_kernel<false><<<grid, 256, 0, s>>>(reinterpret_cast<char*>(mc), static_cast<const char*>(local), static_cast<char*>(out),
                                                off_bytes, n, rank, world, scale, mode);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}
