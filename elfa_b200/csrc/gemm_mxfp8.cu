// Block-scaled MXFP8 GEMM for sm_100a: e4m3 operands with one ue8m0 scale per 32 contraction
// elements, multiplied by tcgen05.mma.kind::mxf8f6f4.block_scale with the scale factors in tensor
// memory, fp32 accumulation, bf16 output.
//
// The reference only has a one-thread-per-output fp8 kernel with a single scalar scale
// (kernels/cuda/gemm_sm100.cu:74-112) and PTX stubs named quantize_mxfp8 / tensor_parallel_matmul_fp4
// (src/ptx/tcgen05_kernels.ptx:183,482) that hold no tensor-core instruction; the MX block format itself
// is src/tensor/dtype.zig:117-147 and src/optimizer/stable_qat.zig:52-130.
//
//   C[M,N] = epilogue( sum_k  (A[m,k] * 2^(sfa[m,k/32]-127)) * (B[n,k] * 2^(sfb[n,k/32]-127)) )
//
// Both operands are K-major e4m3 ([M,K] and [N,K] row-major). Scale factors are stored the way the
// tensor core wants to read them: 512-byte atoms covering 128 rows x 4 K-blocks (128 K-elements),
// byte (r % 32) * 16 + (r / 32) * 4 + kb inside an atom, atoms ordered [row block][K block]. One atom
// is one 32-lane x 128-bit tcgen05.cp into 4 tensor-memory columns (replicated to the 4 lane quarters);
// the k-th MMA of a 128-wide K tile selects byte k of those columns through the instruction descriptor.
//
// Roles per CTA (192 threads, persistent, one CTA per SM):
//   warp 0   : producer - TMA loads of the A / B tiles (128-byte swizzle) and bulk copies of the scale atoms
//   warp 1   : tensor-memory owner; one lane copies scales to tensor memory and issues the MMAs
//   warps 2-5: epilogue (one 32-lane quarter each): tcgen05.ld -> bias / GELU -> bf16 -> global
// Every wait is bounded (status word + abort flag), like the bf16 kernel.
//
// TWO = true: the two CTAs of a cluster form a pair (tcgen05 cta_group::2) on a 256 x BN tile. Each CTA
// loads its 128 rows of A, its half of B and the scales it needs (its rows of A, all columns of B); the
// even CTA issues the scale copies and the MMAs for both. Shared-memory fill per FLOP drops by a third,
// which is what bounds the single-CTA kernel (about 100 GB/s of L2 -> SM fill per SM, measured).
//
// Scale tensor of B is stored [K tile][row block] so that the atoms a tile needs are one contiguous copy.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "comm.cuh"
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

constexpr int QBM = 128;       // tile rows
constexpr int QBK = 128;       // K elements (= bytes) per stage: one 128-byte swizzle row
constexpr int QUMMA_K = 32;    // K per instruction for 8-bit operands
constexpr int Q_THREADS = 192;
constexpr int Q_THREADS_AG = 256;   // + two push warps (all-gather variant)
constexpr int SF_ATOM = 512;   // bytes of one scale atom (128 rows x 4 K-blocks)

// All-gather variant (AG = true): A = all_gather_rows of the ranks' quantised rows. Every rank has quantised its rows into
// its own gathered buffer (payload [M, K] followed by the scale atoms [M / 128][K tiles]); two extra warps per CTA push
// those two byte ranges into the same offsets of every peer's buffer (comm.cuh: push_ranges) while the tensor cores start
// on the own rows; tiles are visited own shard first, then in the order the pushes arrive, and the producer waits for a
// shard's arrival counter before its first tile of that shard. All TMA loads read this GPU's own memory.
struct QComm {
  int rank, world, rows_per_rank;
  long long wait_cycles;
  unsigned long long peer_buf[MAX_RANKS];     // peers' gathered buffers (entry `rank` = this rank's own)
  unsigned long long peer_flags[MAX_RANKS];   // peers' arrival counters, one u32 per source rank
  const unsigned int* my_flags;
  unsigned int flag_target;
  PushPlan plan;
};

struct QParams {
  int M, N, K;
  __nv_bfloat16* C;
  long long ldc;
  const uint8_t* sfa;
  const uint8_t* sfb;
  int kt;            // K tiles (= scale atoms per row block)
  int sfb_atoms;     // row blocks of the B scale tensor
  const float* amax_a;   // NVFP4 only: tensor-level abs-max of A and B (the fp32 scale is amax / (448 * 6))
  const float* amax_b;
  const __nv_bfloat16* bias;
  __nv_bfloat16* preact;
  long long ldpre;
  unsigned flags;
  unsigned int* status;
  int tiles_m, tiles_n, group_m;
};

template <int BN, int STAGES, bool TWO, bool FP4 = false>
struct QSmem {
  // B scale atoms per tile: a tile starts 0 / 32 / 64 / 96 rows into a 128-row atom depending on BN
  // (128: always 0 -> 1 atom; 192: 0 or 64 -> 2; 224: 0 / 32 / 64 / 96 -> 3)
  static constexpr int NATOM = BN <= 128 ? 1 : (BN <= 192 ? 2 : 3);
  static constexpr int KSF = FP4 ? 4 : 1;                 // scale atoms along K per stage: an atom covers 4 blocks of 32 (fp8) or 16 (fp4) elements
  static constexpr int A_BYTES = QBM * QBK;
  static constexpr int B_BYTES = (TWO ? BN / 2 : BN) * QBK;
  static constexpr int SF_BYTES = KSF * (1 + NATOM) * SF_ATOM;
  static constexpr int SF_OFF = STAGES * (A_BYTES + B_BYTES);
  static constexpr int BAR_OFF = SF_OFF + STAGES * SF_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4 + 4;   // ring full / empty, accumulator full / empty, push buffers (all-gather variant)
  static constexpr int TOTAL0 = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int EPI_OFF = (TOTAL0 + 127) / 128 * 128;      // epilogue staging: 4 warps x 4 KB (whole-line stores)
  static constexpr int TOTAL = EPI_OFF + 4 * 4096;
  static constexpr int DYN = TOTAL + 1024;
  static constexpr int PUSH_OFF = (TOTAL + 127) / 128 * 128;      // all-gather variant: 2 warps x 2 buffers of PUSH_PIECE bytes
  static constexpr int DYN_AG = PUSH_OFF + 4 * PUSH_PIECE + 1024;
  static constexpr uint32_t STAGE_TX = A_BYTES + B_BYTES + SF_BYTES;
};

__device__ __forceinline__ void q_tile_coords(const QParams& p, int tile, int& mb, int& nb) {
  const int per_group = p.group_m * p.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * p.group_m;
  const int gsz = min(p.group_m, p.tiles_m - first_m);
  const int r = tile - g * per_group;
  mb = first_m + r % gsz;
  nb = r / gsz;
}

// Tile order of the all-gather variant: tiles grouped by the rank whose rows they read, own rows first, then rank - 1,
// rank - 2, ... (the order in which the pushes arrive).
template <bool AG>
__device__ __forceinline__ void q_tile_coords_ag(const QParams& p, const QComm& c, int tile, int tile_m, int& mb, int& nb, int& shard) {
  if (!AG) {
    q_tile_coords(p, tile, mb, nb);
    shard = 0;
    return;
  }
  const int tm_shard = c.rows_per_rank / tile_m;
  const int per_shard = tm_shard * p.tiles_n;
  const int i = tile / per_shard;
  const int lt = tile - i * per_shard;
  shard = (c.rank - i + c.world) % c.world;
  mb = shard * tm_shard + lt % tm_shard;
  nb = lt / tm_shard;
}

template <int BN, int STAGES, bool TWO, bool FP4 = false, bool AG = false>
__global__ void __launch_bounds__(AG ? Q_THREADS_AG : Q_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB, const QParams p,
                  const QComm cm) {
  using L = QSmem<BN, STAGES, TWO, FP4>;
  static_assert(!(FP4 && TWO), "the NVFP4 variant is single-CTA");
  static_assert(!(FP4 && AG), "the all-gather variant is MXFP8 only");
  constexpr int KSF = L::KSF;
  constexpr int TILE_M = TWO ? 2 * QBM : QBM;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * L::A_BYTES;
  uint8_t* sSF = smem + L::SF_OFF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + L::NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * STAGES + 2 + b); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = TWO ? cluster_ctarank() : 0u;
  const int wid = TWO ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int wstride = TWO ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  // tensor memory: accumulator b at column 256 * b, one set of scale-factor columns behind each accumulator.
  // K tiles alternate between the two sets, so the copy of the next tile's scales does not have to
  // wait for the MMAs that still read the current ones.
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t ACC_STRIDE = 256;
  constexpr uint32_t SFA_COL = BN;                 // 4 columns per atom, KSF atoms
  constexpr uint32_t SFB_COL = BN + 4 * KSF;       // 4 columns per atom, KSF * NATOM atoms
  static_assert(BN % 16 == 0 && BN + 4 * KSF * (1 + L::NATOM) <= 256, "tile does not fit the tensor-memory plan");

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmSFA);
    prefetch_tmap(&tmSFB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), TWO ? 8 : 4);
    }
    for (int b = 0; b < 4; ++b) mbar_init(bar0 + 8u * (2 * STAGES + 4 + b), 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    if (TWO) {
      tmem_alloc_pair(smem_u32(tmem_holder), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = p.kt;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int ready_shard = AG ? cm.rank : -1;
      for (int tile = wid; tile < num_tiles && ok; tile += wstride) {
        int mb, nb, shard;
        q_tile_coords_ag<AG>(p, cm, tile, TILE_M, mb, nb, shard);
        if (AG && shard != ready_shard) {
          // the shard's payload and scales were written by a peer GPU: acquire its counter, then order those writes
          // before this thread's TMA (async proxy) reads
          if (!flag_wait(cm.my_flags + shard, cm.flag_target, cm.wait_cycles, abort_flag, p.status)) { ok = false; break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");
          ready_shard = shard;
        }
        const int m0 = mb * TILE_M + (int)cta_rank * QBM, n0 = nb * BN;
        const int mblk = m0 / QBM;               // row block of the A scales
        const int atom0 = n0 / 128;              // first row block of the B scales (the tensor is padded by one atom)
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status)) { ok = false; break; }
          const uint32_t a_dst = smem_u32(sA + s * L::A_BYTES), b_dst = smem_u32(sB + s * L::B_BYTES);
          const uint32_t sf_dst = smem_u32(sSF + s * L::SF_BYTES);
          // scale atoms are rows of 128 32-bit words in two tensor maps (no swizzle); rows past the end read as zero
          const int sfa_row = (mblk * p.kt + kb) * KSF, sfb_row = kb * KSF * (p.sfb_atoms + 1) + atom0;
          if (TWO) {
            const uint32_t fb = map_to_cta(full_bar(s), 0);
            if (cta_rank == 0) mbar_expect_tx(full_bar(s), 2 * L::STAGE_TX);
            tma_load_2d_pair(a_dst, &tmA, kb * QBK, m0, fb);
            tma_load_2d_pair(b_dst, &tmB, kb * QBK, n0 + (int)cta_rank * (BN / 2), fb);
            tma_load_2d_pair(sf_dst, &tmSFA, 0, sfa_row, fb);
            tma_load_2d_pair(sf_dst + SF_ATOM, &tmSFB, 0, sfb_row, fb);
          } else {
            mbar_expect_tx(full_bar(s), L::STAGE_TX);
            tma_load_2d(a_dst, &tmA, kb * QBK, m0, full_bar(s));
            tma_load_2d(b_dst, &tmB, kb * QBK, n0, full_bar(s));
            tma_load_2d(sf_dst, &tmSFA, 0, sfa_row, full_bar(s));                       // KSF atoms of A
#pragma unroll
            for (int q = 0; q < KSF; ++q)                                               // NATOM atoms of B per group of K blocks
              tma_load_2d(sf_dst + (KSF + q * L::NATOM) * SF_ATOM, &tmSFB, 0, sfb_row + q * (p.sfb_atoms + 1), full_bar(s));
          }
        }
      }
      if (!ok) {
        for (uint32_t j = it > (uint32_t)STAGES ? it - STAGES : 0; j < it; ++j) {
          const long long t0 = clock64();
          while (!mbar_try(full_bar(j % STAGES), (j / STAGES) & 1) && clock64() - t0 < 4000000) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ scale copies + MMA issue
    // The warp walks the loop converged; one elected lane issues the tensor-core instructions.
    if (cta_rank == 0) {
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int tile = wid; tile < num_tiles && ok; tile += wstride, ++tile_iter) {
        int mb, nb, shard;
        q_tile_coords_ag<AG>(p, cm, tile, TILE_M, mb, nb, shard);
        const uint32_t sfb_shift = (uint32_t)((nb * BN) % 128) / 32;   // tile starts inside an atom: skip its first columns
        const uint32_t buf = tile_iter & 1, bph = (tile_iter >> 1) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(buf), bph ^ 1, abort_flag, p.status));
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * ACC_STRIDE;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, abort_flag, p.status));
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * L::A_BYTES);
          const uint32_t b_base = smem_u32(sB + s * L::B_BYTES);
          const uint32_t sf_base = smem_u32(sSF + s * L::SF_BYTES);
          // scale atoms: 32 rows of 16 bytes, no swizzle, 8-row core matrices 128 bytes apart
          const uint32_t sf_tmem = tmem_base + (it & 1u) * ACC_STRIDE;
          if (elect_one()) {
#pragma unroll
          for (int q = 0; q < KSF; ++q) {
            if (TWO) tc_cp_32x128b_warpx4_pair(sf_tmem + SFA_COL + 4 * q, make_smem_desc(sf_base + q * SF_ATOM, 0, 128, 0));
            else tc_cp_32x128b_warpx4(sf_tmem + SFA_COL + 4 * q, make_smem_desc(sf_base + q * SF_ATOM, 0, 128, 0));
          }
#pragma unroll
          for (int j = 0; j < KSF * L::NATOM; ++j) {
            if (TWO) tc_cp_32x128b_warpx4_pair(sf_tmem + SFB_COL + 4 * j, make_smem_desc(sf_base + (KSF + j) * SF_ATOM, 0, 128, 0));
            else tc_cp_32x128b_warpx4(sf_tmem + SFB_COL + 4 * j, make_smem_desc(sf_base + (KSF + j) * SF_ATOM, 0, 128, 0));
          }
#pragma unroll
          for (int k = 0; k < QBK / QUMMA_K; ++k) {
            const uint64_t da = make_smem_desc(a_base + k * 32, 16, 1024, 2);
            const uint64_t db = make_smem_desc(b_base + k * 32, 16, 1024, 2);
            if (FP4)   // all four scale bytes of a column belong to this instruction's 64 K-elements
              tc_mma_nvf4(tmem_d, da, db, make_idesc_nvf4(TILE_M, BN), (kb | k) != 0 ? 1u : 0u, sf_tmem + SFA_COL + 4 * k,
                          sf_tmem + SFB_COL + 4 * L::NATOM * k + sfb_shift);
            else if (TWO) tc_mma_mxf8_pair(tmem_d, da, db, make_idesc_mxf8(TILE_M, BN, k, k), (kb | k) != 0 ? 1u : 0u, sf_tmem + SFA_COL,
                                      sf_tmem + SFB_COL + sfb_shift);
            else tc_mma_mxf8(tmem_d, da, db, make_idesc_mxf8(TILE_M, BN, k, k), (kb | k) != 0 ? 1u : 0u, sf_tmem + SFA_COL,
                             sf_tmem + SFB_COL + sfb_shift);
          }
          if (TWO) tc_commit_pair(empty_bar(s)); else tc_commit(empty_bar(s));
          }
          __syncwarp();
        }
        if (ok && elect_one()) {
          if (TWO) tc_commit_pair(tfull_bar(buf)); else tc_commit(tfull_bar(buf));
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    uint32_t tile_iter = 0;
    const unsigned fl = p.flags;
    float alpha = 1.f;
    if (FP4) {   // product of the two tensor-level scales
      const float aa = *p.amax_a, ab = *p.amax_b;
      alpha = (aa > 0.f ? aa / (448.f * 6.f) : 1.f) * (ab > 0.f ? ab / (448.f * 6.f) : 1.f);
    }
    for (int tile = wid; tile < num_tiles; tile += wstride, ++tile_iter) {
      int mb, nb, shard;
      q_tile_coords_ag<AG>(p, cm, tile, TILE_M, mb, nb, shard);
      const int m0 = mb * TILE_M + (int)cta_rank * QBM, n0 = nb * BN;
      const uint32_t buf = tile_iter & 1, bph = (tile_iter >> 1) & 1;
      bool ok = mbar_wait(tfull_bar(buf), bph, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t tcol0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * ACC_STRIDE;
      if (!(fl & ELFA_EPI_BIAS)) {
        // bf16 output (optionally the pre-activation too): 64 accumulator columns at a time through the warp's private 4 KB of shared memory, written as
        // whole 128-byte lines (common.cuh: warp_stage_64cols / warp_flush_64cols)
        const uint32_t stage = smem_u32(smem + L::EPI_OFF) + q * 4096;
        const int row0 = m0 + q * 32;
        __nv_bfloat16* cbase = p.C + (long long)row0 * p.ldc + n0;
        const int rows_valid = p.M - row0;
        uint32_t ra[32], rb[32];
        tmem_ld32(tcol0, ra);
        tmem_ld32(tcol0 + 32, rb);
#pragma unroll
        for (int c = 0; c < BN / 32; c += 2) {
          tmem_ld_wait();
          if (fl & ELFA_EPI_STORE_PREACT) {
            warp_stage_64cols(stage, ra, rb, alpha, lane);
            __syncwarp();
            warp_flush_64cols(stage, p.preact + (long long)row0 * p.ldpre + n0 + c * 32, p.ldpre, rows_valid, p.N - n0 - c * 32, lane);
            __syncwarp();
          }
          if (fl & ELFA_EPI_GELU) warp_stage_64cols<true>(stage, ra, rb, alpha, lane);
          else warp_stage_64cols(stage, ra, rb, alpha, lane);
          if (c + 2 < BN / 32) {
            tmem_ld32(tcol0 + (c + 2) * 32, ra);
            tmem_ld32(tcol0 + (c + 3) * 32, rb);
          }
          __syncwarp();
          warp_flush_64cols(stage, cbase + c * 32, p.ldc, rows_valid, p.N - n0 - c * 32, lane);
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (TWO) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0)); else mbar_arrive(tempty_bar(buf));
        }
        continue;
      }
      uint32_t rnext[32];
      tmem_ld32(tcol0, rnext);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = rnext[j];
        if (c + 1 < BN / 32) tmem_ld32(tcol0 + (c + 1) * 32, rnext);
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) continue;   // uniform across the warp
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = FP4 ? __uint_as_float(r[j]) * alpha : __uint_as_float(r[j]);
        if (fl & ELFA_EPI_BIAS) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col + 8 > p.N) continue;
            float* w = v + g * 8;
            if (fl & ELFA_EPI_STORE_PREACT) {
              const uint4 o = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
              *reinterpret_cast<uint4*>(p.preact + (long long)row * p.ldpre + col) = o;
            }
            if (fl & ELFA_EPI_GELU) {
#pragma unroll
              for (int j = 0; j < 8; ++j) w[j] = gelu_tanh(w[j]);
            }
            const uint4 o = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
            *reinterpret_cast<uint4*>(p.C + (long long)row * p.ldc + col) = o;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (TWO) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0)); else mbar_arrive(tempty_bar(buf));
      }
    }
  } else if (AG) {
    // ------------------------------------------------------------------ push warps (6, 7)
    const int w = warp - 6;
    push_ranges(reinterpret_cast<const char*>(cm.peer_buf[cm.rank]), cm.peer_buf, cm.peer_flags, cm.rank, cm.world, cm.plan,
                smem_u32(smem + L::PUSH_OFF) + w * 2 * PUSH_PIECE, bar0 + 8u * (2 * STAGES + 4 + w * 2),
                bar0 + 8u * (2 * STAGES + 4 + w * 2 + 1), 1, w, lane, abort_flag, p.status);
  }

  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if (TWO) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// CTAs a launch of the given shape uses (the all-gather variant's arrival counters count them)
template <int BN, bool TWO>
int q_grid_ctas(int M, int N) {
  constexpr int TILE_M = TWO ? 2 * QBM : QBM;
  const int tiles = ((M + TILE_M - 1) / TILE_M) * ((N + BN - 1) / BN);
  const int slots = TWO ? device_sm_count() / 2 : device_sm_count();
  return (TWO ? 2 : 1) * (tiles < slots ? tiles : slots);
}

template <int BN, int STAGES, bool TWO, bool FP4 = false, bool AG = false>
int launch_q(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmSFA, const CUtensorMap& tmSFB, QParams p,
             cudaStream_t stream, const QComm* comm = nullptr) {
  using L = QSmem<BN, STAGES, TWO, FP4>;
  constexpr int TILE_M = TWO ? 2 * QBM : QBM;
  constexpr int DYN = AG ? L::DYN_AG : L::DYN;
  constexpr int NT = AG ? Q_THREADS_AG : Q_THREADS;
  static_assert(DYN <= 227 * 1024, "shared memory plan exceeds the per-CTA limit");
  auto kern = gemm_mxfp8_kernel<BN, STAGES, TWO, FP4, AG>;
  static bool configured = false;
  if (!configured) {
    ELFA_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN));
    configured = true;
  }
  QComm cm{};
  if (comm) cm = *comm;
  p.tiles_m = (p.M + TILE_M - 1) / TILE_M;
  p.tiles_n = (p.N + BN - 1) / BN;
  // rows of A that stay in L2 while the tile order sweeps over N: about 32 MB worth
  const long long rows = std::max(512LL, std::min(4096LL, (32LL << 20) / (long long)(FP4 ? p.K / 2 : p.K)));
  p.group_m = (int)std::max(1LL, rows / TILE_M);
  const int tiles = p.tiles_m * p.tiles_n;
  const int slots = TWO ? device_sm_count() / 2 : device_sm_count();
  const int grid = tiles < slots ? tiles : slots;
  if (TWO) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * grid, 1, 1);
    cfg.blockDim = dim3(NT, 1, 1);
    cfg.dynamicSmemBytes = DYN;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ELFA_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmSFA, tmSFB, p, cm));
  } else {
    kern<<<grid, NT, DYN, stream>>>(tmA, tmB, tmSFA, tmSFB, p, cm);
  }
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Tensor map over a scale tensor viewed as [atoms, 128] 32-bit words, box = `box_atoms` rows. Small cache:
// encoding costs a driver call and the same few tensors come back every step.
struct SfKey {
  const void* base;
  uint64_t atoms;
  uint32_t box;
  bool operator==(const SfKey& o) const { return base == o.base && atoms == o.atoms && box == o.box; }
};
struct SfKeyHash {
  size_t operator()(const SfKey& k) const { return reinterpret_cast<size_t>(k.base) * 1000003u ^ (k.atoms * 31u + k.box); }
};
std::mutex g_sf_mu;
std::unordered_map<SfKey, CUtensorMap, SfKeyHash> g_sf_cache;

int sf_tmap(CUtensorMap* out, const void* base, uint64_t atoms, uint32_t box_atoms) {
  const SfKey key{base, atoms, box_atoms};
  {
    std::lock_guard<std::mutex> lk(g_sf_mu);
    auto it = g_sf_cache.find(key);
    if (it != g_sf_cache.end()) {
      *out = it->second;
      return ELFA_OK;
    }
  }
  const int rc = make_tmap_2d(out, base, 4, atoms, 128, SF_ATOM, box_atoms, 128, false);
  if (rc != ELFA_OK) return rc;
  std::lock_guard<std::mutex> lk(g_sf_mu);
  if (g_sf_cache.size() > 4096) g_sf_cache.clear();
  g_sf_cache.emplace(key, *out);
  return ELFA_OK;
}

// ---- quantiser ------------------------------------------------------------------------------------
// Per 32-element block of a row: payload e4m3, scale byte into the atom layout, and an optional bf16
// copy of the dequantised values (what a fake-quantised bf16 GEMM would multiply).
__device__ __forceinline__ uint8_t mx_scale_q(float amax, float* scale, float* inv) {
  int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 - 8;
  if (amax == 0.f) e = -127;
  e = max(-127, min(127, e));
  *scale = __uint_as_float((uint32_t)(e + 127) << 23);
  if (e == -127) *scale = 5.877471754111438e-39f;
  *inv = e == -127 ? 1.7014118346046923e38f : __uint_as_float((uint32_t)(127 - e) << 23);
  return (uint8_t)(e + 127);
}

// Four adjacent lanes share one 32-element block: a thread owns 8 elements (one 16-byte load, one 8-byte
// payload store, one 16-byte store of the dequantised copy, all contiguous across the warp), the block's
// maximum comes from two shuffles, and the first lane of the four writes the scale byte.
__global__ void __launch_bounds__(256) mxfp8_quantize_gemm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                  uint8_t* __restrict__ payload, uint8_t* __restrict__ sf,
                                                                  __nv_bfloat16* __restrict__ deq, int rows, int cols, int kt,
                                                                  int b_atoms) {
  const uint32_t vpr = (uint32_t)cols / 8;             // vectors per row, a multiple of 4
  const uint32_t nvec = (uint32_t)rows * vpr;
  const uint32_t stride = gridDim.x * blockDim.x;      // a multiple of 32: lane % 4 == vector % 4
  const uint32_t lane = threadIdx.x & 31;
  for (uint32_t v = blockIdx.x * blockDim.x + threadIdx.x; v - lane < nvec; v += stride) {
    const bool ok = v < nvec;
    const uint32_t r = ok ? v / vpr : 0, c8 = ok ? v - r * vpr : 0;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (ok) q = *reinterpret_cast<const uint4*>(x + (long long)r * ldx + c8 * 8);
    const uint32_t pv[4] = {q.x, q.y, q.z, q.w};
    float f[8];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = bf16_lo(pv[j]);
      f[2 * j + 1] = bf16_hi(pv[j]);
      amax = fmaxf(amax, fmaxf(fabsf(f[2 * j]), fabsf(f[2 * j + 1])));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float sc, inv;
    const uint8_t sb = mx_scale_q(amax, &sc, &inv);
    uint32_t w[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint32_t acc = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) acc |= (uint32_t)__nv_cvt_float_to_fp8(f[i * 4 + j] * inv, __NV_SATFINITE, __NV_E4M3) << (8 * j);
      w[i] = acc;
    }
    if (ok) {
      *reinterpret_cast<uint2*>(payload + (long long)r * cols + c8 * 8) = make_uint2(w[0], w[1]);
      const uint32_t kb = c8 >> 2;
      if ((c8 & 3) == 0) {
        // atom order: A operand [row block][K tile]; B operand [K tile][row block (+1 pad)]
        const long long atom = b_atoms > 0 ? (long long)(kb >> 2) * b_atoms + (r >> 7) : (long long)(r >> 7) * kt + (kb >> 2);
        sf[atom * SF_ATOM + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3)] = sb;
      }
      if (deq != nullptr) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t two = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
          const float lo = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(two & 0xff), __NV_E4M3))) * sc;
          const float hi = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(two >> 8), __NV_E4M3))) * sc;
          o[j] = pack_bf16(lo, hi);
        }
        *reinterpret_cast<uint4*>(deq + (long long)r * cols + c8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// Inverse of the quantiser: out[r, c] = e4m3(payload[r, c]) * 2^(scale(r, c / 32) - 127) as bf16 (exact: three
// mantissa bits times a power of two). A thread converts 8 values (8-byte load, 16-byte store).
__global__ void __launch_bounds__(256) mxfp8_dequantize_kernel(const uint8_t* __restrict__ payload, const uint8_t* __restrict__ sf,
                                                               __nv_bfloat16* __restrict__ out, int rows, int cols, int kt,
                                                               int b_atoms) {
  const uint32_t vpr = (uint32_t)cols / 8;
  const uint32_t nvec = (uint32_t)rows * vpr;
  const uint32_t stride = gridDim.x * blockDim.x;
  for (uint32_t v = blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    const uint32_t r = v / vpr, c8 = v - r * vpr, kb = c8 >> 2;
    const uint2 q = *reinterpret_cast<const uint2*>(payload + (long long)r * cols + c8 * 8);
    const long long atom = b_atoms > 0 ? (long long)(kb >> 2) * b_atoms + (r >> 7) : (long long)(r >> 7) * kt + (kb >> 2);
    const uint32_t sb = sf[atom * SF_ATOM + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3)];
    const float sc = sb == 0 ? 5.877471754111438e-39f : __uint_as_float(sb << 23);
    const uint32_t w[2] = {q.x, q.y};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t two = (w[j >> 1] >> (16 * (j & 1))) & 0xffffu;
      const float lo = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(two & 0xff), __NV_E4M3))) * sc;
      const float hi = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)(two >> 8), __NV_E4M3))) * sc;
      o[j] = pack_bf16(lo, hi);
    }
    *reinterpret_cast<uint4*>(out + (long long)r * cols + c8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// Bytes of the scale tensor that belongs to a [rows, cols] operand.
ELFA_API long long elfa_mxfp8_sf_bytes(int rows, int cols, int b_operand) {
  return (long long)((rows + 127) / 128 + (b_operand ? 1 : 0)) * ((cols + 127) / 128) * SF_ATOM;
}

// x [rows, cols] bf16 (row pitch ldx elements) -> payload [rows, cols] e4m3 (dense), scale atoms, optional
// dequantised bf16 copy [rows, cols]. `b_operand` selects the atom order of the scales (A: [row block][K tile];
// B: [K tile][row block + 1 pad]). `sf` must be zero-filled by the caller when rows or cols are not multiples
// of 128 or for a B operand (entries of the padding are not written).
ELFA_API int elfa_mxfp8_quantize_gemm(const void* x, long long ldx, void* payload, void* sf, void* deq, int rows, int cols,
                                      int b_operand, void* stream) {
  ELFA_REQUIRE(x && payload && sf && rows > 0 && cols > 0, "mxfp8_quantize_gemm: bad arguments");
  ELFA_REQUIRE(cols % 32 == 0 && ldx % 8 == 0, "mxfp8_quantize_gemm: cols must be a multiple of 32 and the pitch of 8");
  const long long nv = (long long)rows * (cols / 8);
  ELFA_REQUIRE(nv < (1ll << 31) - (1 << 20), "mxfp8_quantize_gemm: tensor too large (2^34 elements at most)");
  const int grid = (int)((nv + 255) / 256 < 148 * 16 ? (nv + 255) / 256 : 148 * 16);
  mxfp8_quantize_gemm_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(payload), static_cast<uint8_t*>(sf),
      static_cast<__nv_bfloat16*>(deq), rows, cols, (cols + 127) / 128, b_operand ? (rows + 127) / 128 + 1 : 0);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}

// payload [rows, cols] e4m3 + scale atoms (order per `b_operand`) -> out [rows, cols] bf16, the values the block-scaled
// GEMM multiplies. Used where an operand arrives quantised (all-gather of payloads) and backward needs it in bf16.
ELFA_API int elfa_mxfp8_dequantize(const void* payload, const void* sf, void* out, int rows, int cols, int b_operand, void* stream) {
  ELFA_REQUIRE(payload && sf && out && rows > 0 && cols > 0 && cols % 32 == 0, "mxfp8_dequantize: bad arguments");
  const long long nv = (long long)rows * (cols / 8);
  ELFA_REQUIRE(nv < (1ll << 31) - (1 << 20), "mxfp8_dequantize: tensor too large (2^34 elements at most)");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(payload) & 7) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               "mxfp8_dequantize: payload must be 8-byte and out 16-byte aligned");
  const int grid = (int)((nv + 255) / 256 < 148 * 16 ? (nv + 255) / 256 : 148 * 16);
  mxfp8_dequantize_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(payload), static_cast<const uint8_t*>(sf), static_cast<__nv_bfloat16*>(out), rows, cols,
      (cols + 127) / 128, b_operand ? (rows + 127) / 128 + 1 : 0);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}

// C[M,N] bf16 = epilogue(A[M,K] * B[N,K]^T), e4m3 payloads with ue8m0 block scales (see the layout above).
// flags: ELFA_EPI_BIAS | ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT.
ELFA_API int elfa_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K,
                             long long ldc, const void* bias, void* preact, long long ldpre, unsigned flags, int force_bn,
                             void* stream) {
  ELFA_REQUIRE(A && B && C && sfa && sfb, "gemm_mxfp8: null operand");
  ELFA_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_mxfp8: empty problem");
  ELFA_REQUIRE(K % 32 == 0 && N % 8 == 0 && ldc % 8 == 0, "gemm_mxfp8: K must be a multiple of 32, N and ldc of 8");
  ELFA_REQUIRE(!(flags & ~(ELFA_EPI_BIAS | ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT)), "gemm_mxfp8: unsupported epilogue flag");
  ELFA_REQUIRE(!(flags & ELFA_EPI_BIAS) || bias, "gemm_mxfp8: bias flag without pointer");
  ELFA_REQUIRE(!(flags & ELFA_EPI_STORE_PREACT) || (preact && ldpre % 8 == 0), "gemm_mxfp8: preact flag without pointer");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(sfa) & 15) == 0 && (reinterpret_cast<uintptr_t>(sfb) & 15) == 0,
               "gemm_mxfp8: scale tensors must be 16-byte aligned");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm_mxfp8: no status word");
  // force_bn: 128 / 192 single-CTA tiles, 384 = CTA pairs on 256 x 192 tiles (the default for problems that fill at
  // least one wave of pairs). A 256 x 224 pair tile was tried and raised a misaligned-address fault on multi-tile
  // problems; it is not instantiated.
  const bool pair = force_bn == 384 ||
                    (force_bn == 0 && N > 128 && (long long)((M + 255) / 256) * ((N + 191) / 192) >= device_sm_count() / 2);
  const int BN = pair ? 192 : ((force_bn == 128 || force_bn == 192) ? force_bn : (N <= 128 ? 128 : 192));
  CUtensorMap tmA, tmB;
  int rc = shared_tmap(&tmA, A, 1, (uint64_t)M, (uint64_t)K, (uint64_t)K, QBM, QBK);
  if (rc != ELFA_OK) return rc;
  rc = shared_tmap(&tmB, B, 1, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)(pair ? BN / 2 : BN), QBK);
  if (rc != ELFA_OK) return rc;
  // scale tensors as [atoms, 128] 32-bit words; one box = the atoms of one tile and K tile
  const int kt = (K + QBK - 1) / QBK;
  const int natom_b = BN <= 128 ? 1 : (BN <= 192 ? 2 : 3);
  CUtensorMap tmSFA, tmSFB;
  rc = sf_tmap(&tmSFA, sfa, (uint64_t)((M + 127) / 128) * kt, 1);
  if (rc != ELFA_OK) return rc;
  rc = sf_tmap(&tmSFB, sfb, (uint64_t)((N + 127) / 128 + 1) * kt, (uint32_t)natom_b);
  if (rc != ELFA_OK) return rc;
  QParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.kt = (K + QBK - 1) / QBK;
  p.sfb_atoms = (N + 127) / 128;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.preact = static_cast<__nv_bfloat16*>(preact);
  p.ldpre = ldpre;
  p.flags = flags;
  p.status = st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pair) return launch_q<192, 7, true>(tmA, tmB, tmSFA, tmSFB, p, s);
  if (BN == 192) return launch_q<192, 5, false>(tmA, tmB, tmSFA, tmSFB, p, s);
  return launch_q<128, 6, false>(tmA, tmB, tmSFA, tmSFB, p, s);
}

// C[M,N] bf16 = epilogue(all_gather_rows(A)[M,K] * B[N,K]^T) with MXFP8 operands, one kernel. M = world * rows.
//   peer_buf   : host array of `world` device addresses of the ranks' gathered buffers (entry `rank` = this rank's own):
//                payload [M, K] e4m3 followed by the scale atoms of a left operand ([M / 128][K / 128] x 512 bytes).
//                This rank's rows and atoms must already be in ITS buffer (elfa_mxfp8_quantize_gemm into the slice);
//                the kernel sends them to the same offsets of every peer's buffer while it multiplies.
//   peer_flags / my_flags / arrivals_io : arrival counters as in elfa_gemm_ag.
// After the call this rank's buffer holds the whole gathered operand.
ELFA_API int elfa_gemm_ag_mxfp8(const unsigned long long* peer_buf, const unsigned long long* peer_flags, const void* my_flags,
                                unsigned int* arrivals_io, const void* B, const void* sfb, void* C, int M, int N, int K, long long ldc,
                                void* preact, long long ldpre, unsigned flags, int rank, int world, int wait_ms, void* stream) {
  ELFA_REQUIRE(peer_buf && peer_flags && my_flags && arrivals_io && B && sfb && C, "gemm_ag_mxfp8: null argument");
  ELFA_REQUIRE(world >= 2 && world <= MAX_RANKS && rank >= 0 && rank < world, "gemm_ag_mxfp8: bad rank/world");
  ELFA_REQUIRE(M % world == 0 && (M / world) % QBM == 0, "gemm_ag_mxfp8: rows per rank must be a multiple of 128");
  ELFA_REQUIRE(K % QBK == 0 && N % 8 == 0 && ldc % 8 == 0, "gemm_ag_mxfp8: K must be a multiple of 128, N and ldc of 8");
  ELFA_REQUIRE(!(flags & ~(ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT)), "gemm_ag_mxfp8: unsupported epilogue flag");
  ELFA_REQUIRE(!(flags & ELFA_EPI_STORE_PREACT) || (preact && ldpre % 8 == 0), "gemm_ag_mxfp8: preact flag without pointer");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(sfb) & 15) == 0, "gemm_ag_mxfp8: scale tensor must be 16-byte aligned");
  for (int i = 0; i < world; ++i) ELFA_REQUIRE((peer_buf[i] & 1023) == 0, "gemm_ag_mxfp8: gathered buffers must be 1024-byte aligned");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm_ag_mxfp8: no status word");
  const int rows = M / world;
  const int kt = K / QBK;
  const bool pair = N > 128 && rows % (2 * QBM) == 0 && (long long)(M / 256) * ((N + 191) / 192) >= device_sm_count() / 2;
  const int BN = (pair || N > 128) ? 192 : 128;
  const uint8_t* mine = reinterpret_cast<const uint8_t*>(peer_buf[rank]);
  const uint8_t* sfa = mine + (long long)M * K;
  CUtensorMap tmA, tmB, tmSFA, tmSFB;
  int rc = shared_tmap(&tmA, mine, 1, (uint64_t)M, (uint64_t)K, (uint64_t)K, QBM, QBK);
  if (rc != ELFA_OK) return rc;
  rc = shared_tmap(&tmB, B, 1, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)(pair ? BN / 2 : BN), QBK);
  if (rc != ELFA_OK) return rc;
  rc = sf_tmap(&tmSFA, sfa, (uint64_t)(M / 128) * kt, 1);
  if (rc != ELFA_OK) return rc;
  rc = sf_tmap(&tmSFB, sfb, (uint64_t)((N + 127) / 128 + 1) * kt, (uint32_t)(BN <= 128 ? 1 : 2));
  if (rc != ELFA_OK) return rc;
  QParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.sfa = sfa;
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.kt = kt;
  p.sfb_atoms = (N + 127) / 128;
  p.preact = static_cast<__nv_bfloat16*>(preact);
  p.ldpre = ldpre;
  p.flags = flags;
  p.status = st;
  QComm c{};
  c.rank = rank; c.world = world; c.rows_per_rank = rows;
  c.wait_cycles = wait_cycles_of(wait_ms);
  for (int i = 0; i < world; ++i) { c.peer_buf[i] = peer_buf[i]; c.peer_flags[i] = peer_flags[i]; }
  c.my_flags = static_cast<const unsigned int*>(my_flags);
  const long long pay_l = (long long)rows * K, sf_l = (long long)(rows / 128) * kt * SF_ATOM;
  c.plan.off[0] = (long long)rank * pay_l;
  c.plan.bytes[0] = pay_l;
  c.plan.off[1] = (long long)M * K + (long long)rank * sf_l;
  c.plan.bytes[1] = sf_l;
  c.plan.limit = (long long)M * K + (long long)world * sf_l;
  const int ctas = pair ? q_grid_ctas<192, true>(M, N) : (BN == 192 ? q_grid_ctas<192, false>(M, N) : q_grid_ctas<128, false>(M, N));
  *arrivals_io += (unsigned)ctas;                  // every CTA of a source bumps the counter once
  c.flag_target = *arrivals_io;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pair) return launch_q<192, 6, true, false, true>(tmA, tmB, tmSFA, tmSFB, p, s, &c);
  if (BN == 192) return launch_q<192, 4, false, false, true>(tmA, tmB, tmSFA, tmSFB, p, s, &c);
  return launch_q<128, 5, false, false, true>(tmA, tmB, tmSFA, tmSFB, p, s, &c);
}

// ---- NVFP4 ------------------------------------------------------------------------------------------
namespace elfa {
namespace {

// One thread per 16-element block: e2m1 payload (two values per byte, even element in the low nibble),
// ue4m3 block scale into the atom layout (an atom covers 128 rows x 64 K-elements), optional bf16 copy
// of the dequantised values. tensor scale = amax_tensor / (448 * 6), as in the fake-quant kernel.
__global__ void __launch_bounds__(256) nvfp4_quantize_gemm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                                  uint8_t* __restrict__ payload, uint8_t* __restrict__ sf,
                                                                  __nv_bfloat16* __restrict__ deq, int rows, int cols, int k64_stride,
                                                                  int b_atoms, const float* __restrict__ tensor_amax) {
  const float ta = *tensor_amax;
  const float ts = ta > 0.f ? ta / (448.f * 6.f) : 1.f;
  const int bpr = cols / 16;
  const long long nblocks = (long long)rows * bpr;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long blk = (long long)blockIdx.x * blockDim.x + threadIdx.x; blk < nblocks; blk += stride) {
    const int r = (int)(blk / bpr), kb = (int)(blk - (long long)r * bpr);
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ldx + kb * 16);
    float f[16];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 v = src[i];
      const uint32_t pv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[i * 8 + 2 * j] = bf16_lo(pv[j]);
        f[i * 8 + 2 * j + 1] = bf16_hi(pv[j]);
        amax = fmaxf(amax, fmaxf(fabsf(f[i * 8 + 2 * j]), fabsf(f[i * 8 + 2 * j + 1])));
      }
    }
    const __nv_fp8_storage_t sbq = __nv_cvt_float_to_fp8(amax / (6.f * ts), __NV_SATFINITE, __NV_E4M3);
    const float sb = __half2float(__half(__nv_cvt_fp8_to_halfraw(sbq, __NV_E4M3)));
    const float full = sb * ts;
    const float inv = full > 0.f ? 1.f / full : 0.f;
    uint32_t w[2] = {0u, 0u};
    float dq[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const __nv_fp4_storage_t q = __nv_cvt_float_to_fp4(f[i] * inv, __NV_E2M1, cudaRoundNearest);
      w[i >> 3] |= (uint32_t)(q & 0xf) << (4 * (i & 7));
      dq[i] = __half2float(__half(__nv_cvt_fp4_to_halfraw(q, __NV_E2M1))) * full;
    }
    *reinterpret_cast<uint2*>(payload + (long long)r * (cols / 2) + kb * 8) = make_uint2(w[0], w[1]);
    const long long atom = b_atoms > 0 ? (long long)(kb >> 2) * b_atoms + (r >> 7) : (long long)(r >> 7) * k64_stride + (kb >> 2);
    sf[atom * SF_ATOM + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3)] = (uint8_t)sbq;
    if (deq != nullptr) {
      uint4* dd = reinterpret_cast<uint4*>(deq + (long long)r * cols + kb * 16);
      dd[0] = make_uint4(pack_bf16(dq[0], dq[1]), pack_bf16(dq[2], dq[3]), pack_bf16(dq[4], dq[5]), pack_bf16(dq[6], dq[7]));
      dd[1] = make_uint4(pack_bf16(dq[8], dq[9]), pack_bf16(dq[10], dq[11]), pack_bf16(dq[12], dq[13]), pack_bf16(dq[14], dq[15]));
    }
  }
}

}  // namespace
}  // namespace elfa

// Bytes of the scale tensor of a [rows, cols] NVFP4 operand: atoms of 128 rows x 64 K-elements, the K extent
// padded to a multiple of 256 (one pipeline stage), one extra row block of padding for a B operand.
ELFA_API long long elfa_nvfp4_sf_bytes(int rows, int cols, int b_operand) {
  return (long long)((rows + 127) / 128 + (b_operand ? 1 : 0)) * ((cols + 255) / 256 * 4) * SF_ATOM;
}

// x [rows, cols] bf16 -> payload [rows, cols / 2] (two e2m1 per byte), ue4m3 scale atoms, optional dequantised
// bf16 copy. tensor_amax: device pointer to max |x| (see elfa_amax). `sf` must be zero-filled by the caller.
ELFA_API int elfa_nvfp4_quantize_gemm(const void* x, long long ldx, void* payload, void* sf, void* deq, int rows, int cols,
                                      int b_operand, const float* tensor_amax, void* stream) {
  ELFA_REQUIRE(x && payload && sf && tensor_amax && rows > 0 && cols > 0, "nvfp4_quantize_gemm: bad arguments");
  ELFA_REQUIRE(cols % 32 == 0 && ldx % 8 == 0, "nvfp4_quantize_gemm: cols must be a multiple of 32 and the pitch of 8");
  const long long nb = (long long)rows * (cols / 16);
  const int grid = (int)((nb + 255) / 256 < 148 * 16 ? (nb + 255) / 256 : 148 * 16);
  nvfp4_quantize_gemm_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<uint8_t*>(payload), static_cast<uint8_t*>(sf),
      static_cast<__nv_bfloat16*>(deq), rows, cols, (cols + 255) / 256 * 4, b_operand ? (rows + 127) / 128 + 1 : 0, tensor_amax);
  ELFA_CUDA(cudaGetLastError());
  count_launches(1);
  return ELFA_OK;
}

// C[M,N] bf16 = epilogue(s_a * s_b * A[M,K] * B[N,K]^T): e2m1 payloads, ue4m3 scales per 16 K-elements, fp32 tensor
// scales s = amax / (448 * 6) read from device memory. flags: ELFA_EPI_BIAS | ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT.
ELFA_API int elfa_gemm_nvfp4(const void* A, const void* sfa, const float* amax_a, const void* B, const void* sfb, const float* amax_b,
                             void* C, int M, int N, int K, long long ldc, const void* bias, void* preact, long long ldpre,
                             unsigned flags, int force_bn, void* stream) {
  ELFA_REQUIRE(A && B && C && sfa && sfb && amax_a && amax_b, "gemm_nvfp4: null operand");
  ELFA_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_nvfp4: empty problem");
  ELFA_REQUIRE(K % 32 == 0 && N % 8 == 0 && ldc % 8 == 0, "gemm_nvfp4: K must be a multiple of 32, N and ldc of 8");
  ELFA_REQUIRE(!(flags & ~(ELFA_EPI_BIAS | ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT)), "gemm_nvfp4: unsupported epilogue flag");
  ELFA_REQUIRE(!(flags & ELFA_EPI_BIAS) || bias, "gemm_nvfp4: bias flag without pointer");
  ELFA_REQUIRE(!(flags & ELFA_EPI_STORE_PREACT) || (preact && ldpre % 8 == 0), "gemm_nvfp4: preact flag without pointer");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(sfa) & 15) == 0 && (reinterpret_cast<uintptr_t>(sfb) & 15) == 0,
               "gemm_nvfp4: scale tensors must be 16-byte aligned");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm_nvfp4: no status word");
  const int BN = force_bn == 128 ? 128 : (N <= 128 ? 128 : 192);
  const uint64_t kbytes = (uint64_t)K / 2;
  CUtensorMap tmA, tmB, tmSFA, tmSFB;
  int rc = shared_tmap(&tmA, A, 1, (uint64_t)M, kbytes, kbytes, QBM, QBK);
  if (rc != ELFA_OK) return rc;
  rc = shared_tmap(&tmB, B, 1, (uint64_t)N, kbytes, kbytes, (uint32_t)BN, QBK);
  if (rc != ELFA_OK) return rc;
  const int kt = (int)((kbytes + QBK - 1) / QBK);          // pipeline stages along K (256 elements each)
  const int natom_b = BN <= 128 ? 1 : 2;
  rc = sf_tmap(&tmSFA, sfa, (uint64_t)((M + 127) / 128) * kt * 4, 4);
  if (rc != ELFA_OK) return rc;
  rc = sf_tmap(&tmSFB, sfb, (uint64_t)((N + 127) / 128 + 1) * kt * 4, (uint32_t)natom_b);
  if (rc != ELFA_OK) return rc;
  QParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.sfa = static_cast<const uint8_t*>(sfa);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.kt = kt;
  p.sfb_atoms = (N + 127) / 128;
  p.amax_a = amax_a;
  p.amax_b = amax_b;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.preact = static_cast<__nv_bfloat16*>(preact);
  p.ldpre = ldpre;
  p.flags = flags;
  p.status = st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (BN == 192) return launch_q<192, 4, false, true>(tmA, tmB, tmSFA, tmSFB, p, s);
  return launch_q<128, 5, false, true>(tmA, tmB, tmSFA, tmSFB, p, s);
}
