// Persistent warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory ring -> tcgen05.mma with
// fp32 accumulators in tensor memory (double buffered) -> tcgen05.ld epilogue with fused
// bias / GELU / dGELU / residual / accumulate.
//
// Replaces the reference's cuBLAS wrapper and its one-thread-per-output "sm100" GEMM
// (reference: kernels/cuda/gemm.cu:212-232,315-327,412-423 forward/backward through cublasGemmEx;
// kernels/cuda/gemm_sm100.cu:46-72 naive bf16 kernel, :142-171 static tile table;
// kernels/cuda/gemm.cu:50-72 bias add and column sum).
//
// C[M,N] = epilogue(alpha * A * B) where each operand is given either
//   K-major  : A as [M,K] row-major / B as [N,K] row-major  (contraction index contiguous), or
//   MN-major : A as [K,M] row-major / B as [K,N] row-major  (output index contiguous).
// This covers forward (x[M,K] * W[K,N]), input gradient (dy[M,N] * W[K,N]^T) and weight gradient
// (x[M,K]^T * dy[M,N]) of a Linear layer without materialising any transpose.
//
// Roles per CTA (192 threads, one CTA per SM, grid = min(tiles, SMs)):
//   warp 0   : TMA producer (one lane) - fills a STAGES-deep ring of {A 128x64, B BNx64} bf16 tiles
//   warp 1   : allocates tensor memory; one lane issues tcgen05.mma (128 x BN x 16 per instruction)
//   warps 2-5: epilogue - each owns one 32-lane quarter of the accumulator
// Every wait is bounded; on a timeout the CTA sets the device status word, stops and tears down.
//
// Fused collectives (tensor + sequence parallel layers; reference call sites
// src/distributed/tensor_parallel.zig:77-129, src/distributed/sequence_parallel.zig:79-128 gather then
// GEMM, tensor_parallel.zig:154-170 / sequence_parallel.zig:184-200 GEMM then reduce), COMM template:
//   COMM_AG: A = all_gather_rows(x_local). Two extra warps push this rank's shard into every peer's
//            gathered buffer (plain stores over NVLink, one peer after the other, then a release
//            increment of that peer's arrival counter). Tiles are scheduled own shard first, then
//            the shards in the order they arrive; the TMA producer waits for a shard's counter
//            before its first tile. Remote data crosses NVLink once, into local memory; the TMA
//            loads themselves are always local and never cluster-multicast.
//   COMM_RS: C = reduce_scatter_rows(A B). The epilogue stores each partial tile into the owner
//            rank's receive slot [source rank] (peer stores), tiles of other owners first, and
//            bumps the owner's counter. After its tiles every CTA helps to sum the slots of the
//            rows this rank owns, in fixed rank order (deterministic), once all counters arrived.
#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "comm.cuh"
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 288;   // 9 warps: TMA, MMA, 4 epilogue, store, 2 push (all-gather variant only)

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux;
  long long ldaux;
  __nv_bfloat16* preact;
  long long ldpre;
  float alpha;
  unsigned flags;
  unsigned int* status;
  int tiles_m, tiles_n, group_m;
  int staged;        // epilogue goes through shared memory + TMA store (plain bf16 output)
  int splits;        // split-K factor (fp32 accumulate outputs only; partial tiles are added atomically)
  int kb_per_split;  // K blocks per split
  int sfb_atoms;     // MXFP8: row blocks of the B scale tensor
};

enum { COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2, COMM_GB = 3 };

struct CommParams {
  int rank, world;
  int rows_per_rank;                       // M / world, a multiple of BM
  long long wait_cycles;                   // limit of every flag wait
  // all-gather of A
  const __nv_bfloat16* x_local;            // [rows_per_rank, K]
  long long ldx;
  int piece_bytes, pieces_per_row;         // a row of x_local is pushed in `pieces_per_row` pieces of `piece_bytes` (<= 8 KB, x16)
  unsigned long long peer_xfull[MAX_RANKS];   // peers' gathered-A buffers [M, K] (ld = K)
  unsigned long long peer_flags[MAX_RANKS];   // peers' counters, one u32 per source rank
  const unsigned int* my_flags;            // this rank's counters
  unsigned int flag_target;                // value a counter reaches when the source's push is complete
  // reduce-scatter of C
  unsigned long long peer_recv[MAX_RANKS];    // peers' receive buffers [world][rows_per_rank][N] bf16
  const __nv_bfloat16* my_recv;
  __nv_bfloat16* rs_out;                   // [rows_per_rank, N]
  long long ld_out;
  // chunk-major receive slots: every staged 128-row x 64-column chunk (16 KB, 128-byte swizzled as it lies in shared
  // memory) travels as ONE contiguous bulk copy and lands at chunk index ((row block * tiles_n + nb) * chunks per tile + cc)
  // of the source's slot; the reduce phase undoes the permutation. Row-major slots (TMA tensor stores, 128-byte row
  // segments) when 0.
  int chunk_major;
  long long slot_chunks;                   // chunks per source slot
  // gather of B (COMM_GB): B is a parameter that lies sharded over the ranks - bytes [gb_w_off, gb_w_off + gb_w_bytes) of a
  // bucket whose rank r holds bytes [r * gb_shard_bytes, (r + 1) * gb_shard_bytes) at gb_src[r] (peer addressable). Two warps
  // per CTA copy the parameter's pieces into the local full-size bucket at gb_dst (bulk loads from the owners, bulk stores to
  // local memory) and raise the LOCAL counter gb_flags[r] once per CTA and owner; the TMA producer waits for the owners of
  // the B rows of a K block before it loads them.
  unsigned long long gb_src[MAX_RANKS];
  char* gb_dst;
  long long gb_w_off, gb_w_bytes, gb_shard_bytes, gb_row_bytes;
  unsigned int* gb_flags;
  unsigned int gb_target;
  int gb_kb_rot;                           // the K loop starts at this K block (the first one inside this rank's own part) and wraps
};

// SF: bytes of scale atoms per stage (block-scaled MXFP8 operands: one atom of A scales + the atoms of B scales; 0 for bf16)
template <int BN, int STAGES, int SF = 0>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;      // bf16: 128 rows x 64 elements; MXFP8: 128 rows x 128 one-byte elements
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int SF_BYTES = SF;
  static constexpr int SF_OFF = STAGES * (A_BYTES + B_BYTES);
  static constexpr int BAR_OFF = SF_OFF + STAGES * SF_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4 + 4;   // ring full/empty, accumulator full/empty, push buffers (all-gather variant)
  static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16;
  static constexpr int DYN = TOTAL + 1024;  // slack for manual 1024-byte alignment
  // reduce-scatter variant: two [128 x 64] bf16 staging tiles for the TMA stores to the owner rank
  static constexpr int OUT_OFF = (TOTAL + 1023) / 1024 * 1024;
  static constexpr int OUT_BYTES = 2 * BM * 128;
  static constexpr int DYN_RS = OUT_OFF + OUT_BYTES + 1024;
};

struct OutMaps {   // tensor maps over every rank's receive buffer, viewed as [world * rows_per_rank, N] bf16
  CUtensorMap m[MAX_RANKS];
  CUtensorMap sfa, sfb;   // MXFP8 operands: scale atoms of A / B as rows of 128 32-bit words (see gemm_mxfp8.cu)
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& mb, int& nb) {
  int per_group = p.group_m * p.tiles_n;
  int g = tile / per_group;
  int first_m = g * p.group_m;
  int gsz = min(p.group_m, p.tiles_m - first_m);
  int r = tile - g * per_group;
  mb = first_m + r % gsz;
  nb = r / gsz;
}

// Tile order of the fused variants: tiles are grouped by the rank that owns their rows ("shard").
// COMM_AG visits the own shard first, then rank-1, rank-2, ... (the order in which pushes arrive);
// COMM_RS visits rank+1, rank+2, ... and the own shard last (its partial does not travel).
template <int COMM>
__device__ __forceinline__ void tile_coords_comm(const GemmParams& p, const CommParams& c, int tile, int& mb, int& nb, int& shard,
                                                 int tile_m = BM) {
  if (COMM == COMM_NONE || COMM == COMM_GB) {
    tile_coords(p, tile, mb, nb);
    shard = 0;
    return;
  }
  const int tm_shard = c.rows_per_rank / tile_m;   // tiles (of tile_m rows: 128, or 256 for CTA pairs) per shard
  const int per_shard = tm_shard * p.tiles_n;
  const int i = tile / per_shard;
  const int lt = tile - i * per_shard;
  shard = COMM == COMM_AG ? (c.rank - i + c.world) % c.world : (c.rank + 1 + i) % c.world;
  mb = shard * tm_shard + lt % tm_shard;
  nb = lt / tm_shard;
}

// TWO: the CTAs of a 2-CTA cluster work as a pair on 256 x BN tiles (tcgen05 cta_group::2). Each CTA
// loads its 128 rows of A and its half of B (BN / 2 rows), the even CTA issues one MMA for both, and
// each CTA ends up with its 128 rows of the accumulator in its own tensor memory. Per CTA this
// needs a third less shared-memory fill per FLOP than a 128 x BN tile. In the fused variants a pair's 256 rows lie
// inside one rank's shard (rows per rank a multiple of 256); flags, pushes and the reduce phase work per CTA as before.
// MX = true: block-scaled MXFP8 operands (e4m3 payloads, both K-major, one ue8m0 scale per 32 K-elements in 512-byte atoms,
// tcgen05.mma.kind::mxf8f6f4.block_scale with the scales in tensor memory) through the same roles: used by the fused
// GEMM -> reduce-scatter kernel of the MXFP8 layers. A stage then holds 128 K-elements (= bytes) per row plus the scale
// atoms; accumulator b sits at tensor-memory column 256 * b with the scale columns behind it (BN <= 192).
template <int BN, bool A_MN, bool B_MN, int STAGES, int COMM, bool TWO = false, bool MX = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const GemmParams p, const CommParams cm,
                 const __grid_constant__ OutMaps om) {
  constexpr int BN_CTA = TWO ? BN / 2 : BN;   // rows of B this CTA keeps in shared memory
  constexpr int TILE_M = TWO ? 2 * BM : BM;   // rows of one work unit
  constexpr int NATOM = BN <= 128 ? 1 : 2;                 // B scale atoms a tile touches (tiles start 0 or 64 rows into an atom)
  constexpr int SF_ATOM = 512;
  using L = SmemLayout<BN_CTA, STAGES, MX ? (1 + NATOM) * SF_ATOM : 0>;
  static_assert(!MX || (!A_MN && !B_MN && BN <= 192), "block-scaled operands are K-major and leave room for the scale columns");
  constexpr int KSTEP = MX ? 128 : BK;                     // contraction elements per stage
  constexpr uint32_t ACC_STRIDE = MX ? 256 : BN;           // tensor-memory columns between the two accumulators
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * L::A_BYTES;
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
  constexpr uint32_t TMEM_COLS = MX ? 512 : 2 * BN;  // 128 / 256 / 512: a power of two >= 32
  const uint32_t cta_rank = TWO ? cluster_ctarank() : 0u;                       // position in the pair; 0 issues the MMAs
  const int wid = TWO ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;               // work slot: one per CTA, or one per pair
  const int wstride = TWO ? (int)(gridDim.x >> 1) : (int)gridDim.x;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), TWO ? 8 : 4);   // pair: the epilogue warps of both CTAs release the even CTA's barrier
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
  if (TWO) cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + KSTEP - 1) / KSTEP;
  const bool staged = COMM == COMM_RS || p.staged != 0;
  const int splits = COMM == COMM_NONE ? p.splits : 1;
  const int num_units = num_tiles * splits;   // work unit = (tile, K split)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int ready_shard = -1;
      uint32_t gb_ready = 0;            // COMM_GB: owners whose part of B is known to be in place
      for (int unit = wid; unit < num_units && ok; unit += wstride) {
        const int tile = unit / splits;
        const int kb0 = (unit - tile * splits) * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        int mb, nb, shard;
        tile_coords_comm<COMM>(p, cm, tile, mb, nb, shard, TILE_M);
        if (!bounds_ok(mb, p.tiles_m, p.status) || !bounds_ok(nb, p.tiles_n, p.status) || !bounds_ok(shard, COMM == COMM_NONE ? 1 : cm.world, p.status)) {
          *abort_flag = 1;     // checked build: a tile outside the grid ends the CTA (every role sees the flag)
          break;
        }
        const int m0 = mb * TILE_M + (int)cta_rank * BM, n0 = nb * BN;
        const bool own = COMM == COMM_AG && shard == cm.rank;
        if (COMM == COMM_AG && !own && shard != ready_shard) {
          // the shard was written by a peer GPU with ordinary stores: acquire its counter, then
          // order those writes before this thread's TMA (async proxy) reads
          if (!flag_wait(cm.my_flags + shard, cm.flag_target, cm.wait_cycles, abort_flag, p.status)) { ok = false; break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");
          ready_shard = shard;
        }
        for (int kb_seq = kb0; kb_seq < kb1; ++kb_seq, ++it) {
          int kb = kb_seq;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (COMM == COMM_GB) {
            // the K blocks are visited own part first, then in the order in which the copy warps fetch the other owners'
            // parts (a sum over K may start anywhere); the MMA warp only counts blocks
            kb = (kb_seq + cm.gb_kb_rot) % num_kb;
            // rows [kb * BK, kb * BK + BK) of B: the ranks that own those bytes of the bucket must have been copied in
            const long long lo = cm.gb_w_off + (long long)kb * BK * cm.gb_row_bytes;
            long long hi = lo + (long long)BK * cm.gb_row_bytes;
            if (hi > cm.gb_w_off + cm.gb_w_bytes) hi = cm.gb_w_off + cm.gb_w_bytes;
            const int r_lo = (int)(lo / cm.gb_shard_bytes), r_hi = (int)((hi - 1) / cm.gb_shard_bytes);
            for (int r = r_lo; r <= r_hi && ok; ++r) {
              if (gb_ready & (1u << r)) continue;
              if (!bounds_ok(r, cm.world, p.status) || !flag_wait(cm.gb_flags + r, cm.gb_target, cm.wait_cycles, abort_flag, p.status)) { ok = false; break; }
              asm volatile("fence.proxy.async.global;" ::: "memory");   // the copies were bulk stores of other warps / CTAs
              gb_ready |= 1u << r;
            }
            if (!ok) break;
          }
          if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, p.status)) { ok = false; break; }
          const uint32_t a_dst = smem_u32(sA + s * L::A_BYTES);
          const uint32_t b_dst = smem_u32(sB + s * L::B_BYTES);
          if (MX) {
            // payload tiles (128 bytes of K per row) and the scale atoms of this tile and K tile
            const uint32_t sf_dst = smem_u32(smem + L::SF_OFF + s * L::SF_BYTES);
            const int sfa_row = (m0 / BM) * num_kb + kb, sfb_row = kb * (p.sfb_atoms + 1) + n0 / 128;
            constexpr uint32_t TX = L::A_BYTES + L::B_BYTES + L::SF_BYTES;
            if (TWO) {
              const uint32_t fb = map_to_cta(full_bar(s), 0);
              if (cta_rank == 0) mbar_expect_tx(full_bar(s), 2 * TX);
              tma_load_2d_pair(a_dst, &tmA, kb * KSTEP, m0, fb);
              tma_load_2d_pair(b_dst, &tmB, kb * KSTEP, n0 + (int)cta_rank * BN_CTA, fb);
              tma_load_2d_pair(sf_dst, &om.sfa, 0, sfa_row, fb);
              tma_load_2d_pair(sf_dst + SF_ATOM, &om.sfb, 0, sfb_row, fb);
            } else {
              mbar_expect_tx(full_bar(s), TX);
              tma_load_2d(a_dst, &tmA, kb * KSTEP, m0, full_bar(s));
              tma_load_2d(b_dst, &tmB, kb * KSTEP, n0, full_bar(s));
              tma_load_2d(sf_dst, &om.sfa, 0, sfa_row, full_bar(s));
              tma_load_2d(sf_dst + SF_ATOM, &om.sfb, 0, sfb_row, full_bar(s));
            }
            continue;
          }
          if (TWO) {
            // both CTAs' copies complete on the even CTA's barrier, which expects the bytes of both
            const uint32_t fb = map_to_cta(full_bar(s), 0);
            if (cta_rank == 0) mbar_expect_tx(full_bar(s), 2 * (L::A_BYTES + L::B_BYTES));
            const int nB = n0 + (int)cta_rank * BN_CTA;
            if (own) {
              tma_load_2d_pair(a_dst, &tmA2, kb * BK, m0 - cm.rank * cm.rows_per_rank, fb);
            } else if (!A_MN) {
              tma_load_2d_pair(a_dst, &tmA, kb * BK, m0, fb);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(a_dst + j * 8192, &tmA, m0 + j * 64, kb * BK, fb);
            }
            if (!B_MN) {
              tma_load_2d_pair(b_dst, &tmB, kb * BK, nB, fb);
            } else {
#pragma unroll
              for (int j = 0; j < BN_CTA / 64; ++j) tma_load_2d_pair(b_dst + j * 8192, &tmB, nB + j * 64, kb * BK, fb);
            }
            continue;
          }
          mbar_expect_tx(full_bar(s), L::A_BYTES + L::B_BYTES);
          if (own) {
            tma_load_2d(a_dst, &tmA2, kb * BK, m0 - cm.rank * cm.rows_per_rank, full_bar(s));
          } else if (!A_MN) {
            tma_load_2d(a_dst, &tmA, kb * BK, m0, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, m0 + j * 64, kb * BK, full_bar(s));
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tmB, kb * BK, n0, full_bar(s));
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, n0 + j * 64, kb * BK, full_bar(s));
          }
        }
      }
      if (!ok) {
        // give the copies already issued a bounded chance to land before the CTA exits
        for (uint32_t j = it > (uint32_t)STAGES ? it - STAGES : 0; j < it; ++j) {
          const long long t0 = clock64();
          while (!mbar_try(full_bar(j % STAGES), (j / STAGES) & 1) && clock64() - t0 < 4000000) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the loop (converged); one elected lane issues the tensor-core instructions.
    if (cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TILE_M, BN, A_MN, B_MN);
      uint32_t it = 0, tile_iter = 0;
      bool ok = true;
      for (int unit = wid; unit < num_units && ok; unit += wstride, ++tile_iter) {
        const int kb0 = (unit % splits) * p.kb_per_split, kb1 = min(num_kb, kb0 + p.kb_per_split);
        const uint32_t buf = tile_iter & 1, bph = (tile_iter >> 1) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(buf), bph ^ 1, abort_flag, p.status));
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * ACC_STRIDE;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, abort_flag, p.status));
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(sA + s * L::A_BYTES);
          const uint32_t b_base = smem_u32(sB + s * L::B_BYTES);
          if (MX) {
            // scale atoms -> tensor memory (two column sets alternate between K tiles), then four block-scaled MMAs of
            // 32 K-elements each; byte k of the scale columns belongs to MMA k (selected through the descriptor)
            const uint32_t sf_base = smem_u32(smem + L::SF_OFF + s * L::SF_BYTES);
            const uint32_t sf_tmem = tmem_base + (it & 1u) * ACC_STRIDE;
            constexpr uint32_t SFA_COL = BN, SFB_COL = BN + 4;
            int mb_, nb_, sh_;
            tile_coords_comm<COMM>(p, cm, unit / splits, mb_, nb_, sh_, TILE_M);
            const uint32_t sfb_shift = (uint32_t)((nb_ * BN) % 128) / 32;
            if (elect_one()) {
              if (TWO) tc_cp_32x128b_warpx4_pair(sf_tmem + SFA_COL, make_smem_desc(sf_base, 0, 128, 0));
              else tc_cp_32x128b_warpx4(sf_tmem + SFA_COL, make_smem_desc(sf_base, 0, 128, 0));
#pragma unroll
              for (int j = 0; j < NATOM; ++j) {
                if (TWO) tc_cp_32x128b_warpx4_pair(sf_tmem + SFB_COL + 4 * j, make_smem_desc(sf_base + (1 + j) * SF_ATOM, 0, 128, 0));
                else tc_cp_32x128b_warpx4(sf_tmem + SFB_COL + 4 * j, make_smem_desc(sf_base + (1 + j) * SF_ATOM, 0, 128, 0));
              }
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint64_t da = make_smem_desc(a_base + k * 32, 16, 1024, 2);
                const uint64_t db = make_smem_desc(b_base + k * 32, 16, 1024, 2);
                const uint32_t acc = ((kb - kb0) | k) != 0 ? 1u : 0u;
                if (TWO) tc_mma_mxf8_pair(tmem_d, da, db, make_idesc_mxf8(TILE_M, BN, k, k), acc, sf_tmem + SFA_COL, sf_tmem + SFB_COL + sfb_shift);
                else tc_mma_mxf8(tmem_d, da, db, make_idesc_mxf8(TILE_M, BN, k, k), acc, sf_tmem + SFA_COL, sf_tmem + SFB_COL + sfb_shift);
              }
              if (TWO) tc_commit_pair(empty_bar(s)); else tc_commit(empty_bar(s));
            }
            __syncwarp();
            continue;
          }
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              // K-major: 16 elements = 32 bytes along the swizzled 128-byte row.
              // MN-major: 16 K-rows of 128 bytes = two 1024-byte swizzle atoms.
              const uint64_t da = A_MN ? make_smem_desc(a_base + k * 2048, 8192, 1024, 2)
                                       : make_smem_desc(a_base + k * 32, 16, 1024, 2);
              const uint64_t db = B_MN ? make_smem_desc(b_base + k * 2048, 8192, 1024, 2)
                                       : make_smem_desc(b_base + k * 32, 16, 1024, 2);
              if (TWO) tc_mma_f16_pair(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
              else tc_mma_f16(tmem_d, da, db, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
            }
            // frees the smem slot (in both CTAs of a pair) once these MMAs have read it
            if (TWO) tc_commit_pair(empty_bar(s)); else tc_commit(empty_bar(s));
          }
          __syncwarp();
        }
        if (ok && elect_one()) {
          if (TWO) tc_commit_pair(tfull_bar(buf)); else tc_commit(tfull_bar(buf));
        }
        __syncwarp();
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    uint32_t tile_iter = 0;
    const unsigned fl = p.flags;
    bool dead = false;
    for (int unit = wid; unit < num_units; unit += wstride, ++tile_iter) {
      const int tile = unit / splits;
      int mb, nb, shard;
      tile_coords_comm<COMM>(p, cm, tile, mb, nb, shard, TILE_M);
      const int m0 = mb * TILE_M + (int)cta_rank * BM, n0 = nb * BN;
      const uint32_t buf = tile_iter & 1, bph = (tile_iter >> 1) & 1;
      bool ok = !dead && mbar_wait(tfull_bar(buf), bph, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (!staged) break;
        dead = true;   // staged epilogue: keep walking the tiles so the named barriers shared with the store warp stay balanced
      }
      tc_fence_after();
      if (staged) {
        // tile -> shared staging (128-byte swizzle); warp 6 sends each staged 128-row x 128-byte chunk with
        // a TMA store / reduce-add (to the owner rank in the reduce-scatter variant), so these warps never
        // wait for the stores. A chunk is 64 bf16 or 32 fp32 columns = 32 accumulator columns per 64 bytes.
        // named barriers: 2 + buf = "chunk staged", 4 + buf = "staging buffer free again"
        const uint32_t out0 = smem_u32(smem + L::OUT_OFF);
        const int rloc = q * 32 + lane;
        const bool f32 = p.staged == 2;
        const int nchunk = f32 ? BN / 32 : BN / 64;
        const uint32_t tcol0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * ACC_STRIDE;
        uint32_t ra[32], rb[32];
        if (!dead) tmem_ld32(tcol0, ra);                           // first 32 accumulator columns in flight
#pragma unroll 1
        for (int cc = 0; cc < nchunk; ++cc) {
          const uint32_t g = tile_iter * nchunk + cc;              // running chunk number of this CTA
          const uint32_t sbuf = out0 + (g & 1) * (BM * 128);
          const uint32_t srow = sbuf + rloc * 128;
          if (g >= 2) named_bar_sync(4 + (g & 1), 160);
          if (!dead) {
            if (f32) {
              tmem_ld_wait();
              if (cc > 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) ra[j] = rb[j];
              }
              if (cc + 1 < nchunk) tmem_ld32(tcol0 + (cc + 1) * 32, rb);   // prefetch the next chunk
#pragma unroll
              for (int gq = 0; gq < 8; ++gq) {
                const uint32_t addr = srow + ((gq ^ (rloc & 7)) << 4);
                const float x0 = __uint_as_float(ra[gq * 4 + 0]) * p.alpha, x1 = __uint_as_float(ra[gq * 4 + 1]) * p.alpha;
                const float x2 = __uint_as_float(ra[gq * 4 + 2]) * p.alpha, x3 = __uint_as_float(ra[gq * 4 + 3]) * p.alpha;
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(x0), "f"(x1), "f"(x2), "f"(x3) : "memory");
              }
            } else {
              tmem_ld_wait();
              tmem_ld32(tcol0 + cc * 64 + 32, rb);                  // second half of this chunk
#pragma unroll
              for (int hf = 0; hf < 2; ++hf) {
                if (hf == 1) {
                  tmem_ld_wait();
#pragma unroll
                  for (int j = 0; j < 32; ++j) ra[j] = rb[j];
                  if (cc + 1 < nchunk) tmem_ld32(tcol0 + (cc + 1) * 64, rb);   // first half of the next chunk
                }
                if (COMM != COMM_RS) {   // alpha, bias, GELU on the way out
                  const int colb = n0 + cc * 64 + hf * 32;
#pragma unroll
                  for (int j = 0; j < 32; ++j) {
                    float v = __uint_as_float(ra[j]) * p.alpha;
                    if ((fl & ELFA_EPI_BIAS) && colb + j < p.N) v += __bfloat162float(p.bias[colb + j]);
                    if (fl & ELFA_EPI_GELU) v = gelu_tanh(v);
                    ra[j] = __float_as_uint(v);
                  }
                }
#pragma unroll
                for (int gq = 0; gq < 4; ++gq) {
                  const int idx = hf * 4 + gq;
                  const uint32_t addr = srow + ((idx ^ (rloc & 7)) << 4);
                  const uint32_t w0 = pack_bf16(__uint_as_float(ra[gq * 8 + 0]), __uint_as_float(ra[gq * 8 + 1]));
                  const uint32_t w1 = pack_bf16(__uint_as_float(ra[gq * 8 + 2]), __uint_as_float(ra[gq * 8 + 3]));
                  const uint32_t w2 = pack_bf16(__uint_as_float(ra[gq * 8 + 4]), __uint_as_float(ra[gq * 8 + 5]));
                  const uint32_t w3 = pack_bf16(__uint_as_float(ra[gq * 8 + 6]), __uint_as_float(ra[gq * 8 + 7]));
                  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
                }
              }
              if (cc + 1 < nchunk) {
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) ra[j] = rb[j];
              }
            }
            if (cc == nchunk - 1) {   // accumulator fully read: hand the buffer back to the MMA warp
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if (TWO) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0)); else mbar_arrive(tempty_bar(buf));
              }
            }
          }
          fence_proxy_async();
          asm volatile("bar.arrive %0, %1;" ::"r"(2 + (int)(g & 1)), "r"(160) : "memory");
        }
        continue;
      }
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      if (!(fl & ~(ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT)) && COMM != COMM_AG && COMM != COMM_GB) {
        // plain bf16 output (narrow-K products are bound by this loop): 64 accumulator columns at a time go through the warp's
        // private 4 KB of the staging area and leave as whole 128-byte lines; the next 64 columns are requested from tensor
        // memory before the lines are written. (The all-gather variant's push warps own the staging area: it keeps the
        // register path below.)
        const uint32_t tcol0 = tmem_base + ((uint32_t)(q * 32) << 16) + buf * ACC_STRIDE;
        const uint32_t stage = smem_u32(smem + L::OUT_OFF) + q * 4096;
        const int row0 = m0 + q * 32;
        __nv_bfloat16* cbase = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row0 * p.ldc + n0;
        const int rows_valid = p.M - row0;
        uint32_t ra[32], rb[32];
        tmem_ld32(tcol0, ra);
        tmem_ld32(tcol0 + 32, rb);
#pragma unroll
        for (int c = 0; c < BN / 32; c += 2) {
          tmem_ld_wait();
          if (fl & ELFA_EPI_STORE_PREACT) {      // the value before the activation goes out first, through the same staging
            warp_stage_64cols(stage, ra, rb, p.alpha, lane);
            __syncwarp();
            warp_flush_64cols(stage, p.preact + (long long)row0 * p.ldpre + n0 + c * 32, p.ldpre, rows_valid, p.N - n0 - c * 32, lane);
            __syncwarp();
          }
          if (fl & ELFA_EPI_GELU) warp_stage_64cols<true>(stage, ra, rb, p.alpha, lane);
          else warp_stage_64cols(stage, ra, rb, p.alpha, lane);
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
      tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * ACC_STRIDE, rnext);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = rnext[j];
        if (c + 1 < BN / 32) tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * ACC_STRIDE + (c + 1) * 32, rnext);   // next chunk in flight
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) continue;  // uniform across the warp
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
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
              uint4 o = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
              *reinterpret_cast<uint4*>(p.preact + (long long)row * p.ldpre + col) = o;
            }
            if (fl & ELFA_EPI_GELU) {
#pragma unroll
              for (int j = 0; j < 8; ++j) w[j] = gelu_tanh(w[j]);
            }
            if (fl & (ELFA_EPI_DGELU_AUX | ELFA_EPI_ADD_AUX)) {
              const uint4 a = *reinterpret_cast<const uint4*>(p.aux + (long long)row * p.ldaux + col);
              const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float lo = bf16_lo(aw[j]), hi = bf16_hi(aw[j]);
                if (fl & ELFA_EPI_DGELU_AUX) {
                  w[2 * j] *= dgelu_tanh(lo);
                  w[2 * j + 1] *= dgelu_tanh(hi);
                } else {
                  w[2 * j] += lo;
                  w[2 * j + 1] += hi;
                }
              }
            }
            if (fl & ELFA_EPI_OUT_F32) {
              float* cp = reinterpret_cast<float*>(p.C) + (long long)row * p.ldc + col;
              float4 o0 = make_float4(w[0], w[1], w[2], w[3]), o1 = make_float4(w[4], w[5], w[6], w[7]);
              if (splits > 1) {     // partial sums of one tile come from several CTAs
                atomicAdd(reinterpret_cast<float4*>(cp), o0);
                atomicAdd(reinterpret_cast<float4*>(cp + 4), o1);
                continue;
              }
              if (fl & ELFA_EPI_ACCUM) {
                const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
                o0.x += c0.x; o0.y += c0.y; o0.z += c0.z; o0.w += c0.w;
                o1.x += c1.x; o1.y += c1.y; o1.z += c1.z; o1.w += c1.w;
              }
              *reinterpret_cast<float4*>(cp) = o0;
              *reinterpret_cast<float4*>(cp + 4) = o1;
            } else {
              __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col;
              if (fl & ELFA_EPI_ACCUM) {
                const uint4 c = *reinterpret_cast<const uint4*>(cp);
                const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  w[2 * j] += bf16_lo(cw[j]);
                  w[2 * j + 1] += bf16_hi(cw[j]);
                }
              }
              uint4 o = make_uint4(pack_bf16(w[0], w[1]), pack_bf16(w[2], w[3]), pack_bf16(w[4], w[5]), pack_bf16(w[6], w[7]));
              *reinterpret_cast<uint4*>(cp) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
                if (TWO) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0)); else mbar_arrive(tempty_bar(buf));
              }
    }
  } else if (staged && warp == 6) {
    // ------------------------------------------------------------------ store warp
    // Sends every staged chunk to its owner, frees staging buffers as soon as the TMA engine has read
    // them, and bumps the owner's arrival counter once a tile's stores have completed - two tiles
    // late, so that the NVLink round trip of the newest tiles is never waited for.
    const bool f32 = p.staged == 2;
    const int CPT = f32 ? BN / 32 : BN / 64;             // chunks per tile
    const int ccols = f32 ? 32 : 64;                     // output columns per chunk
    int my_tiles = 0;
    for (int unit = wid; unit < num_units; unit += wstride) ++my_tiles;
    const uint32_t total_chunks = (uint32_t)my_tiles * CPT;
    const uint32_t out0 = smem_u32(smem + L::OUT_OFF);
    const bool reduce_add = f32 && (p.flags & ELFA_EPI_ACCUM);
    int pend[2] = {-1, -1};                              // owners of the two most recent tiles
    uint32_t g = 0;
    for (int unit = wid; unit < num_units; unit += wstride) {
      const int tile = unit / splits;
      int mb, nb, shard;
      tile_coords_comm<COMM>(p, cm, tile, mb, nb, shard, TILE_M);
      const int m0 = mb * TILE_M + (int)cta_rank * BM, n0 = nb * BN;
      const int dst_row = COMM == COMM_RS ? cm.rank * cm.rows_per_rank + (m0 - shard * cm.rows_per_rank) : m0;
      const int dst_map = COMM == COMM_RS ? shard : 0;
      for (int cc = 0; cc < CPT; ++cc, ++g) {
        named_bar_sync(2 + (g & 1), 160);               // chunk g is staged
        if (lane == 0) {
          const uint32_t src = out0 + (g & 1) * (BM * 128);
          if (n0 + cc * ccols < p.N && !*abort_flag) {
            if (COMM == COMM_RS && cm.chunk_major) {
              const long long chunk = ((long long)((m0 - shard * cm.rows_per_rank) / BM) * p.tiles_n + nb) * CPT + cc;
              char* dst = reinterpret_cast<char*>(cm.peer_recv[shard]) + ((long long)cm.rank * cm.slot_chunks + chunk) * (BM * 128);
              if (bounds_ok(chunk, cm.slot_chunks, p.status))      // checked build: the chunk lies inside this rank's slot
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(BM * 128) : "memory");
            } else if (reduce_add) {
              tma_reduce_add_2d(&om.m[dst_map], src, n0 + cc * ccols, dst_row);
            } else {
              tma_store_2d(&om.m[dst_map], src, n0 + cc * ccols, dst_row);
            }
          }
          tma_store_commit();
          tma_store_wait_read<0>();                     // chunk g has left shared memory
        }
        __syncwarp();
        // release the buffer right away (it is waited for by chunk g + 2, if there is one)
        if (g + 2 < total_chunks) asm volatile("bar.arrive %0, %1;" ::"r"(4 + (int)(g & 1)), "r"(160) : "memory");
      }
      if (lane == 0 && COMM == COMM_RS) {
        if (pend[1] >= 0) {
          if (CPT == 4) tma_store_wait<8>(); else if (CPT == 3) tma_store_wait<6>(); else if (CPT == 2) tma_store_wait<4>(); else tma_store_wait<2>();   // all but the last two tiles' groups
          __threadfence_system();
          unsigned int* cnt = reinterpret_cast<unsigned int*>(cm.peer_flags[pend[1]]) + cm.rank;
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
        }
        pend[1] = pend[0];
        pend[0] = shard;
      }
    }
    if (lane == 0) {
      tma_store_wait<0>();
      __threadfence_system();
      for (int i = 1; i >= 0; --i) {
        if (COMM == COMM_RS && pend[i] >= 0) {
          unsigned int* cnt = reinterpret_cast<unsigned int*>(cm.peer_flags[pend[i]]) + cm.rank;
          asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
        }
      }
    }
  } else if (COMM == COMM_AG && warp >= 7) {
    // ------------------------------------------------------------------ push warps (7, 8)
    // This rank's shard goes to peer rank+1 first, then rank+2, ...; the own copy (needed later by
    // the weight-gradient GEMM) is written last. One lane per warp drives a two-buffer pipeline of
    // bulk copies: local global memory -> shared memory -> the peer's gathered buffer. The loads are
    // local, the stores cross NVLink as large transactions; nothing here is a multicast.
    const int w = warp - 7;
    const uint32_t buf0 = smem_u32(smem + L::OUT_OFF) + w * 16384;
    auto pbar = [&](int b) { return bar0 + 8u * (2 * STAGES + 4 + w * 2 + b); };
    const long long nchunks = (long long)cm.rows_per_rank * cm.pieces_per_row;
    const long long c_first = (long long)blockIdx.x * 2 + w, c_step = (long long)gridDim.x * 2;
    const uint32_t pb = (uint32_t)cm.piece_bytes;
    const char* src0 = reinterpret_cast<const char*>(cm.x_local);
    uint32_t n_issued = 0, n_done = 0;   // loads issued / consumed: buffer = index & 1, phase = (index >> 1) & 1
    bool okp = true;
    auto src_of = [&](long long c) {
      const long long r = c / cm.pieces_per_row, pc = c - r * cm.pieces_per_row;
      return src0 + r * cm.ldx * 2 + pc * pb;
    };
    auto dst_off = [&](long long c) {
      const long long r = c / cm.pieces_per_row, pc = c - r * cm.pieces_per_row;
      return ((long long)cm.rank * cm.rows_per_rank + r) * p.K * 2 + pc * pb;
    };
    auto issue_load = [&](long long c) {
      const int b = n_issued & 1;
      tma_store_wait_read<0>();                       // the store that last used this buffer has read it
      mbar_expect_tx(pbar(b), pb);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(buf0 + b * 8192), "l"(src_of(c)), "r"(pb), "r"(pbar(b)) : "memory");
      ++n_issued;
    };
    // Peers are served one after the other without draining the pipeline in between: a peer's counter is raised once the
    // NEXT peer's stores have been issued and this peer's (older) bulk groups are known to be complete.
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
    auto signal = [&](int peer) {              // both push warps have finished `peer`: one counter increment per CTA
      named_bar_sync(1, 64);
      if (w == 0 && lane == 0 && peer != cm.rank) {
        unsigned int* cnt = reinterpret_cast<unsigned int*>(cm.peer_flags[peer]) + cm.rank;
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
      }
    };
    int prev_peer = -1;
    for (int i = 1; i <= cm.world; ++i) {
      const int peer = (cm.rank + i) % cm.world;
      if (lane == 0) {
        char* dst = reinterpret_cast<char*>(cm.peer_xfull[peer]);
        uint32_t stores = 0;
        if (okp && c_first < nchunks) issue_load(c_first);
        for (long long c = c_first; c < nchunks && okp; c += c_step) {
          if (c + c_step < nchunks) issue_load(c + c_step);
          const int b = n_done & 1;
          if (!mbar_wait(pbar(b), (n_done >> 1) & 1, abort_flag, p.status)) { okp = false; break; }
          if (bounds_ok(dst_off(c) + pb - 1, (long long)cm.world * cm.rows_per_rank * p.K * 2, p.status))
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(dst + dst_off(c)), "r"(buf0 + b * 8192), "r"(pb) : "memory");
          tma_store_commit();
          ++n_done;
          ++stores;
        }
        if (prev_peer >= 0) {
          wait_all_but(okp ? stores : 0u);              // every store to the previous peer has completed
          __threadfence_system();
        }
      }
      __syncwarp();
      if (prev_peer >= 0) signal(prev_peer);
      prev_peer = peer;
    }
    if (lane == 0) {
      tma_store_wait<0>();
      __threadfence_system();
    }
    __syncwarp();
    signal(prev_peer);
    if (lane == 0 && !okp) {   // give a load that is still in flight a bounded chance to land before the CTA exits
      for (uint32_t j = n_done; j < n_issued; ++j) {
        const long long t0 = clock64();
        while (!mbar_try(pbar(j & 1), (j >> 1) & 1) && clock64() - t0 < 4000000) {}
      }
    }
  }

  if (COMM == COMM_GB && warp >= 7) {
    // ------------------------------------------------------------------ gather warps (7, 8)
    // The parameter's bytes are fetched owner by owner, this rank's own part first (a local copy), then rank + 1, ...:
    // bulk load from the owner's shard (peer memory, no multicast) into shared memory, bulk store into the local bucket.
    // After an owner's pieces of this CTA have landed, warp 7 raises the local counter of that owner once.
    const int w = warp - 7;
    const uint32_t buf0 = smem_u32(smem + L::OUT_OFF) + w * 16384;
    auto pbar = [&](int b) { return bar0 + 8u * (2 * STAGES + 4 + w * 2 + b); };
    uint32_t n_issued = 0, n_done = 0;
    bool okp = true;
    const long long w_end = cm.gb_w_off + cm.gb_w_bytes;
    for (int i = 0; i < cm.world; ++i) {
      const int r = (cm.rank + i) % cm.world;
      long long lo = (long long)r * cm.gb_shard_bytes, hi = lo + cm.gb_shard_bytes;
      if (lo < cm.gb_w_off) lo = cm.gb_w_off;
      if (hi > w_end) hi = w_end;
      const long long npieces = hi > lo ? (hi - lo + 8191) / 8192 : 0;
      const long long c_first = (long long)blockIdx.x * 2 + w, c_step = (long long)gridDim.x * 2;
      if (lane == 0) {
        const char* src = reinterpret_cast<const char*>(cm.gb_src[r]) + (lo - (long long)r * cm.gb_shard_bytes);
        char* dst = cm.gb_dst + lo;
        auto nbytes_of = [&](long long c) { const long long rem = hi - lo - c * 8192; return (uint32_t)(rem < 8192 ? rem : 8192); };
        auto issue_load = [&](long long c) {
          const int b = n_issued & 1;
          tma_store_wait_read<0>();                       // the store that last used this buffer has read it
          mbar_expect_tx(pbar(b), nbytes_of(c));
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(buf0 + b * 8192), "l"(src + c * 8192), "r"(nbytes_of(c)), "r"(pbar(b)) : "memory");
          ++n_issued;
        };
        if (okp && c_first < npieces) issue_load(c_first);
        for (long long c = c_first; c < npieces && okp; c += c_step) {
          if (c + c_step < npieces) issue_load(c + c_step);
          const int b = n_done & 1;
          if (!mbar_wait(pbar(b), (n_done >> 1) & 1, abort_flag, p.status)) { okp = false; break; }
          if (bounds_ok(lo + c * 8192 + nbytes_of(c) - 1, w_end, p.status))
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                         ::"l"(dst + c * 8192), "r"(buf0 + b * 8192), "r"(nbytes_of(c)) : "memory");
          tma_store_commit();
          ++n_done;
        }
        tma_store_wait<0>();                              // this owner's pieces are in local memory
        __threadfence();
      }
      __syncwarp();
      named_bar_sync(1, 64);                              // both gather warps are done with this owner
      if (w == 0 && lane == 0 && okp) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(cm.gb_flags + r) : "memory");
    }
    if (lane == 0 && !okp) {   // give a load that is still in flight a bounded chance to land before the CTA exits
      for (uint32_t j = n_done; j < n_issued; ++j) {
        const long long t0 = clock64();
        while (!mbar_try(pbar(j & 1), (j >> 1) & 1) && clock64() - t0 < 4000000) {}
      }
    }
  }

  if (COMM == COMM_RS) {
    // ------------------------------------------------------------------ reduce the owned rows
    // Threads without a role park at this barrier (no spinning next to the producer / MMA lanes);
    // one thread then polls the arrival counters for the whole CTA.
    __syncthreads();
    __shared__ int rs_ok;
    if (threadIdx.x == 0) {
      bool ok0 = true;
      for (int src = 0; src < cm.world && ok0; ++src)
        ok0 = flag_wait(cm.my_flags + src, cm.flag_target, cm.wait_cycles, abort_flag, p.status);
      rs_ok = ok0 ? 1 : 0;
    }
    __syncthreads();
    const bool ok = rs_ok != 0;
    if (ok && cm.chunk_major) {
      // slots hold 16 KB chunks in shared-memory order: vector v of a slot = chunk v / 1024, row (v % 1024) / 8 of the
      // chunk, 16-byte unit (v % 8) ^ (row % 8) of that row's 128 bytes
      constexpr int CPT = BN / 64;
      const long long nvec = cm.slot_chunks * 1024;
      const long long slot = cm.slot_chunks * (BM * 64);
      for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
        const long long chunk = v >> 10;
        const int within = (int)(v & 1023), rr = within >> 3, unit = (within & 7) ^ (rr & 7);
        const int cc = (int)(chunk % CPT);
        const long long t = chunk / CPT;
        const int nb = (int)(t % p.tiles_n);
        const long long row = (t / p.tiles_n) * BM + rr;
        const int col = nb * BN + cc * 64 + unit * 8;
        if (col >= p.N) continue;
        if (!bounds_ok(row, cm.rows_per_rank, p.status)) continue;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 q[MAX_RANKS];
#pragma unroll
        for (int src = 0; src < MAX_RANKS; ++src)      // every slot's load in flight before the first add
          if (src < cm.world) q[src] = *reinterpret_cast<const uint4*>(cm.my_recv + src * slot + v * 8);
#pragma unroll
        for (int src = 0; src < MAX_RANKS; ++src) {    // fixed order
          if (src < cm.world) {
            const uint32_t qw[4] = {q[src].x, q[src].y, q[src].z, q[src].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              acc[2 * j] += bf16_lo(qw[j]);
              acc[2 * j + 1] += bf16_hi(qw[j]);
            }
          }
        }
        uint4 o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
        *reinterpret_cast<uint4*>(cm.rs_out + row * cm.ld_out + col) = o;
      }
    } else if (ok) {
      const long long vec_per_row = p.N / 8;
      const long long nvec = (long long)cm.rows_per_rank * vec_per_row;
      const long long slot = (long long)cm.rows_per_rank * p.N;
      for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
        const long long r = v / vec_per_row, cv = v - r * vec_per_row;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 q[MAX_RANKS];
#pragma unroll
        for (int src = 0; src < MAX_RANKS; ++src)      // every slot's load in flight before the first add
          if (src < cm.world) q[src] = *reinterpret_cast<const uint4*>(cm.my_recv + src * slot + r * p.N + cv * 8);
#pragma unroll
        for (int src = 0; src < MAX_RANKS; ++src) {    // fixed order
          if (src < cm.world) {
            const uint32_t qw[4] = {q[src].x, q[src].y, q[src].z, q[src].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              acc[2 * j] += bf16_lo(qw[j]);
              acc[2 * j + 1] += bf16_hi(qw[j]);
            }
          }
        }
        uint4 o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
        *reinterpret_cast<uint4*>(cm.rs_out + r * cm.ld_out + cv * 8) = o;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (TWO) cluster_sync_all();   // the peer no longer reads this CTA's shared memory or signals its barriers
  if (warp == 1) {
    tc_fence_after();
    if (TWO) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
struct TmapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t br, bc;
  bool operator==(const TmapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && br == o.br && bc == o.bc;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ (((uint64_t)k.br << 32) | k.bc);
    return h;
  }
};
static std::mutex g_tm_mu;
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tm_cache;

int cached_tmap(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                uint32_t box_rows, uint32_t box_cols) {
  TmapKey key{base, rows, cols, ld_elems * 8 + (uint64_t)elem_bytes, box_rows, box_cols};
  {
    std::lock_guard<std::mutex> lk(g_tm_mu);
    auto it = g_tm_cache.find(key);
    if (it != g_tm_cache.end()) {
      *out = it->second;
      return ELFA_OK;
    }
  }
  int rc = make_tmap_2d(out, base, elem_bytes, rows, cols, ld_elems * elem_bytes, box_rows, box_cols, true);
  if (rc != ELFA_OK) return rc;
  std::lock_guard<std::mutex> lk(g_tm_mu);
  if (g_tm_cache.size() > 8192) g_tm_cache.clear();
  g_tm_cache.emplace(key, *out);
  return ELFA_OK;
}

int cached_tmap_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows,
                     uint32_t box_cols) {
  return cached_tmap(out, base, 2, rows, cols, ld_elems, box_rows, box_cols);
}

static int g_sm_count = 0;
int sm_count() {
  if (!g_sm_count) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (g_sm_count <= 0) g_sm_count = 148;
  }
  return g_sm_count;
}

template <int BN, bool A_MN, bool B_MN, int COMM = COMM_NONE, bool TWO = false, bool MX = false>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams p, int max_ctas, cudaStream_t stream,
                const CUtensorMap* tmA2 = nullptr, const CommParams* comm = nullptr, const OutMaps* om = nullptr) {
  constexpr int STAGES = MX ? (TWO ? 6 : (BN == 192 ? 4 : 5)) : (TWO ? 6 : (BN == 256 ? 4 : (BN == 128 ? 6 : 8)));
  constexpr int TILE_M = TWO ? 2 * BM : BM;
  using L = SmemLayout<TWO ? BN / 2 : BN, STAGES, MX ? (1 + (BN <= 128 ? 1 : 2)) * 512 : 0>;
  static_assert(L::DYN_RS <= 227 * 1024, "shared-memory plan exceeds the per-CTA limit");
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, STAGES, COMM, TWO, MX>;
  constexpr int DYN = L::DYN_RS;   // every variant carries the two staging tiles of the TMA-store epilogue
  static bool configured = false;
  if (!configured) {
    ELFA_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN));
    configured = true;
  }
  p.tiles_m = (p.M + TILE_M - 1) / TILE_M;
  p.tiles_n = (p.N + BN - 1) / BN;
  {
    // tile order: sweep over N inside groups of M tiles whose rows of A (about 32 MB) stay in L2
    const long long rows = std::max(512LL, std::min(4096LL, (32LL << 20) / ((long long)p.K * 2)));
    p.group_m = (int)std::max(1LL, rows / TILE_M);
  }
  if (TWO) max_ctas /= 2;    // work slots are CTA pairs
  const int num_kb_host = MX ? (p.K + 127) / 128 : (p.K + BK - 1) / BK;
  p.splits = 1;
  if (COMM == COMM_NONE && !deterministic_mode() && (p.flags & (ELFA_EPI_ACCUM | ELFA_EPI_OUT_F32)) == (ELFA_EPI_ACCUM | ELFA_EPI_OUT_F32)) {
    // fp32 accumulate outputs (weight gradients): split K when the tile count fills the SMs badly
    const int t = p.tiles_m * p.tiles_n;
    auto eff = [&](int sp) { const int u = t * sp; return (double)u / (double)(((u + max_ctas - 1) / max_ctas) * max_ctas); };
    double best = eff(1);
    const int cand[5] = {2, 3, 4, 6, 8};
    for (int i = 0; i < 5; ++i) {
      if (num_kb_host / cand[i] < 8) break;
      const double e = eff(cand[i]);
      if (e > best + 0.04) { best = e; p.splits = cand[i]; }
    }
  }
  p.kb_per_split = (num_kb_host + p.splits - 1) / p.splits;
  int tiles = p.tiles_m * p.tiles_n * p.splits;
  int grid = tiles < max_ctas ? tiles : max_ctas;
  CommParams c{};
  if (comm) c = *comm;
  static const OutMaps no_maps{};
  if (TWO) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2 * grid, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = DYN;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ELFA_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmA2 ? *tmA2 : tmA, p, c, om ? *om : no_maps));
  } else {
    kern<<<grid, GEMM_THREADS, DYN, stream>>>(tmA, tmB, tmA2 ? *tmA2 : tmA, p, c, om ? *om : no_maps);
  }
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

int dispatch_pair(int a_mn, int b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int max_ctas,
                  cudaStream_t stream, const OutMaps* om) {
  if (!a_mn && !b_mn) return launch_gemm<256, false, false, COMM_NONE, true>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
  if (!a_mn && b_mn) return launch_gemm<256, false, true, COMM_NONE, true>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
  if (a_mn && !b_mn) return launch_gemm<256, true, false, COMM_NONE, true>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
  return launch_gemm<256, true, true, COMM_NONE, true>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
}

template <int BN>
int dispatch_layout(int a_mn, int b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int max_ctas,
                    cudaStream_t stream, const OutMaps* om) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
  if (!a_mn && b_mn) return launch_gemm<BN, false, true>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
  if (a_mn && !b_mn) return launch_gemm<BN, true, false>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
  return launch_gemm<BN, true, true>(tmA, tmB, p, max_ctas, stream, nullptr, nullptr, om);
}

}  // namespace

// entry points for the other GEMM translation units (tensor-map cache, SM count)
int shared_tmap(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                uint32_t box_rows, uint32_t box_cols) {
  return cached_tmap(out, base, elem_bytes, rows, cols, ld_elems, box_rows, box_cols);
}
int device_sm_count() { return sm_count(); }

int pick_bn(int M, int N, int forced) {
  if (forced == 64 || forced == 128 || forced == 256) return forced;
  const int sms = sm_count();
  const long long tm = (M + BM - 1) / BM;
  if (N >= 256 && tm * ((N + 255) / 256) >= sms) return 256;
  if (N >= 128 && tm * ((N + 127) / 128) >= sms / 2) return 128;
  if (N > 64 && tm * ((N + 127) / 128) >= sms / 4) return 128;
  return N > 128 ? 128 : 64;
}

}  // namespace elfa

using namespace elfa;

ELFA_API int elfa_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int a_mn_major, int b_mn_major, const void* bias, const void* aux,
                            long long ldaux, void* preact, long long ldpre, float alpha, unsigned flags, int force_bn,
                            int max_ctas, void* stream) {
  ELFA_REQUIRE(A && B && C, "gemm: null operand");
  ELFA_REQUIRE(M > 0 && N > 0 && K > 0, "gemm: empty problem");
  ELFA_REQUIRE(N % 8 == 0, "gemm: N must be a multiple of 8");
  ELFA_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "gemm: operand row pitch must be a multiple of 8 elements");
  ELFA_REQUIRE(ldc % ((flags & ELFA_EPI_OUT_F32) ? 4 : 8) == 0, "gemm: ldc alignment");
  ELFA_REQUIRE(!(flags & ELFA_EPI_BIAS) || bias, "gemm: bias flag without pointer");
  ELFA_REQUIRE(!(flags & (ELFA_EPI_DGELU_AUX | ELFA_EPI_ADD_AUX)) || (aux && ldaux % 8 == 0), "gemm: aux flag without pointer");
  ELFA_REQUIRE(!(flags & ELFA_EPI_STORE_PREACT) || (preact && ldpre % 8 == 0), "gemm: preact flag without pointer");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm: no status word");

  // force_bn 512 selects the CTA-pair kernel (256 x 256 tiles per pair); by default it is used when the
  // problem fills at least one wave of pairs with such tiles
  const int pairs = sm_count() / 2;
  const bool pair = force_bn == 512 ||
                    (force_bn == 0 && N >= 256 && (long long)((M + 255) / 256) * ((N + 255) / 256) >= pairs && (max_ctas <= 0 || max_ctas >= sm_count()));
  const int BN = pair ? 256 : pick_bn(M, N, force_bn);
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn_major) rc = cached_tmap_bf16(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
  else rc = cached_tmap_bf16(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK, 64);
  if (rc != ELFA_OK) return rc;
  if (!b_mn_major) rc = cached_tmap_bf16(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, pair ? BN / 2 : BN, BK);
  else rc = cached_tmap_bf16(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, 64);
  if (rc != ELFA_OK) return rc;

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.aux = static_cast<const __nv_bfloat16*>(aux);
  p.ldaux = ldaux;
  p.preact = static_cast<__nv_bfloat16*>(preact);
  p.ldpre = ldpre;
  p.alpha = alpha;
  p.flags = flags;
  p.status = st;
  const int ctas = (max_ctas > 0 && max_ctas < sm_count()) ? max_ctas : sm_count();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  OutMaps om{};
  // bf16 outputs keep the direct register -> global epilogue: measured faster than staging for them
  // (16384x4096x512: 0.095 ms direct vs 0.27 ms staged); fp32 outputs gain 2x from staging + reduce-add.
  if ((flags & ELFA_EPI_OUT_F32) && !(flags & ~(ELFA_EPI_OUT_F32 | ELFA_EPI_ACCUM)) && N % 4 == 0) {
    // fp32 output (weight gradients): staged 32-column chunks, TMA store or TMA reduce-add (+=)
    rc = cached_tmap(&om.m[0], C, 4, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, BM, 32);
    if (rc != ELFA_OK) return rc;
    p.staged = 2;
  } else if ((flags & ELFA_EPI_STAGED) && !(flags & ~(ELFA_EPI_STAGED | ELFA_EPI_BIAS | ELFA_EPI_GELU)) && N % 64 == 0) {
    rc = cached_tmap(&om.m[0], C, 2, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, BM, 64);
    if (rc != ELFA_OK) return rc;
    p.staged = 1;
  }
  if (pair) return dispatch_pair(a_mn_major, b_mn_major, tmA, tmB, p, ctas, s, &om);
  switch (BN) {
    case 256: return dispatch_layout<256>(a_mn_major, b_mn_major, tmA, tmB, p, ctas, s, &om);
    case 128: return dispatch_layout<128>(a_mn_major, b_mn_major, tmA, tmB, p, ctas, s, &om);
    default: return dispatch_layout<64>(a_mn_major, b_mn_major, tmA, tmB, p, ctas, s, &om);
  }
}


namespace elfa {
namespace {

template <int COMM>
int dispatch_comm(int BN, int b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmA2, const GemmParams& p,
                  const CommParams& c, cudaStream_t s, const OutMaps* om = nullptr, int max_ctas = 0, bool pair = false) {
  const int ctas = (max_ctas > 0 && max_ctas < sm_count()) ? max_ctas : sm_count();
  if (pair) {
    return b_mn ? launch_gemm<256, false, true, COMM, true>(tmA, tmB, p, ctas, s, &tmA2, &c, om)
                : launch_gemm<256, false, false, COMM, true>(tmA, tmB, p, ctas, s, &tmA2, &c, om);
  }
  if (BN == 256) {
    return b_mn ? launch_gemm<256, false, true, COMM>(tmA, tmB, p, ctas, s, &tmA2, &c, om)
                : launch_gemm<256, false, false, COMM>(tmA, tmB, p, ctas, s, &tmA2, &c, om);
  }
  return b_mn ? launch_gemm<128, false, true, COMM>(tmA, tmB, p, ctas, s, &tmA2, &c, om)
              : launch_gemm<128, false, false, COMM>(tmA, tmB, p, ctas, s, &tmA2, &c, om);
}

int comm_grid(int M, int N, int BN, bool pair = false) {
  if (pair) {   // CTAs of the pair launch: two per 256 x 256 tile, at most one pair per two SMs
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    const int pairs = sm_count() / 2;
    return 2 * (tiles < pairs ? tiles : pairs);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return tiles < sm_count() ? tiles : sm_count();
}

// CTA pairs for a fused kernel: 256-wide tiles, every pair's 256 rows inside one shard, at least one wave of pairs
bool comm_pair(int M, int N, int rows_per_rank) {
  return N >= 256 && rows_per_rank % (2 * BM) == 0 && (long long)(M / (2 * BM)) * ((N + 255) / 256) >= sm_count() / 2;
}

}  // namespace
}  // namespace elfa

// C[M,N] = epilogue(all_gather_rows(x_local)[M,K] * op(B)), M = world * rows. One kernel: the shard
// is pushed to every peer's `xfull` buffer while the tensor cores start on the local rows.
//   peer_xfull / peer_flags : host arrays of `world` device addresses (entry `rank` = this rank's own)
//   my_flags                : this rank's arrival counters (u32 per source rank), never reset
//   arrivals_io             : host counter of arrivals expected so far on this flag set; updated
// After the call xfull (this rank's entry) holds the gathered A (kept for the weight gradient).
ELFA_API int elfa_gemm_ag(const void* x_local, long long ldx, const unsigned long long* peer_xfull,
                          const unsigned long long* peer_flags, const void* my_flags, unsigned int* arrivals_io, const void* B,
                          void* C, int M, int N, int K, long long ldb, long long ldc, int b_mn_major, void* preact, long long ldpre,
                          unsigned flags, int rank, int world, int wait_ms, void* stream) {
  ELFA_REQUIRE(x_local && peer_xfull && peer_flags && my_flags && arrivals_io && B && C, "gemm_ag: null argument");
  ELFA_REQUIRE(world >= 2 && world <= MAX_RANKS && rank >= 0 && rank < world, "gemm_ag: bad rank/world");
  ELFA_REQUIRE(M % world == 0 && (M / world) % BM == 0, "gemm_ag: rows per rank must be a multiple of 128");
  ELFA_REQUIRE(N % 8 == 0 && K % 8 == 0 && ldx % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0, "gemm_ag: alignment");
  ELFA_REQUIRE(!(flags & ~(ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT)), "gemm_ag: unsupported epilogue flag");
  ELFA_REQUIRE(!(flags & ELFA_EPI_STORE_PREACT) || (preact && ldpre % 8 == 0), "gemm_ag: preact flag without pointer");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm_ag: no status word");
  const int rows = M / world;
  const bool pair = comm_pair(M, N, rows);
  const int BN = (pair || (N >= 256 && (long long)(M / BM) * ((N + 255) / 256) >= sm_count())) ? 256 : 128;
  CUtensorMap tmA, tmA2, tmB;
  int rc = cached_tmap_bf16(&tmA, reinterpret_cast<const void*>(peer_xfull[rank]), (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, BK);
  if (rc != ELFA_OK) return rc;
  rc = cached_tmap_bf16(&tmA2, x_local, (uint64_t)rows, (uint64_t)K, (uint64_t)ldx, BM, BK);
  if (rc != ELFA_OK) return rc;
  if (!b_mn_major) rc = cached_tmap_bf16(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, pair ? BN / 2 : BN, BK);
  else rc = cached_tmap_bf16(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, 64);
  if (rc != ELFA_OK) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.preact = static_cast<__nv_bfloat16*>(preact);
  p.ldpre = ldpre;
  p.alpha = 1.f;
  p.flags = flags;
  p.status = st;
  CommParams c{};
  c.rank = rank; c.world = world; c.rows_per_rank = rows;
  c.wait_cycles = wait_cycles_of(wait_ms);
  c.x_local = static_cast<const __nv_bfloat16*>(x_local);
  c.ldx = ldx;
  {
    // a row travels in equal pieces of at most 8 KB whose size is a multiple of 16 bytes (bulk-copy rule)
    const long long rb = (long long)K * 2;
    int ppr = (int)((rb + 8191) / 8192);
    while (ppr <= 64 && rb % ((long long)ppr * 16) != 0) ++ppr;
    ELFA_REQUIRE(ppr <= 64, "gemm_ag: K * 2 bytes cannot be split into 16-byte aligned pieces of at most 8 KB");
    c.pieces_per_row = ppr;
    c.piece_bytes = (int)(rb / ppr);
  }
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(x_local) & 15) == 0, "gemm_ag: x_local must be 16-byte aligned");
  for (int i = 0; i < world; ++i) {
    ELFA_REQUIRE((peer_xfull[i] & 15) == 0, "gemm_ag: gathered buffers must be 16-byte aligned");
    c.peer_xfull[i] = peer_xfull[i];
    c.peer_flags[i] = peer_flags[i];
  }
  c.my_flags = static_cast<const unsigned int*>(my_flags);
  *arrivals_io += (unsigned)comm_grid(M, N, BN, pair);        // every CTA of a source bumps the counter once
  c.flag_target = *arrivals_io;
  OutMaps om{};
  return dispatch_comm<COMM_AG>(BN, b_mn_major, tmA, tmB, tmA2, p, c, static_cast<cudaStream_t>(stream), &om, 0, pair);
}

// C[M,N] = epilogue(A[M,K] * B[K,N]) where B (row-major, ld = N) is a parameter sharded over `world` ranks: bytes
// [w_off, w_off + K * N * 2) of a bucket whose rank r keeps bytes [r * shard_bytes, (r + 1) * shard_bytes) at shard_src[r]
// (peer addressable, stable during the call). The kernel copies the parameter into the local full-size bucket
// (`bucket_dst`, the bucket's base; B = bucket_dst + w_off) while the tensor cores start on the K blocks that have arrived:
// the parameter all-gather of ZeRO stage 3 inside the consuming GEMM. `flags_dev`: `world` zeroed u32 counters in local
// memory. Nothing is signalled to another GPU; the owners' shards only have to stay unchanged.
ELFA_API int elfa_gemm_gb(const void* A, long long lda, void* C, long long ldc, int M, int N, int K, void* preact, long long ldpre,
                          unsigned flags, const unsigned long long* shard_src, void* bucket_dst, long long w_off, long long shard_bytes,
                          void* flags_dev, int rank, int world, int wait_ms, void* stream) {
  ELFA_REQUIRE(A && C && shard_src && bucket_dst && flags_dev, "gemm_gb: null argument");
  ELFA_REQUIRE(world >= 2 && world <= MAX_RANKS && rank >= 0 && rank < world, "gemm_gb: bad rank/world");
  ELFA_REQUIRE(M > 0 && N % 8 == 0 && K % 8 == 0 && lda % 8 == 0 && ldc % 8 == 0, "gemm_gb: alignment");
  ELFA_REQUIRE(w_off >= 0 && w_off % 16 == 0 && shard_bytes > 0 && shard_bytes % 16 == 0, "gemm_gb: byte ranges must be 16-byte aligned");
  ELFA_REQUIRE(w_off + (long long)K * N * 2 <= shard_bytes * world, "gemm_gb: the parameter must lie inside the bucket");
  ELFA_REQUIRE(!(flags & ~(ELFA_EPI_GELU | ELFA_EPI_STORE_PREACT)), "gemm_gb: unsupported epilogue flag");
  ELFA_REQUIRE(!(flags & ELFA_EPI_STORE_PREACT) || (preact && ldpre % 8 == 0), "gemm_gb: preact flag without pointer");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(bucket_dst) & 15) == 0, "gemm_gb: bucket must be 16-byte aligned");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm_gb: no status word");
  const void* B = static_cast<const char*>(bucket_dst) + w_off;
  const bool pair = N >= 256 && (long long)((M + 255) / 256) * ((N + 255) / 256) >= sm_count() / 2;
  const int BN = (pair || (N >= 256 && (long long)((M + BM - 1) / BM) * ((N + 255) / 256) >= sm_count())) ? 256 : 128;
  CUtensorMap tmA, tmB;
  int rc = cached_tmap_bf16(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
  if (rc != ELFA_OK) return rc;
  rc = cached_tmap_bf16(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)N, BK, 64);
  if (rc != ELFA_OK) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc;
  p.preact = static_cast<__nv_bfloat16*>(preact);
  p.ldpre = ldpre;
  p.alpha = 1.f;
  p.flags = flags;
  p.status = st;
  CommParams c{};
  c.rank = rank; c.world = world;
  c.wait_cycles = wait_cycles_of(wait_ms);
  for (int i = 0; i < world; ++i) {
    ELFA_REQUIRE(shard_src[i] && (shard_src[i] & 15) == 0, "gemm_gb: shard addresses must be 16-byte aligned");
    c.gb_src[i] = shard_src[i];
  }
  c.gb_dst = static_cast<char*>(bucket_dst);
  c.gb_w_off = w_off;
  c.gb_w_bytes = (long long)K * N * 2;
  c.gb_shard_bytes = shard_bytes;
  c.gb_row_bytes = (long long)N * 2;
  c.gb_flags = static_cast<unsigned int*>(flags_dev);
  c.gb_target = (unsigned)comm_grid(M, N, BN, pair);       // every CTA raises every owner's counter once
  {
    const long long own_lo = std::max(w_off, (long long)rank * shard_bytes), blk = (long long)BK * c.gb_row_bytes;
    const int num_kb = (K + BK - 1) / BK;
    const long long rot = own_lo < w_off + c.gb_w_bytes ? (own_lo - w_off + blk - 1) / blk : 0;
    c.gb_kb_rot = rot < num_kb ? (int)rot : 0;
  }
  OutMaps om{};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int ctas = sm_count();
  if (pair) return launch_gemm<256, false, true, COMM_GB, true>(tmA, tmB, p, ctas, s, &tmA, &c, &om);
  if (BN == 256) return launch_gemm<256, false, true, COMM_GB>(tmA, tmB, p, ctas, s, &tmA, &c, &om);
  return launch_gemm<128, false, true, COMM_GB>(tmA, tmB, p, ctas, s, &tmA, &c, &om);
}

// out[M/world, N] = reduce_scatter_rows(A[M,K] * op(B)): partial tiles travel to the owner's receive
// buffer ([world][M/world][N] bf16, symmetric) and are summed there in rank order.
ELFA_API int elfa_gemm_rs(const void* A, long long lda, const void* B, long long ldb, int b_mn_major, int M, int N, int K,
                          const unsigned long long* peer_recv, const unsigned long long* peer_flags, const void* my_flags,
                          unsigned int* arrivals_io, void* out, long long ld_out, int rank, int world, int wait_ms, int max_ctas,
                          void* stream) {
  ELFA_REQUIRE(A && B && peer_recv && peer_flags && my_flags && arrivals_io && out, "gemm_rs: null argument");
  ELFA_REQUIRE(world >= 2 && world <= MAX_RANKS && rank >= 0 && rank < world, "gemm_rs: bad rank/world");
  ELFA_REQUIRE(M % world == 0 && (M / world) % BM == 0, "gemm_rs: rows per rank must be a multiple of 128");
  ELFA_REQUIRE(N % 64 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ld_out % 8 == 0, "gemm_rs: alignment (N must be a multiple of 64)");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm_rs: no status word");
  const int rows = M / world;
  const bool pair = comm_pair(M, N, rows) && (max_ctas <= 0 || max_ctas >= sm_count());
  const int BN = (pair || (N >= 256 && (long long)(M / BM) * ((N + 255) / 256) >= sm_count())) ? 256 : 128;
  CUtensorMap tmA, tmB;
  int rc = cached_tmap_bf16(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
  if (rc != ELFA_OK) return rc;
  if (!b_mn_major) rc = cached_tmap_bf16(&tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, pair ? BN / 2 : BN, BK);
  else rc = cached_tmap_bf16(&tmB, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, BK, 64);
  if (rc != ELFA_OK) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = out; p.ldc = ld_out;
  p.alpha = 1.f;
  p.status = st;
  CommParams c{};
  c.rank = rank; c.world = world; c.rows_per_rank = rows;
  c.wait_cycles = wait_cycles_of(wait_ms);
  for (int i = 0; i < world; ++i) { c.peer_recv[i] = peer_recv[i]; c.peer_flags[i] = peer_flags[i]; }
  c.my_flags = static_cast<const unsigned int*>(my_flags);
  c.my_recv = reinterpret_cast<const __nv_bfloat16*>(peer_recv[rank]);
  c.rs_out = static_cast<__nv_bfloat16*>(out);
  c.ld_out = ld_out;
  {
    // chunk-major slots need whole tiles along N (the slot is then exactly rows x N); ELFA_RS_CHUNK_MAJOR=0 keeps row-major slots
    const char* e = getenv("ELFA_RS_CHUNK_MAJOR");
    const bool want = !(e && e[0] == '0');
    c.chunk_major = (want && N % BN == 0) ? 1 : 0;
    c.slot_chunks = (long long)(rows / BM) * ((N + BN - 1) / BN) * (BN / 64);
  }
  // per source rank: one bump per tile of the shard
  *arrivals_io += (unsigned)((rows / BM) * ((N + BN - 1) / BN));
  c.flag_target = *arrivals_io;
  OutMaps om{};
  for (int i = 0; i < world; ++i) {
    rc = cached_tmap_bf16(&om.m[i], reinterpret_cast<const void*>(peer_recv[i]), (uint64_t)M, (uint64_t)N, (uint64_t)N, BM, 64);
    if (rc != ELFA_OK) return rc;
  }
  // max_ctas < SM count leaves SMs to a kernel on another stream (a weight-gradient GEMM next to this comm-bound kernel)
  return dispatch_comm<COMM_RS>(BN, b_mn_major, tmA, tmB, tmA, p, c, static_cast<cudaStream_t>(stream), &om, max_ctas, pair);
}

// out[M/world, N] = reduce_scatter_rows(A[M,K] * B[N,K]^T) with MXFP8 operands (e4m3 payloads, scale atoms as produced by
// elfa_mxfp8_quantize_gemm: A a left operand, B a right operand): the block-scaled product of the row-parallel MXFP8 layers
// inside the fused GEMM -> reduce-scatter kernel. Receive slots are chunk-major and hold N rounded up to whole 192- (or
// 128-) wide tiles: `peer_recv` buffers need world * (M / world) * elfa_gemm_rs_slot_cols(N) * 2 bytes.
ELFA_API int elfa_gemm_rs_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, int M, int N, int K,
                                const unsigned long long* peer_recv, const unsigned long long* peer_flags, const void* my_flags,
                                unsigned int* arrivals_io, void* out, long long ld_out, int rank, int world, int wait_ms, int max_ctas,
                                void* stream) {
  ELFA_REQUIRE(A && sfa && B && sfb && peer_recv && peer_flags && my_flags && arrivals_io && out, "gemm_rs_mxfp8: null argument");
  ELFA_REQUIRE(world >= 2 && world <= MAX_RANKS && rank >= 0 && rank < world, "gemm_rs_mxfp8: bad rank/world");
  ELFA_REQUIRE(M % world == 0 && (M / world) % BM == 0, "gemm_rs_mxfp8: rows per rank must be a multiple of 128");
  ELFA_REQUIRE(N % 64 == 0 && K % 32 == 0 && ld_out % 8 == 0, "gemm_rs_mxfp8: N must be a multiple of 64, K of 32");
  ELFA_REQUIRE((reinterpret_cast<uintptr_t>(sfa) & 15) == 0 && (reinterpret_cast<uintptr_t>(sfb) & 15) == 0,
               "gemm_rs_mxfp8: scale tensors must be 16-byte aligned");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "gemm_rs_mxfp8: no status word");
  const int rows = M / world;
  const bool wide = N > 128;
  const int BN = wide ? 192 : 128;
  // max_ctas < SM count leaves SMs to a kernel on another stream (a weight-gradient GEMM next to this NVLink-bound kernel);
  // arrivals are counted per tile, so the grid size does not enter the protocol
  const bool whole = max_ctas <= 0 || max_ctas >= sm_count();
  const bool pair = whole && wide && rows % (2 * BM) == 0 && (long long)(M / (2 * BM)) * ((N + 191) / 192) >= sm_count() / 2;
  const int kt = (K + 127) / 128;
  CUtensorMap tmA, tmB;
  int rc = cached_tmap(&tmA, A, 1, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, 128);
  if (rc != ELFA_OK) return rc;
  rc = cached_tmap(&tmB, B, 1, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)(pair ? BN / 2 : BN), 128);
  if (rc != ELFA_OK) return rc;
  OutMaps om{};
  rc = make_tmap_2d(&om.sfa, sfa, 4, (uint64_t)((M + 127) / 128) * kt, 128, 512, 1, 128, false);
  if (rc != ELFA_OK) return rc;
  rc = make_tmap_2d(&om.sfb, sfb, 4, (uint64_t)((N + 127) / 128 + 1) * kt, 128, 512, (uint32_t)(wide ? 2 : 1), 128, false);
  if (rc != ELFA_OK) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = out; p.ldc = ld_out;
  p.alpha = 1.f;
  p.status = st;
  p.sfb_atoms = (N + 127) / 128;
  CommParams c{};
  c.rank = rank; c.world = world; c.rows_per_rank = rows;
  c.wait_cycles = wait_cycles_of(wait_ms);
  for (int i = 0; i < world; ++i) { c.peer_recv[i] = peer_recv[i]; c.peer_flags[i] = peer_flags[i]; }
  c.my_flags = static_cast<const unsigned int*>(my_flags);
  c.my_recv = reinterpret_cast<const __nv_bfloat16*>(peer_recv[rank]);
  c.rs_out = static_cast<__nv_bfloat16*>(out);
  c.ld_out = ld_out;
  c.chunk_major = 1;
  c.slot_chunks = (long long)(rows / BM) * ((N + BN - 1) / BN) * (BN / 64);
  *arrivals_io += (unsigned)((rows / BM) * ((N + BN - 1) / BN));
  c.flag_target = *arrivals_io;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int ctas = whole ? sm_count() : max_ctas;
  if (pair) return launch_gemm<192, false, false, COMM_RS, true, true>(tmA, tmB, p, ctas, s, &tmA, &c, &om);
  if (wide) return launch_gemm<192, false, false, COMM_RS, false, true>(tmA, tmB, p, ctas, s, &tmA, &c, &om);
  return launch_gemm<128, false, false, COMM_RS, false, true>(tmA, tmB, p, ctas, s, &tmA, &c, &om);
}

// Columns a receive slot of the fused reduce-scatter kernels must hold for an N-column output: N rounded up to whole tiles
// of every tile width the kernels may choose.
ELFA_API int elfa_gemm_rs_slot_cols(int N) {
  const int a = (N + 127) / 128 * 128, b = (N + 191) / 192 * 192, c = (N + 255) / 256 * 256;
  return std::max(a, std::max(b, c));
}
