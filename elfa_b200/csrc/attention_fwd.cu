// Causal (or full) softmax attention forward on tcgen05: S = Q K^T and O_j = P V are tensor-memory
// MMAs, the online softmax runs in registers between them, K/V tiles arrive by TMA.
//
// The reference has no CUDA attention; its definition of the op is the Futhark sketch
// (reference: src/futhark/attention.fut:28-51 causal SDPA, :94-165 blocked attention with
// log-sum-exp). This kernel is the Blackwell realisation used by the GPT model family.
//
// One CTA handles a PAIR of 128-row query tiles (A = tile 2p, B = tile 2p+1) of one (batch, head):
//   warp 0      : TMA producer (Q tiles once, then K_j / V_j per 128-key block)
//   warp 1      : issues every tcgen05.mma
//   warps 2-3   : idle (they complete the first warp group, which hands its registers to the other two)
//   warps 4-7   : softmax + output accumulation of tile A (one thread per query row)
//   warps 8-11  : the same for tile B
// Registers: the kernel is compiled for 168 per thread; the first warp group shrinks to 72 and the softmax groups grow
// to 208 (setmaxnreg), which lets a softmax thread hold its whole S row.
// While one warp group runs exp() on its S tile, the tensor core works on the other tile, so the
// two pipelines hide each other. K_j and V_j are loaded once for both tiles.
// Tensor memory: S_A | S_B | O_A | O_B (4 x 128 fp32 columns). P (bf16) goes through shared
// memory in the 128-byte-swizzled K-major layout the MMA expects. O accumulates in tensor memory
// across the key blocks; the exponent uses a row maximum that is allowed to lag behind the true
// one by up to 2^8, and only when a row's maximum grows by more than that is O rescaled in
// tensor memory (tcgen05.ld / multiply / tcgen05.st), which is rare after the first blocks. Each
// S row is read from tensor memory once.
// Every wait is bounded (status word + abort flag), as in the GEMM.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

constexpr int ATT_THREADS = 384;
constexpr int SUB_BYTES = 128 * 128;  // one [128 rows x 64 bf16] swizzled sub-tile

// Grouped-query attention: H query heads share Hkv key / value heads (H / Hkv consecutive query heads per key head); the
// fused tensor then holds H + 2 * Hkv heads per token: [q heads | k heads | v heads].
// Packed sequences: `doc_start[b, s]` is the position of the first token of the document that token s belongs to; a query
// sees keys in [doc_start, s] only, and key blocks that lie wholly before a query tile's first document are skipped.
struct AttnFwdParams {
  int S, B, H, hd;
  int Hkv;
  const int* doc_start;              // [B, S] or null
  __nv_bfloat16* O;
  long long o_stride_s, o_stride_b;  // elements; head stride = hd
  float* lse;                        // [B, H, S]
  float scale_log2;
  int causal;
  int n_qtiles;
  unsigned int* status;
};

enum { BAR_Q = 0, BAR_KFULL, BAR_VFULL, BAR_KFREE, BAR_VFREE, BAR_SFULL0, BAR_SFULL1, BAR_PREADY0, BAR_PREADY1, BAR_OFULL0, BAR_OFULL1,
       BAR_KFULL_B, BAR_KFREE_B, BAR_SREAD0, BAR_SREAD1, BAR_COUNT };

template <int HDP, int KST>
struct AttnSmem {
  static constexpr int NSUB = HDP / 64;
  static constexpr int Q_OFF = 0;                              // [2 tiles][NSUB]
  static constexpr int K_OFF = Q_OFF + 2 * NSUB * SUB_BYTES;   // [KST stages][NSUB]
  static constexpr int V_OFF = K_OFF + KST * NSUB * SUB_BYTES; // [NSUB]
  static constexpr int P_OFF = V_OFF + NSUB * SUB_BYTES;       // [2 tiles][2]
  static constexpr int BAR_OFF = P_OFF + 4 * SUB_BYTES;
  static constexpr int TOTAL = BAR_OFF + BAR_COUNT * 8 + 16;
  static constexpr int DYN = TOTAL + 1024;
};

// PT = true: the probabilities stay in tensor memory - each softmax thread writes its row's bf16 P over the first 64 columns
// of the S tile it came from (two values per 32-bit column) and the P V product reads its A operand from there - instead of
// going through a 128-byte-swizzled shared-memory tile and an async-proxy fence.
// ONE = true: a softmax thread loads its whole S row (128 fp32) into registers with four back-to-back tensor-memory loads and
// one wait, takes the maximum and the exponentials from the registers - one tensor-memory latency per key block instead of
// eight dependent ones.
// ONE && !PT ("early S"): P goes through shared memory, so the S columns are free as soon as the row sits in registers. The
// softmax warps say so (BAR_SREAD) and the MMA warp issues S of the NEXT key block (K is double buffered) while the
// exponentials of this one are computed: the softmax of a tile then never waits for a tensor-core product, and the P V
// product leaves its critical path.
template <int HDP, bool PT, bool ONE>
__global__ void __launch_bounds__(ATT_THREADS, 1) attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const AttnFwdParams p) {
  constexpr bool EARLY = ONE && !PT;
  using L = AttnSmem<HDP, EARLY ? 2 : 1>;
  constexpr int NSUB = L::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one-dimensional grid, longest work first over the WHOLE grid (a pair's length grows with its index under a causal mask):
  // every (batch, head) runs its last pair before any runs its second-to-last, so the short CTAs fill the tail
  const int npairs = (p.n_qtiles + 1) / 2;
  const int hb = (int)(blockIdx.x % (unsigned)(p.H * p.B));
  const int h = hb % p.H, b = hb / p.H;
  const int pair = npairs - 1 - (int)(blockIdx.x / (unsigned)(p.H * p.B));
  // tile B always exists; tile A is absent when the pair is a lone last tile
  const bool has_a = 2 * pair + 1 < p.n_qtiles;
  const int tile_a = 2 * pair, tile_b = has_a ? 2 * pair + 1 : 2 * pair;
  const int n_kv = (p.S + 127) / 128;
  const int n_a = has_a ? (p.causal ? tile_a + 1 : n_kv) : 0;
  const int n_b = p.causal ? tile_b + 1 : n_kv;
  const int kvh = h / (p.H / p.Hkv);                      // key / value head of this query head
  // first key block any row of the pair can see (documents start at non-decreasing positions along the sequence)
  const int j0 = p.doc_start ? p.doc_start[(long long)b * p.S + (has_a ? tile_a : tile_b) * 128] / 128 : 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQKV);
    for (int i = 0; i < BAR_COUNT; ++i) mbar_init(bar(i), (i == BAR_PREADY0 || i == BAR_PREADY1 || i == BAR_SREAD0 || i == BAR_SREAD1) ? 4 : 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t TM_S[2] = {tmem_base + 0, tmem_base + 128};
  const uint32_t TM_O[2] = {tmem_base + 256, tmem_base + 256 + HDP};

  // each register change sits inside its own branch: after a join the allocator has to assume the smaller of the two limits
  if (warp < 4) {
  reg_dec<72>();
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const int ntile = has_a ? 2 : 1;
      mbar_expect_tx(bar(BAR_Q), ntile * NSUB * SUB_BYTES);
      for (int t = has_a ? 0 : 1; t < 2; ++t) {
        const int q0 = (t == 0 ? tile_a : tile_b) * 128;
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d(sbase + L::Q_OFF + (t * NSUB + s) * SUB_BYTES, &tmQKV, s * 64, 0 * p.H + h, b, q0, bar(BAR_Q));
      }
      if constexpr (EARLY) {
        // K runs one block ahead in two stages (stage = block parity); V has one buffer
        auto load_k = [&](int j) {
          const int jj = j - j0, st = jj & 1;
          if (jj >= 2 && !mbar_wait(bar(st ? BAR_KFREE_B : BAR_KFREE), ((jj >> 1) - 1) & 1, abort_flag, p.status)) return false;
          const uint32_t full = bar(st ? BAR_KFULL_B : BAR_KFULL);
          mbar_expect_tx(full, NSUB * SUB_BYTES);
          for (int s = 0; s < NSUB; ++s)
            tma_load_4d(sbase + L::K_OFF + (st * NSUB + s) * SUB_BYTES, &tmQKV, s * 64, p.H + kvh, b, j * 128, full);
          return true;
        };
        bool okp = load_k(j0);
        for (int j = j0; j < n_b && okp; ++j) {
          if (j + 1 < n_b && !load_k(j + 1)) break;
          if (j > j0 && !mbar_wait(bar(BAR_VFREE), (j - j0 - 1) & 1, abort_flag, p.status)) break;
          mbar_expect_tx(bar(BAR_VFULL), NSUB * SUB_BYTES);
          for (int s = 0; s < NSUB; ++s)
            tma_load_4d(sbase + L::V_OFF + s * SUB_BYTES, &tmQKV, s * 64, p.H + p.Hkv + kvh, b, j * 128, bar(BAR_VFULL));
        }
      } else {
      for (int j = j0; j < n_b; ++j) {
        if (j > j0 && !mbar_wait(bar(BAR_KFREE), (j - j0 - 1) & 1, abort_flag, p.status)) break;
        mbar_expect_tx(bar(BAR_KFULL), NSUB * SUB_BYTES);
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d(sbase + L::K_OFF + s * SUB_BYTES, &tmQKV, s * 64, p.H + kvh, b, j * 128, bar(BAR_KFULL));
        if (j > j0 && !mbar_wait(bar(BAR_VFREE), (j - j0 - 1) & 1, abort_flag, p.status)) break;
        mbar_expect_tx(bar(BAR_VFULL), NSUB * SUB_BYTES);
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d(sbase + L::V_OFF + s * SUB_BYTES, &tmQKV, s * 64, p.H + p.Hkv + kvh, b, j * 128, bar(BAR_VFULL));
      }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The warp runs converged; one elected lane issues the tensor-core instructions (descriptors stay uniform).
    {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, HDP, false, true);
      auto wait = [&](int bi, uint32_t ph) { return __all_sync(0xffffffffu, mbar_wait(bar(bi), ph, abort_flag, p.status)) != 0; };
      auto commit = [&](int bi) {
        if (elect_one()) tc_commit(bar(bi));
        __syncwarp();
      };
      // descriptors as (low, high) words: per K step only a small constant is added to the low word
      const uint64_t dq = make_smem_desc(sbase + L::Q_OFF, 16, 1024, 2), dk = make_smem_desc(sbase + L::K_OFF, 16, 1024, 2);
      const uint64_t dp = make_smem_desc(sbase + L::P_OFF, 16, 1024, 2), dv = make_smem_desc(sbase + L::V_OFF, SUB_BYTES, 1024, 2);
      const uint32_t q_lo = (uint32_t)dq, q_hi = (uint32_t)(dq >> 32), k_lo = (uint32_t)dk, k_hi = (uint32_t)(dk >> 32);
      const uint32_t p_lo = (uint32_t)dp, p_hi = (uint32_t)(dp >> 32), v_lo = (uint32_t)dv, v_hi = (uint32_t)(dv >> 32);
      auto issue_s = [&](int t, int st = 0) {  // S_t = Q_t K^T (K from stage st)
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < HDP / 16; ++kk) {
            const uint32_t off = ((kk / 4) * SUB_BYTES + (kk % 4) * 32) >> 4;
            tc_mma_f16_lh(TM_S[t], q_lo + ((t * NSUB * SUB_BYTES) >> 4) + off, q_hi, k_lo + ((st * NSUB * SUB_BYTES) >> 4) + off, k_hi,
                          idesc_s, kk != 0);
          }
          tc_commit(bar(BAR_SFULL0 + t));
        }
        __syncwarp();
      };
      auto issue_o = [&](int t, int j) {  // O_t += P_t V_j
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t poff = ((kk / 4) * SUB_BYTES + (kk % 4) * 32) >> 4;
            if (PT)   // A = P from tensor memory: 16 keys of this K step = 8 columns
              tc_mma_f16_ts_lh(TM_O[t], TM_S[t] + kk * 8, v_lo + ((kk * 2048) >> 4), v_hi, idesc_o, (j != j0 || kk != 0) ? 1u : 0u);
            else
              tc_mma_f16_lh(TM_O[t], p_lo + ((t * 2 * SUB_BYTES) >> 4) + poff, p_hi, v_lo + ((kk * 2048) >> 4), v_hi, idesc_o,
                            (j != j0 || kk != 0) ? 1u : 0u);
          }
          tc_commit(bar(BAR_OFULL0 + t));
        }
        __syncwarp();
      };
      bool ok = wait(BAR_Q, 0) && wait(BAR_KFULL, 0);
      if (ok) {
        tc_fence_after();
        if (n_a > 0) issue_s(0);
        issue_s(1);
        commit(BAR_KFREE);
      }
      if constexpr (EARLY) {
        for (int j = j0; j < n_b && ok; ++j) {
          const int jj = j - j0;
          const uint32_t ph = jj & 1;
          if (j + 1 < n_b) {
            // S of the next key block, as soon as the rows of this one sit in the softmax threads' registers
            const int st = (jj + 1) & 1;
            if (!wait(st ? BAR_KFULL_B : BAR_KFULL, ((jj + 1) >> 1) & 1)) break;
            if (j + 1 < n_a) {
              if (!wait(BAR_SREAD0, ph)) break;
              tc_fence_after();
              issue_s(0, st);
            }
            if (!wait(BAR_SREAD1, ph)) break;
            tc_fence_after();
            issue_s(1, st);
            commit(st ? BAR_KFREE_B : BAR_KFREE);
          }
          if (!wait(BAR_VFULL, ph)) break;
          if (j < n_a) {
            if (!wait(BAR_PREADY0, ph)) break;
            tc_fence_after();
            issue_o(0, j);
          }
          if (!wait(BAR_PREADY1, ph)) break;
          tc_fence_after();
          issue_o(1, j);
          commit(BAR_VFREE);
        }
      } else {
      for (int j = j0; j < n_b && ok; ++j) {
        const uint32_t ph = (j - j0) & 1;
        if (!wait(BAR_VFULL, ph)) break;
        if (j < n_a) {
          if (!wait(BAR_PREADY0, ph)) break;
          tc_fence_after();
          issue_o(0, j);
          if (j + 1 < n_a) {
            if (!wait(BAR_KFULL, ph ^ 1)) break;
            tc_fence_after();
            issue_s(0);
          }
        }
        if (!wait(BAR_PREADY1, ph)) break;
        tc_fence_after();
        issue_o(1, j);
        commit(BAR_VFREE);
        if (j + 1 < n_b) {
          if (!wait(BAR_KFULL, ph ^ 1)) break;
          tc_fence_after();
          issue_s(1);
          commit(BAR_KFREE);
        }
      }
      }
    }
  }
  } else {
    reg_inc<208>();
    // ---------------------------------------------------------------- softmax warp groups
    const int t = (warp - 4) >> 2;  // 0: tile A, 1: tile B
    const int quarter = warp & 3;
    const int n_t = t == 0 ? n_a : n_b;
    const int tile = t == 0 ? tile_a : tile_b;
    const int row_local = quarter * 32 + lane;
    const int row = tile * 128 + row_local;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t p_row = sbase + L::P_OFF + t * 2 * SUB_BYTES + row_local * 128;
    float m = -INFINITY, l = 0.f;   // m: the maximum used in the exponent (may lag the true maximum)
    bool ok = true;
    // packed sequences: first key this row may see, and the largest such position in the tile (its last row's)
    const int lower = p.doc_start ? p.doc_start[(long long)b * p.S + min(row, p.S - 1)] : 0;
    const int lower_max = p.doc_start ? p.doc_start[(long long)b * p.S + min(tile * 128 + 127, p.S - 1)] : 0;
    for (int j = j0; j < n_t; ++j) {
      const uint32_t ph = (j - j0) & 1;
      ok = mbar_wait(bar(BAR_SFULL0 + t), ph, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int key0 = j * 128;
      const int limit = p.causal ? row : (p.S - 1);       // last key this row may see
      const bool need_mask = key0 + 127 > (p.causal ? tile * 128 : p.S - 1) || key0 < lower_max;
      if constexpr (ONE) {
        uint32_t r[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(TM_S[t] + lane_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_ld_wait();
        if constexpr (EARLY) {   // the S columns may be overwritten by the next key block's product
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(BAR_SREAD0 + t));
        }
        bool o_landed = false;   // whether the previous P V product is known to have completed
        if (need_mask) {   // warp-uniform: only diagonal / ragged / document-boundary tiles pay for the per-element test
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (key0 + i > limit || key0 + i < lower) r[i] = 0xff800000u;   // -inf
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 128; i += 2)
          mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
        if (j == j0) {
          m = mx;
        } else {
          const bool grow = mx - m > 8.f;
          if (__any_sync(0xffffffffu, grow)) {
            ok = mbar_wait(bar(BAR_OFULL0 + t), (j - j0 - 1) & 1, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            o_landed = true;
            tc_fence_after();
            const float m_new = grow ? mx : m;
            const float alpha = m_new == m ? 1.f : fast_exp2(m - m_new);
#pragma unroll 1
            for (int c = 0; c < HDP / 16; ++c) {     // narrow chunks: the S row stays in registers meanwhile
              uint32_t q[16];
              tmem_ld16(TM_O[t] + lane_addr + c * 16, q);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) q[i] = __float_as_uint(__uint_as_float(q[i]) * alpha);
              tmem_st16(TM_O[t] + lane_addr + c * 16, q);
            }
            tmem_st_wait();
            l *= alpha;
            m = m_new;
          }
        }
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
        const float sc2 = p.scale_log2;
        const uint64_t sc2x2 = pack_f32x2(sc2, sc2), negm_x2 = pack_f32x2(neg_m, neg_m);
        uint64_t lsp[2] = {0ull, 0ull};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0, x1;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[c * 32 + i]), __uint_as_float(r[c * 32 + i + 1])), sc2x2, negm_x2), x0, x1);
            const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
            lsp[(i >> 1) & 1] = add_f32x2(lsp[(i >> 1) & 1], pack_f32x2(e0, e1));
            w[i >> 1] = pack_bf16(e0, e1);
          }
          if constexpr (PT) {
            tmem_st16(TM_S[t] + lane_addr + 16 * c, w);   // the whole row is in registers: its columns may be overwritten
          } else {
            if (c == 0 && j > j0 && !o_landed) {
              // the shared-memory P tile is still the A operand of the previous P V product until that has completed
              ok = mbar_wait(bar(BAR_OFULL0 + t), (j - j0 - 1) & 1, abort_flag, p.status);
              ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int q8 = c * 4 + g;  // 16-byte chunk index along the 128 keys
                const uint32_t addr = p_row + (q8 >> 3) * SUB_BYTES + (((q8 & 7) ^ (row_local & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[g * 4]), "r"(w[g * 4 + 1]), "r"(w[g * 4 + 2]),
                             "r"(w[g * 4 + 3]) : "memory");
              }
            }
          }
        }
        if (!ok) break;
        float a0, a1, a2, a3;
        unpack_f32x2(lsp[0], a0, a1);
        unpack_f32x2(lsp[1], a2, a3);
        l += (a0 + a1) + (a2 + a3);
      } else {
      // Two passes over the S row in 32-column chunks (row maximum, then exponentials), each chunk loaded
      // from tensor memory while the previous one is processed: about 64 live registers instead of 128.
      uint32_t cb[2][32];
      tmem_ld32(TM_S[t] + lane_addr, cb[0]);
      // four independent chains for the maximum (scale > 0, so scaling commutes with it)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      // `need_mask` is the same for the whole warp: only diagonal / tail tiles pay for the per-element test
      auto row_max = [&](auto masked) {
        constexpr bool MASK = decltype(masked)::value;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c + 1 < 4) tmem_ld32(TM_S[t] + lane_addr + (c + 1) * 32, cb[(c + 1) & 1]);
          else tmem_ld32(TM_S[t] + lane_addr, cb[(c + 1) & 1]);          // first chunk of the second pass
          if (MASK) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float sv = __uint_as_float(cb[c & 1][i]);
              if (key0 + c * 32 + i > limit || key0 + c * 32 + i < lower) sv = -INFINITY;
              mx4[i & 3] = fmaxf(mx4[i & 3], sv);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2)   // 3-input maximum: half an instruction per element
              mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(cb[c & 1][i]), __uint_as_float(cb[c & 1][i + 1]));
          }
        }
      };
      if (need_mask) row_max(std::true_type{}); else row_max(std::false_type{});
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      if (j == j0) {
        m = mx;
      } else {
        const bool grow = mx - m > 8.f;
        if (__any_sync(0xffffffffu, grow)) {
          // rescale this warp's O rows in tensor memory; the previous P V must have landed
          ok = mbar_wait(bar(BAR_OFULL0 + t), (j - j0 - 1) & 1, abort_flag, p.status);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          const float m_new = grow ? mx : m;
          // a row that has seen no key yet (packed sequences: -inf so far) keeps factor 1: exp2(-inf + inf) would be NaN
          const float alpha = m_new == m ? 1.f : fast_exp2(m - m_new);
          tmem_ld_wait();                                  // the chunk prefetched for the second pass
#pragma unroll 1
          for (int c = 0; c < HDP / 32; ++c) {
            uint32_t q[32];
            tmem_ld32(TM_O[t] + lane_addr + c * 32, q);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) q[i] = __float_as_uint(__uint_as_float(q[i]) * alpha);
            tmem_st32(TM_O[t] + lane_addr + c * 32, q);
          }
          tmem_st_wait();
          l *= alpha;
          m = m_new;
        }
      }
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
      const float neg_m = (m == -INFINITY) ? 0.f : -m;   // a fully masked row so far: exp2(-inf) = 0 without inf - inf
      const float sc2 = p.scale_log2;
      const uint64_t sc2x2 = pack_f32x2(sc2, sc2), negm_x2 = pack_f32x2(neg_m, neg_m);
      uint64_t lsp[2] = {0ull, 0ull};      // two packed pairs of partial sums (unmasked path)
      auto row_exp = [&](auto masked) {
        constexpr bool MASK = decltype(masked)::value;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          tmem_ld_wait();
          if (c + 1 < 4) tmem_ld32(TM_S[t] + lane_addr + (c + 1) * 32, cb[(c + 1) & 1]);
          uint32_t (&r)[32] = cb[c & 1];
          if (MASK) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float sv = __uint_as_float(r[i]);
              if (key0 + c * 32 + i > limit || key0 + c * 32 + i < lower) sv = -INFINITY;
              const float e = fast_exp2(fmaf(sv, sc2, neg_m));
              ls4[i & 3] += e;
              r[i] = __float_as_uint(e);
            }
          } else {
            // packed fp32 pairs: one FFMA and one FADD instruction per two elements
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sc2x2, negm_x2), x0, x1);
              const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
              lsp[(i >> 1) & 1] = add_f32x2(lsp[(i >> 1) & 1], pack_f32x2(e0, e1));
              r[i] = __float_as_uint(e0);
              r[i + 1] = __float_as_uint(e1);
            }
          }
          if (PT) {
            // this chunk's 32 probabilities as 16 packed words over columns [16 c, 16 c + 16) of the row's own S tile: those
            // columns held S values of chunks this thread has already consumed (chunk c sits at columns [32 c, 32 c + 32))
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) w[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
            tmem_st16(TM_S[t] + lane_addr + 16 * c, w);
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int q8 = c * 4 + g;  // 16-byte chunk index along the 128 keys
              const uint32_t addr = p_row + (q8 >> 3) * SUB_BYTES + (((q8 & 7) ^ (row_local & 7)) << 4);
              const uint32_t w0 = pack_bf16(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
              const uint32_t w1 = pack_bf16(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
              const uint32_t w2 = pack_bf16(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
              const uint32_t w3 = pack_bf16(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
            }
          }
        }
      };
      if (need_mask) row_exp(std::true_type{}); else row_exp(std::false_type{});
      {
        float a0, a1, a2, a3;
        unpack_f32x2(lsp[0], a0, a1);
        unpack_f32x2(lsp[1], a2, a3);
        l += ((ls4[0] + ls4[1]) + (ls4[2] + ls4[3])) + ((a0 + a1) + (a2 + a3));
      }
      }
      if (PT) tmem_st_wait(); else fence_proxy_async();
      tc_fence_before();
      __syncwarp();                                   // one arrival per warp: 128 arrivals on one word would queue up
      if (lane == 0) mbar_arrive(bar(BAR_PREADY0 + t));
    }
    if (ok && n_t > 0) {
      ok = mbar_wait(bar(BAR_OFULL0 + t), (n_t - 1 - j0) & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && n_t > 0) {
      tc_fence_after();
      const float inv = 1.f / l;
      __nv_bfloat16* orow = p.O + (long long)row * p.o_stride_s + (long long)b * p.o_stride_b + (long long)h * p.hd;
#pragma unroll 1
      for (int c = 0; c < HDP / 32; ++c) {
        uint32_t q[32];
        tmem_ld32(TM_O[t] + lane_addr + c * 32, q);
        tmem_ld_wait();
        if (row < p.S) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int d0 = c * 32 + g * 8;
            if (d0 < p.hd) {
              uint4 vv = make_uint4(pack_bf16(__uint_as_float(q[g * 8 + 0]) * inv, __uint_as_float(q[g * 8 + 1]) * inv),
                                    pack_bf16(__uint_as_float(q[g * 8 + 2]) * inv, __uint_as_float(q[g * 8 + 3]) * inv),
                                    pack_bf16(__uint_as_float(q[g * 8 + 4]) * inv, __uint_as_float(q[g * 8 + 5]) * inv),
                                    pack_bf16(__uint_as_float(q[g * 8 + 6]) * inv, __uint_as_float(q[g * 8 + 7]) * inv));
              *reinterpret_cast<uint4*>(orow + d0) = vv;
            }
          }
        }
      }
      if (row < p.S && p.lse) p.lse[((long long)b * p.H + h) * p.S + row] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HDP, bool PT, bool ONE>
int launch_attn_fwd(const CUtensorMap& tm, const AttnFwdParams& p, cudaStream_t stream) {
  using L = AttnSmem<HDP, (ONE && !PT) ? 2 : 1>;
  auto kern = attn_fwd_kernel<HDP, PT, ONE>;
  static bool configured = false;
  if (!configured) {
    ELFA_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN));
    configured = true;
  }
  dim3 grid((unsigned)((p.n_qtiles + 1) / 2) * p.H * p.B);
  kern<<<grid, ATT_THREADS, L::DYN, stream>>>(tm, p);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

}  // namespace

// 4-D map over a fused tensor of `planes * H` heads per token: dims {hd, planes * H, B, S}, box {64, 1, 1, box_rows}.
int make_qkv_tmap(CUtensorMap* tm, const void* qkv, int S, int B, int H, int hd, long long stride_s, long long stride_b,
                  int planes, uint32_t box_rows) {
  const uint64_t dims[4] = {(uint64_t)hd, (uint64_t)planes * H, (uint64_t)B, (uint64_t)S};
  const uint64_t strides[3] = {(uint64_t)hd * 2, (uint64_t)stride_b * 2, (uint64_t)stride_s * 2};
  const uint32_t box[4] = {64, 1, 1, box_rows};
  return make_tmap_nd_bf16(tm, qkv, 4, dims, strides, box);
}

}  // namespace elfa

using namespace elfa;

// qkv: element (s, b, head, d) at s*stride_s + b*stride_b + head*hd + d (bf16); heads are [H query | Hkv key | Hkv value]
// (Hkv == H: the classic [3][H] layout). out: element (s, b, h, d) at s*o_stride_s + b*o_stride_b + h*hd + d.
// lse: [B, H, S] fp32 or null. doc_start: [B, S] int32 (first position of each token's document) or null.
ELFA_API int elfa_attention_fwd_ex(const void* qkv, long long stride_s, long long stride_b, void* out, long long o_stride_s,
                                   long long o_stride_b, float* lse, int S, int B, int H, int Hkv, int hd, float scale, int causal,
                                   const int* doc_start, void* stream) {
  ELFA_REQUIRE(qkv && out && S > 0 && B > 0 && H > 0, "attention_fwd: bad arguments");
  ELFA_REQUIRE(Hkv > 0 && H % Hkv == 0, "attention_fwd: the query heads must be a multiple of the key / value heads");
  ELFA_REQUIRE(!doc_start || causal, "attention_fwd: document masks need causal attention");
  ELFA_REQUIRE(hd % 8 == 0 && hd >= 8 && hd <= 128, "attention_fwd: head_dim must be a multiple of 8 in [8, 128]");
  ELFA_REQUIRE(stride_s % 8 == 0 && stride_b % 8 == 0 && o_stride_s % 8 == 0 && o_stride_b % 8 == 0, "attention_fwd: strides must be multiples of 8");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "attention_fwd: no status word");
  CUtensorMap tm;
  int rc = make_qkv_tmap(&tm, qkv, S, B, H + 2 * Hkv, hd, stride_s, stride_b, 1, 128);
  if (rc != ELFA_OK) return rc;
  AttnFwdParams p{};
  p.S = S; p.B = B; p.H = H; p.hd = hd;
  p.Hkv = Hkv;
  p.doc_start = doc_start;
  p.O = static_cast<__nv_bfloat16*>(out);
  p.o_stride_s = o_stride_s; p.o_stride_b = o_stride_b;
  p.lse = lse;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.n_qtiles = (S + 127) / 128;
  p.status = st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // ELFA_ATTN_MODE selects the variant (see the kernel's template parameters): "early" = P through shared memory with the next S
  // product issued early, "one" = P in tensor memory, one pass over the row in registers, "pt" = P in tensor memory, two passes,
  // "smem" = P through shared memory, two passes.
  const char* e = getenv("ELFA_ATTN_MODE");
  const char mode = e && e[0] ? e[0] : 'e';
  if (mode == 's') return hd <= 64 ? launch_attn_fwd<64, false, false>(tm, p, s) : launch_attn_fwd<128, false, false>(tm, p, s);
  if (mode == 'p') return hd <= 64 ? launch_attn_fwd<64, true, false>(tm, p, s) : launch_attn_fwd<128, true, false>(tm, p, s);
  if (mode == 'o') return hd <= 64 ? launch_attn_fwd<64, true, true>(tm, p, s) : launch_attn_fwd<128, true, true>(tm, p, s);
  return hd <= 64 ? launch_attn_fwd<64, false, true>(tm, p, s) : launch_attn_fwd<128, false, true>(tm, p, s);
}

ELFA_API int elfa_attention_fwd(const void* qkv, long long stride_s, long long stride_b, void* out, long long o_stride_s,
                                long long o_stride_b, float* lse, int S, int B, int H, int hd, float scale, int causal, void* stream) {
  return elfa_attention_fwd_ex(qkv, stride_s, stride_b, out, o_stride_s, o_stride_b, lse, S, B, H, H, hd, scale, causal, nullptr, stream);
}
