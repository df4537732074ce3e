// Attention backward on tcgen05, recompute style: only O and the row log-sum-exp are kept by
// forward; the probabilities are rebuilt per [128 x 128] block of (query, key) pairs.
//
//   delta = rowsum(dO * O)                                    (small pre-pass)
//   MODE_DKV (CTA owns a key tile, loops over query tiles), everything transposed so that the key
//   index runs along the tensor-memory lanes:
//       S^T = K Q^T, dP^T = V dO^T                                 (tensor memory, fp32)
//       P^T = exp(S^T*scale - lse[q]), dS^T = P^T * (dP^T - delta[q]) * scale  -> bf16, written back
//       into tensor memory over the fp32 values they were computed from
//       dV += P^T dO,  dK += dS^T Q                                 (A operand read from tensor memory)
//   MODE_DQ  (CTA owns a query tile, loops over key tiles):
//       S = Q K^T, dP = dO V^T;  dS -> bf16 in tensor memory;  dQ += dS K
// P / dS never touch shared memory; the Q / K / V / dO tiles are used K-major or MN-major through
// the descriptor only, so no transpose is materialised. The inner tiles are double buffered (TMA
// runs one iteration ahead). Two passes keep every accumulator in tensor memory and make the
// result deterministic (no floating-point atomics on dQ).
//
// reference: the op is defined by src/futhark/attention.fut:28-51; the reference ships no
// attention backward at all.
//
// Roles per CTA (320 threads): warp 0 TMA, warp 1 MMA issue, warps 2-9 compute (warps w and w+4
// share a tensor-memory lane quarter and split the 128 columns in halves).
#include <type_traits>

#include "common.cuh"
#include "elfa_native.h"

namespace elfa {

int make_qkv_tmap(CUtensorMap* tm, const void* qkv, int S, int B, int H, int hd, long long stride_s, long long stride_b,
                  int planes, uint32_t box_rows);

namespace {

constexpr int ATTB_THREADS = 320;
constexpr int SUBB = 128 * 128;

// Grouped-query attention (Hkv < H): the key-tile pass runs one CTA per key / value head and walks the query tiles of every
// query head of its group one after the other, so dK / dV are summed in a fixed order; the query-tile pass reads the group's
// key head. Packed sequences (doc_start, see the forward kernel): masked like the causal diagonal, block pairs without a
// visible (query, key) pair are skipped.
struct AttnBwdParams {
  int S, B, H, hd;
  int Hkv;
  const int* doc_start;   // [B, S] or null
  const float* lse;    // [B, H, S] natural log
  const float* delta;  // [B, H, S]
  __nv_bfloat16* dqkv;
  long long d_stride_s, d_stride_b;
  float scale, scale_log2;
  int causal;
  int n_tiles;
  unsigned int* status;
};

enum { BB_RES = 0, BB_INFULL0, BB_INFULL1, BB_INFREE0, BB_INFREE1, BB_S, BB_DP, BB_P, BB_DS, BB_ACC, BB_COUNT };

template <int HDP>
struct BwdSmem {
  static constexpr int NSUB = HDP / 64;
  static constexpr int RES0 = 0;
  static constexpr int RES1 = RES0 + NSUB * SUBB;
  static constexpr int IN0 = RES1 + NSUB * SUBB;           // [2 slots][NSUB]
  static constexpr int IN1 = IN0 + 2 * NSUB * SUBB;        // [2 slots][NSUB]
  static constexpr int VEC_OFF = IN1 + 2 * NSUB * SUBB;    // lse2 / delta / document start of the inner query tile: [2 slots][3][128] words
  static constexpr int BAR_OFF = VEC_OFF + 2 * 3 * 128 * 4;
  static constexpr int TOTAL = BAR_OFF + BB_COUNT * 8 + 16;
  static constexpr int DYN = TOTAL + 1024;
};

// delta[b,h,s] = sum_d dO[s,b,h,d] * O[s,b,h,d]; one warp per (s,b,h).
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                                         long long o_stride_s, long long o_stride_b, float* __restrict__ delta, int S,
                                                         int B, int H, int hd) {
  const long long gw = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const long long total = (long long)S * B * H;
  if (gw >= total) return;
  const int h = (int)(gw % H);
  const int b = (int)((gw / H) % B);
  const int s = (int)(gw / ((long long)H * B));
  const long long off = (long long)s * o_stride_s + (long long)b * o_stride_b + (long long)h * hd;
  float acc = 0.f;
  for (int v = lane; v < hd / 8; v += 32) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + off + v * 8);
    const uint4 d = *reinterpret_cast<const uint4*>(dout + off + v * 8);
    const uint32_t* pa = reinterpret_cast<const uint32_t*>(&a);
    const uint32_t* pd = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
    for (int j = 0; j < 4; ++j) acc += bf16_lo(pa[j]) * bf16_lo(pd[j]) + bf16_hi(pa[j]) * bf16_hi(pd[j]);
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[((long long)b * H + h) * S + s] = acc;
}

template <int HDP, bool DKV>
__global__ void __launch_bounds__(ATTB_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO, const AttnBwdParams p) {
  using L = BwdSmem<HDP>;
  constexpr int NSUB = L::NSUB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + BB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* svec = reinterpret_cast<float*>(smem + L::VEC_OFF);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one-dimensional grid, heaviest outer tile first over the whole grid: every (batch, head) runs its longest tile before any
  // runs its second longest, so the short CTAs fill the tail of the launch
  const int n_heads = DKV ? p.Hkv : p.H;
  const int hb = (int)(blockIdx.x % (unsigned)(n_heads * p.B));
  const int rank = (int)(blockIdx.x / (unsigned)(n_heads * p.B));
  const int h = hb % n_heads, b = hb / n_heads;     // DKV: key / value head; DQ: query head
  const int group = p.H / p.Hkv;
  const int kvh = DKV ? h : h / group;
  // outer tile and the inner range it loops over
  const int outer = DKV ? rank : p.n_tiles - 1 - rank;   // heaviest first in both modes
  int in_begin = DKV ? (p.causal ? outer : 0) : 0;
  int in_end = DKV ? p.n_tiles : (p.causal ? outer + 1 : p.n_tiles);
  const int* dstart = p.doc_start ? p.doc_start + (long long)b * p.S : nullptr;
  if (dstart) {
    if (DKV) {      // query tiles whose first row's document starts after this key tile see none of it
      int e = in_begin + 1;
      while (e < in_end && dstart[e * 128] <= outer * 128 + 127) ++e;
      in_end = e;
    } else {
      in_begin = dstart[outer * 128] / 128;
    }
  }
  const int n_in = in_end - in_begin;                     // inner tiles per head
  const int n_iter = DKV ? n_in * group : n_in;           // DKV: every query head of the group in turn

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmQKV);
    prefetch_tmap(&tmDO);
    for (int i = 0; i < BB_COUNT; ++i) mbar_init(bar(i), (i == BB_P || i == BB_DS) ? 8 : 1);   // one arrival per compute warp
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
  // fp32 S (or S^T) and dP (or dP^T); their bf16 successors P / dS overwrite the first 64 columns
  const uint32_t TM_S = tmem_base, TM_DP = tmem_base + 128, TM_ACC0 = tmem_base + 256, TM_ACC1 = tmem_base + 256 + HDP;

  // resident pair: (K_j, V_j) in DKV mode, (Q_i, dO_i) in DQ mode; the inner pair is the other one
  const uint32_t sRes0 = sbase + L::RES0, sRes1 = sbase + L::RES1;
  auto sIn0 = [&](int slot) { return sbase + L::IN0 + slot * NSUB * SUBB; };
  auto sIn1 = [&](int slot) { return sbase + L::IN1 + slot * NSUB * SUBB; };

  if (warp == 0) {
    if (lane == 0) {
      auto load_qdo = [&](uint32_t dq, uint32_t ddo, int hq, int tile, int bar_id) {
        for (int s = 0; s < NSUB; ++s) {
          tma_load_4d(dq + s * SUBB, &tmQKV, s * 64, hq, b, tile * 128, bar(bar_id));
          tma_load_4d(ddo + s * SUBB, &tmDO, s * 64, hq, b, tile * 128, bar(bar_id));
        }
      };
      auto load_kv = [&](uint32_t dk, uint32_t dv, int tile, int bar_id) {
        for (int s = 0; s < NSUB; ++s) {
          tma_load_4d(dk + s * SUBB, &tmQKV, s * 64, p.H + kvh, b, tile * 128, bar(bar_id));
          tma_load_4d(dv + s * SUBB, &tmQKV, s * 64, p.H + p.Hkv + kvh, b, tile * 128, bar(bar_id));
        }
      };
      mbar_expect_tx(bar(BB_RES), 2 * NSUB * SUBB);
      if (DKV) load_kv(sRes0, sRes1, outer, BB_RES); else load_qdo(sRes0, sRes1, h, outer, BB_RES);
      for (int it = 0; it < n_iter; ++it) {
        const int slot = it & 1;
        if (it >= 2 && !mbar_wait(bar(BB_INFREE0 + slot), ((it >> 1) - 1) & 1, abort_flag, p.status)) break;
        mbar_expect_tx(bar(BB_INFULL0 + slot), 2 * NSUB * SUBB);
        if (DKV) load_qdo(sIn0(slot), sIn1(slot), kvh * group + it / n_in, in_begin + it % n_in, BB_INFULL0 + slot);
        else load_kv(sIn0(slot), sIn1(slot), in_begin + it, BB_INFULL0 + slot);
      }
    }
  } else if (warp == 1) {
    // MMA issuer: the warp runs converged, one elected lane issues (descriptors stay in uniform registers)
    {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, HDP, false, true);   // A from tensor memory, B MN-major
      auto wait = [&](int bi, uint32_t ph) { return __all_sync(0xffffffffu, mbar_wait(bar(bi), ph, abort_flag, p.status)) != 0; };
      // Issue order per iteration: [dV(it)] S(it+1) | dK or dQ (it) dP(it+1). The products of the next inner tile are
      // queued as soon as the tensor-memory columns they overwrite have been consumed (S after the probabilities were
      // read, dP after dS was multiplied), so the exponentials of tile it+1 overlap the accumulator MMAs of tile it.
      // DKV: S^T = K Q^T, dP^T = V dO^T (A = resident);  DQ: S = Q K^T, dP = dO V^T (A = resident)
      auto issue_s = [&](int it) {
        const uint32_t a0 = sRes0, b0 = sIn0(it & 1);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < HDP / 16; ++kk) {
            const uint32_t off = (kk / 4) * SUBB + (kk % 4) * 32;
            tc_mma_f16(TM_S, make_smem_desc(a0 + off, 16, 1024, 2), make_smem_desc(b0 + off, 16, 1024, 2), idesc_s, kk != 0);
          }
          tc_commit(bar(BB_S));
        }
        __syncwarp();
      };
      auto issue_dp = [&](int it) {
        const uint32_t a1 = sRes1, b1 = sIn1(it & 1);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < HDP / 16; ++kk) {
            const uint32_t off = (kk / 4) * SUBB + (kk % 4) * 32;
            tc_mma_f16(TM_DP, make_smem_desc(a1 + off, 16, 1024, 2), make_smem_desc(b1 + off, 16, 1024, 2), idesc_s, kk != 0);
          }
          tc_commit(bar(BB_DP));
        }
        __syncwarp();
      };
      bool ok = wait(BB_RES, 0);
      if (ok && n_iter > 0) {
        ok = wait(BB_INFULL0, 0);
        if (ok) {
          tc_fence_after();
          issue_s(0);
          issue_dp(0);
        }
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int slot = it & 1;
        const uint32_t b0 = sIn0(slot), b1 = sIn1(slot);
        if (!wait(BB_P, it & 1)) { ok = false; break; }      // the S columns have been read (DKV: P is in place)
        tc_fence_after();
        if (DKV) {
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)   // dV[key, d] += sum_q P^T[key, q] dO[q, d]
              tc_mma_f16_ts(TM_ACC0, TM_S + kk * 8, make_smem_desc(b1 + kk * 2048, SUBB, 1024, 2), idesc_acc, (it | kk) != 0);
          }
          __syncwarp();
        }
        if (it + 1 < n_iter) {
          if (!wait(BB_INFULL0 + ((it + 1) & 1), ((it + 1) >> 1) & 1)) { ok = false; break; }
          tc_fence_after();
          issue_s(it + 1);
        }
        if (!wait(BB_DS, it & 1)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          if (DKV) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)   // dK[key, d] += sum_q dS^T[key, q] Q[q, d]
              tc_mma_f16_ts(TM_ACC1, TM_DP + kk * 8, make_smem_desc(b0 + kk * 2048, SUBB, 1024, 2), idesc_acc, (it | kk) != 0);
          } else {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)   // dQ[q, d] += sum_key dS[q, key] K[key, d]
              tc_mma_f16_ts(TM_ACC0, TM_DP + kk * 8, make_smem_desc(b0 + kk * 2048, SUBB, 1024, 2), idesc_acc, (it | kk) != 0);
          }
          tc_commit(bar(BB_INFREE0 + slot));
        }
        __syncwarp();
        if (it + 1 < n_iter) issue_dp(it + 1);
      }
      if (ok) {
        if (elect_one()) tc_commit(bar(BB_ACC));
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- compute warps
    const int cw = warp - 2;
    const int ct = threadIdx.x - 64;              // 0..255 inside the compute group
    const int quarter = warp & 3;
    const int half = cw >> 2;                     // which 64 columns of the block
    const int row_local = quarter * 32 + lane;    // lane of tensor memory: key row (DKV) or query row (DQ)
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    float lse2 = 0.f, dlt = 0.f;
    bool row_ok = true;
    int lower = 0;                                // DQ: first key this query row may see (packed sequences)
    if (!DKV) {
      const int row = outer * 128 + row_local;
      row_ok = row < p.S;
      if (row_ok) {   // negated / pre-scaled like the shared-memory vectors of the other mode
        lse2 = -p.lse[((long long)b * p.H + h) * p.S + row] * LOG2E;
        dlt = -p.delta[((long long)b * p.H + h) * p.S + row] * p.scale;
        if (dstart) lower = dstart[row];
      }
    }
    for (int it = 0; it < n_iter; ++it) {
      const int q_tile = DKV ? in_begin + it % n_in : outer;
      const int k_tile = DKV ? outer : in_begin + it;
      const int hq = DKV ? kvh * group + it / n_in : h;      // query head of this iteration
      float* vl = svec + (it & 1) * 384;          // [0,128) lse2, [128,256) delta, [256,384) document start of the inner query tile
      const int* vdoc = reinterpret_cast<const int*>(vl + 256);
      if (DKV) {
        const int qi = ct & 127;
        const int qrow = q_tile * 128 + qi;
        const long long idx = ((long long)b * p.H + hq) * p.S + qrow;
        // stored negated (and delta pre-multiplied by the softmax scale) so that both uses are one fused multiply-add
        if (ct < 128) {
          vl[qi] = qrow < p.S ? -p.lse[idx] * LOG2E : -INFINITY;   // -inf -> exp2(-inf) = 0 for rows past the end
          if (dstart) reinterpret_cast<int*>(vl + 256)[qi] = dstart[min(qrow, p.S - 1)];
        } else {
          vl[128 + qi] = qrow < p.S ? -p.delta[idx] * p.scale : 0.f;
        }
        named_bar_sync(1, 256);
      }
      // After a timeout the loop keeps running without touching tensor memory so that every warp
      // still reaches the named barriers below (the waits return immediately once the abort flag is up).
      if (ok) ok = mbar_wait(bar(BB_S), it & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
      const bool diag = p.causal && q_tile == k_tile;
      float ev[64];                      // this thread's 64 probabilities (fp32, kept for dS)
      uint32_t keep[32];                 // ... and as bf16 pairs (P, then dS)
      // ---- phase 1: P = exp2(S * scale - lse). `diag` (and a ragged last tile) is uniform over the CTA: only
      // those tiles pay for the per-element mask test. The per-query vectors come from shared memory four at a time.
      const float sc2 = p.scale_log2;
      const uint64_t sc2x2 = pack_f32x2(sc2, sc2), scx2 = pack_f32x2(p.scale, p.scale);
      auto phase1 = [&](auto masked_tag) {
        constexpr bool MASK = decltype(masked_tag)::value;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = half * 64 + c * 32;
          uint32_t rs[32];
          tmem_ld32(TM_S + lane_addr + col0, rs);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            float l4[4] = {lse2, lse2, lse2, lse2};
            if (DKV) {
              const float4 t4 = *reinterpret_cast<const float4*>(vl + col0 + i);
              l4[0] = t4.x; l4[1] = t4.y; l4[2] = t4.z; l4[3] = t4.w;
            }
            if (MASK) {
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int col = col0 + i + u;
                float e = fast_exp2(fmaf(__uint_as_float(rs[i + u]), sc2, l4[u]));
                // DKV: lane = key, column = query -> masked when key > query; DQ: lane = query, column = key
                bool masked = DKV ? (diag && row_local > col) : (!row_ok || (diag && col > row_local));
                if (dstart) masked = masked || (DKV ? (k_tile * 128 + row_local < vdoc[col]) : (k_tile * 128 + col < lower));
                if (masked) e = 0.f;
                ev[c * 32 + i + u] = e;
              }
            } else {
#pragma unroll
              for (int u = 0; u < 4; u += 2) {   // packed pairs: one FFMA instruction per two elements
                float x0, x1;
                unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(rs[i + u]), __uint_as_float(rs[i + u + 1])), sc2x2,
                                       pack_f32x2(l4[u], l4[u + 1])), x0, x1);
                ev[c * 32 + i + u] = fast_exp2(x0);
                ev[c * 32 + i + u + 1] = fast_exp2(x1);
              }
            }
          }
        }
      };
      if (ok) {
        // a document boundary inside the block pair: the key tile starts before the query tile's last document does
        const bool doc_mask = dstart && k_tile * 128 < dstart[min(q_tile * 128 + 127, p.S - 1)];
        const bool any_mask = diag || doc_mask || (!DKV && (outer + 1) * 128 > p.S);
        if (any_mask) phase1(std::true_type{}); else phase1(std::false_type{});
      }
      if (DKV) {
        // The bf16 results go back into tensor memory on top of fp32 columns: a row's 128 values take
        // 64 columns, so the upper half lands on columns the partner warp (other half, same lanes) was
        // reading. All 256 compute threads therefore finish their loads before anyone stores.
        tc_fence_before();
        named_bar_sync(1, 256);
        tc_fence_after();
        if (ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) keep[i] = pack_bf16(ev[2 * i], ev[2 * i + 1]);
          uint32_t t0[16], t1[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) { t0[i] = keep[i]; t1[i] = keep[16 + i]; }
          tmem_st16(TM_S + lane_addr + half * 32, t0);
          tmem_st16(TM_S + lane_addr + half * 32 + 16, t1);
          tmem_st_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BB_P));
      } else {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(BB_P));            // the S columns have been read: the next S product may overwrite them
      }
      // ---- phase 2: dS = P * (dP - delta) * scale
      if (ok) ok = mbar_wait(bar(BB_DP), it & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        if (!ok) break;
        const int col0 = half * 64 + c * 32;
        uint32_t rd[32];
        tmem_ld32(TM_DP + lane_addr + col0, rd);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float d4[4] = {dlt, dlt, dlt, dlt};
          if (DKV) {
            const float4 t4 = *reinterpret_cast<const float4*>(vl + 128 + col0 + i);
            d4[0] = t4.x; d4[1] = t4.y; d4[2] = t4.z; d4[3] = t4.w;
          }
          // dS = P * (dP * scale - delta * scale): one packed FFMA and one packed FMUL per two elements
          float x0, x1, x2, x3;
          const uint64_t t01 = fma_f32x2(pack_f32x2(__uint_as_float(rd[i]), __uint_as_float(rd[i + 1])), scx2, pack_f32x2(d4[0], d4[1]));
          const uint64_t t23 = fma_f32x2(pack_f32x2(__uint_as_float(rd[i + 2]), __uint_as_float(rd[i + 3])), scx2, pack_f32x2(d4[2], d4[3]));
          unpack_f32x2(fma_f32x2(pack_f32x2(ev[c * 32 + i], ev[c * 32 + i + 1]), t01, 0ull), x0, x1);
          unpack_f32x2(fma_f32x2(pack_f32x2(ev[c * 32 + i + 2], ev[c * 32 + i + 3]), t23, 0ull), x2, x3);
          keep[c * 16 + (i >> 1)] = pack_bf16(x0, x1);
          keep[c * 16 + (i >> 1) + 1] = pack_bf16(x2, x3);
        }
      }
      tc_fence_before();
      named_bar_sync(1, 256);            // every thread has read its dP columns before dS overwrites them
      tc_fence_after();
      if (ok) {
        uint32_t t0[16], t1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { t0[i] = keep[i]; t1[i] = keep[16 + i]; }
        tmem_st16(TM_DP + lane_addr + half * 32, t0);
        tmem_st16(TM_DP + lane_addr + half * 32 + 16, t1);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BB_DS));
    }
    // ---------------------------------------------------------------- epilogue
    if (ok) {
      ok = mbar_wait(bar(BB_ACC), 0, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const int row = outer * 128 + row_local;   // key row (DKV) or query row (DQ)
      constexpr int CHUNKS = HDP / 32;           // 32-column chunks per accumulator
      constexpr int NACC = DKV ? 2 : 1;
      // split the NACC * CHUNKS chunks between the two warps that share this lane quarter
      for (int idx = half; idx < NACC * CHUNKS; idx += 2) {
        const int acc = idx / CHUNKS, c = idx % CHUNKS;
        uint32_t r[32];
        tmem_ld32((acc == 0 ? TM_ACC0 : TM_ACC1) + lane_addr + c * 32, r);
        tmem_ld_wait();
        // DKV: acc 0 = dV, acc 1 = dK of key head `kvh`; DQ: dQ of query head `h`; heads are [H query | Hkv key | Hkv value]
        const int head = DKV ? (acc == 0 ? p.H + p.Hkv + kvh : p.H + kvh) : h;
        if (row < p.S) {
          __nv_bfloat16* dst = p.dqkv + (long long)row * p.d_stride_s + (long long)b * p.d_stride_b + (long long)head * p.hd;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int d0 = c * 32 + g * 8;
            if (d0 < p.hd) {
              uint4 v = make_uint4(pack_bf16(__uint_as_float(r[g * 8]), __uint_as_float(r[g * 8 + 1])),
                                   pack_bf16(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3])),
                                   pack_bf16(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5])),
                                   pack_bf16(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7])));
              *reinterpret_cast<uint4*>(dst + d0) = v;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HDP, bool DKV>
int launch_attn_bwd(const CUtensorMap& tmQKV, const CUtensorMap& tmDO, const AttnBwdParams& p, cudaStream_t stream) {
  using L = BwdSmem<HDP>;
  auto kern = attn_bwd_kernel<HDP, DKV>;
  static bool configured = false;
  if (!configured) {
    ELFA_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN));
    configured = true;
  }
  dim3 grid((unsigned)p.n_tiles * (DKV ? p.Hkv : p.H) * p.B);
  kern<<<grid, ATTB_THREADS, L::DYN, stream>>>(tmQKV, tmDO, p);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// Gradients of attention w.r.t. the fused qkv tensor (heads [H query | Hkv key | Hkv value], see elfa_attention_fwd_ex).
// `out` / `dout` share strides (o_stride_*), `dqkv` has the layout of qkv with its own strides; `delta` is [B, H, S] fp32
// scratch. doc_start: [B, S] int32 or null.
ELFA_API int elfa_attention_bwd_ex(const void* qkv, long long stride_s, long long stride_b, const void* out, const void* dout,
                                   long long o_stride_s, long long o_stride_b, const float* lse, float* delta, void* dqkv,
                                   long long d_stride_s, long long d_stride_b, int S, int B, int H, int Hkv, int hd, float scale,
                                   int causal, const int* doc_start, void* stream) {
  ELFA_REQUIRE(qkv && out && dout && lse && delta && dqkv && S > 0 && B > 0 && H > 0, "attention_bwd: bad arguments");
  ELFA_REQUIRE(Hkv > 0 && H % Hkv == 0, "attention_bwd: the query heads must be a multiple of the key / value heads");
  ELFA_REQUIRE(!doc_start || causal, "attention_bwd: document masks need causal attention");
  ELFA_REQUIRE(hd % 8 == 0 && hd >= 8 && hd <= 128, "attention_bwd: head_dim must be a multiple of 8 in [8, 128]");
  ELFA_REQUIRE(stride_s % 8 == 0 && stride_b % 8 == 0 && o_stride_s % 8 == 0 && o_stride_b % 8 == 0 && d_stride_s % 8 == 0 &&
                   d_stride_b % 8 == 0,
               "attention_bwd: strides must be multiples of 8");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "attention_bwd: no status word");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long nwarps = (long long)S * B * H;
  attn_delta_kernel<<<(unsigned)((nwarps + 7) / 8), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(out),
                                                                 static_cast<const __nv_bfloat16*>(dout), o_stride_s, o_stride_b,
                                                                 delta, S, B, H, hd);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  CUtensorMap tmQKV, tmDO;
  int rc = make_qkv_tmap(&tmQKV, qkv, S, B, H + 2 * Hkv, hd, stride_s, stride_b, 1, 128);
  if (rc != ELFA_OK) return rc;
  rc = make_qkv_tmap(&tmDO, dout, S, B, H, hd, o_stride_s, o_stride_b, 1, 128);
  if (rc != ELFA_OK) return rc;
  AttnBwdParams p{};
  p.S = S; p.B = B; p.H = H; p.hd = hd;
  p.Hkv = Hkv;
  p.doc_start = doc_start;
  p.lse = lse; p.delta = delta;
  p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.d_stride_s = d_stride_s; p.d_stride_b = d_stride_b;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.n_tiles = (S + 127) / 128;
  p.status = st;
  if (hd <= 64) {
    rc = launch_attn_bwd<64, true>(tmQKV, tmDO, p, s);
    if (rc != ELFA_OK) return rc;
    return launch_attn_bwd<64, false>(tmQKV, tmDO, p, s);
  }
  rc = launch_attn_bwd<128, true>(tmQKV, tmDO, p, s);
  if (rc != ELFA_OK) return rc;
  return launch_attn_bwd<128, false>(tmQKV, tmDO, p, s);
}

ELFA_API int elfa_attention_bwd(const void* qkv, long long stride_s, long long stride_b, const void* out, const void* dout,
                                long long o_stride_s, long long o_stride_b, const float* lse, float* delta, void* dqkv,
                                long long d_stride_s, long long d_stride_b, int S, int B, int H, int hd, float scale, int causal,
                                void* stream) {
  return elfa_attention_bwd_ex(qkv, stride_s, stride_b, out, dout, o_stride_s, o_stride_b, lse, delta, dqkv, d_stride_s, d_stride_b, S, B,
                               H, H, hd, scale, causal, nullptr, stream);
}
