// Fused softmax cross-entropy: one pass for the row statistics, one pass that turns the logits
// into their gradient in place, so the [tokens, vocab] probabilities are never materialised.
// Supports label smoothing, an ignore index (-100) and a vocabulary-parallel split in which every
// rank holds a [tokens, vocab/N] slice: the statistics of the slices are combined between the two
// passes.
//
// reference: src/kernels/nn_kernels.zig:269-318 (loss with label smoothing, f64 sum-exp),
// kernels/cuda/elementwise.cu:159-300 (forward / backward kernels, out-of-range target flag; the
// reference gradient carries no 1/N and no upstream gradient - both are folded into `grad_scale` here).
#include "common.cuh"
#include "elfa_native.h"

namespace elfa {
namespace {

constexpr int XENT_THREADS = 512;

struct RowStat {  // per row and per vocabulary slice
  float max, sumexp, target_logit, sumx;
};

__device__ __forceinline__ void online_combine(float& m, float& s, float m2, float s2) {
  const float nm = fmaxf(m, m2);
  if (nm == -INFINITY) return;  // both sides empty
  s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  m = nm;
}

struct StatPeers {      // vocabulary-parallel exchange: every rank's [slices][rows] statistics table (peer-addressable)
  unsigned long long p[8];
  int world, slice, rows;
};

// stats[row] = (max, sum exp(x - max), x[target] if the target is in this slice else 0, sum x).
// With `peers.world > 0` the four numbers are also stored into slot [slice][row] of every rank's table (16-byte peer
// stores over NVLink): the exchange of the vocabulary-parallel loss happens inside this kernel instead of a library
// all-gather (reference call site: src/distributed/tensor_parallel.zig:77-129 gather, then consume).
__global__ void __launch_bounds__(XENT_THREADS) xent_stats_kernel(const __nv_bfloat16* __restrict__ logits, long long ld,
                                                                  const long long* __restrict__ targets, RowStat* __restrict__ stats,
                                                                  int V, int vocab_lo, int vocab_total, unsigned int* status,
                                                                  const StatPeers peers) {
  __shared__ float sm[3][XENT_THREADS / 32];
  const int row = blockIdx.x;
  const __nv_bfloat16* x = logits + (long long)row * ld;
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f, sx = 0.f;
  for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) {
    const uint4 q = reinterpret_cast<const uint4*>(x)[v];
    const uint32_t* pq = reinterpret_cast<const uint32_t*>(&q);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[2 * j] = bf16_lo(pq[j]); f[2 * j + 1] = bf16_hi(pq[j]); }
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc += __expf(f[j] - nm); sx += f[j]; }
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += XENT_THREADS) {
    const float f = __bfloat162float(x[c]);
    online_combine(m, s, f, 1.f);
    sx += f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_combine(m, s, m2, s2);
    sx += __shfl_xor_sync(0xffffffffu, sx, o);
  }
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sm[0][wid] = m; sm[1][wid] = s; sm[2][wid] = sx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = sm[0][0], S = sm[1][0], SX = sm[2][0];
    for (int i = 1; i < XENT_THREADS / 32; ++i) { online_combine(M, S, sm[0][i], sm[1][i]); SX += sm[2][i]; }
    const long long t = targets[row];
    float tl = 0.f;
    if (t >= vocab_lo && t < vocab_lo + V) tl = __bfloat162float(x[t - vocab_lo]);
    else if (t != -100 && (t < 0 || t >= vocab_total)) atomicOr(status, (unsigned)ELFA_ST_BAD_TARGET);
    const RowStat rs{M, S, tl, SX};
    if (stats) stats[row] = rs;
    for (int i = 0; i < peers.world; ++i) {
      const int r = (peers.slice + i) % peers.world;      // own table first, then the peers, staggered by rank
      reinterpret_cast<RowStat*>(peers.p[r])[(long long)peers.slice * peers.rows + row] = rs;
    }
  }
}

// Combines `nslices` statistics per row (slice k of row r at stats[k * rows + r]) into the loss and
// rewrites the local logits slice as d loss / d logits * grad_scale.
__global__ void __launch_bounds__(XENT_THREADS) xent_grad_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                                                                 __nv_bfloat16* __restrict__ dlogits, long long ldd,
                                                                 const long long* __restrict__ targets, const RowStat* __restrict__ stats,
                                                                 int nslices, int rows, float* __restrict__ loss_out, int V, int vocab_lo,
                                                                 int vocab_total, float smoothing, const float* __restrict__ grad_scale_ptr,
                                                                 float grad_scale) {
  const int row = blockIdx.x;
  float M = -INFINITY, S = 0.f, TL = 0.f, SX = 0.f;
  for (int k = 0; k < nslices; ++k) {
    const RowStat st = stats[(long long)k * rows + row];
    online_combine(M, S, st.max, st.sumexp);
    TL += st.target_logit;
    SX += st.sumx;
  }
  const float lse = M + __logf(S);
  const long long t = targets[row];
  const bool valid = t >= 0 && t < vocab_total;
  if (threadIdx.x == 0 && loss_out) {
    float loss = 0.f;
    if (valid) loss = -((1.f - smoothing) * (TL - lse) + (smoothing / (float)vocab_total) * (SX - (float)vocab_total * lse));
    loss_out[row] = loss;
  }
  if (!dlogits) return;
  float gs = grad_scale_ptr ? grad_scale * (*grad_scale_ptr) : grad_scale;
  if (!valid) gs = 0.f;
  const float uni = smoothing / (float)vocab_total;
  const __nv_bfloat16* x = logits + (long long)row * ld;
  __nv_bfloat16* dx = dlogits + (long long)row * ldd;
  const int tcol = (int)(t - vocab_lo);  // may be outside [0, V)
  const int nvec = V / 8;
  for (int v = threadIdx.x; v < nvec; v += XENT_THREADS) {
    const uint4 q = reinterpret_cast<const uint4*>(x)[v];
    const uint32_t* pq = reinterpret_cast<const uint32_t*>(&q);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) { f[2 * j] = bf16_lo(pq[j]); f[2 * j + 1] = bf16_hi(pq[j]); }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - lse) - uni;
      if (v * 8 + j == tcol) p -= (1.f - smoothing);
      f[j] = p * gs;
    }
    reinterpret_cast<uint4*>(dx)[v] = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += XENT_THREADS) {
    float p = __expf(__bfloat162float(x[c]) - lse) - uni;
    if (c == tcol) p -= (1.f - smoothing);
    dx[c] = __float2bfloat16(p * gs);
  }
}

}  // namespace
}  // namespace elfa

using namespace elfa;

// Pass 1. stats: rows * 4 floats (this rank's slice).
ELFA_API int elfa_xent_stats(const void* logits, long long ld, const long long* targets, float* stats, int rows, int V, int vocab_lo,
                             int vocab_total, void* stream) {
  ELFA_REQUIRE(logits && targets && stats && rows > 0 && V > 0, "xent_stats: bad arguments");
  ELFA_REQUIRE(ld % 8 == 0, "xent_stats: row pitch must be a multiple of 8");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "xent: no status word");
  xent_stats_kernel<<<rows, XENT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, targets, reinterpret_cast<RowStat*>(stats), V, vocab_lo, vocab_total, st, StatPeers{});
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Pass 1 of the vocabulary-parallel loss with the exchange inside the kernel: this rank's statistics go to slot [slice] of
// every rank's table (peer_tables: `world` device addresses of [world][rows][4] fp32 tables in peer-addressable memory).
// A barrier over the group (elfa_symm_barrier) must follow before any rank runs pass 2 on its table.
ELFA_API int elfa_xent_stats_push(const void* logits, long long ld, const long long* targets, const unsigned long long* peer_tables,
                                  int slice, int world, int rows, int V, int vocab_lo, int vocab_total, void* stream) {
  ELFA_REQUIRE(logits && targets && peer_tables && rows > 0 && V > 0, "xent_stats_push: bad arguments");
  ELFA_REQUIRE(world >= 1 && world <= 8 && slice >= 0 && slice < world, "xent_stats_push: bad slice / world");
  ELFA_REQUIRE(ld % 8 == 0, "xent_stats_push: row pitch must be a multiple of 8");
  unsigned int* st = status_word();
  ELFA_REQUIRE(st != nullptr, "xent: no status word");
  StatPeers sp{};
  for (int i = 0; i < world; ++i) {
    ELFA_REQUIRE((peer_tables[i] & 15) == 0, "xent_stats_push: tables must be 16-byte aligned");
    sp.p[i] = peer_tables[i];
  }
  sp.world = world; sp.slice = slice; sp.rows = rows;
  xent_stats_kernel<<<rows, XENT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, targets, nullptr, V, vocab_lo, vocab_total, st, sp);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}

// Pass 2. stats: nslices * rows * 4 floats (slice-major). dlogits may alias logits (in place) or be
// null (loss only). loss_out: rows floats (per-token loss) or null. The gradient is multiplied by
// grad_scale and, if grad_scale_ptr is not null, by the device scalar it points to.
ELFA_API int elfa_xent_grad(void* logits, long long ld, void* dlogits, long long ldd, const long long* targets, const float* stats,
                            int nslices, float* loss_out, int rows, int V, int vocab_lo, int vocab_total, float smoothing,
                            const float* grad_scale_ptr, float grad_scale, void* stream) {
  ELFA_REQUIRE(logits && targets && stats && rows > 0 && V > 0 && nslices > 0, "xent_grad: bad arguments");
  ELFA_REQUIRE(ld % 8 == 0 && (!dlogits || ldd % 8 == 0), "xent_grad: row pitch must be a multiple of 8");
  xent_grad_kernel<<<rows, XENT_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), ld, static_cast<__nv_bfloat16*>(dlogits), ldd, targets,
      reinterpret_cast<const RowStat*>(stats), nslices, rows, loss_out, V, vocab_lo, vocab_total, smoothing, grad_scale_ptr, grad_scale);
  ELFA_CUDA(cudaGetLastError());
  ::elfa::count_launches(1);
  return ELFA_OK;
}
