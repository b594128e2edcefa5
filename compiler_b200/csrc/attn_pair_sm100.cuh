// Attention forward, two query tiles per CTA (256 query rows), persistent.
//
// Same arithmetic as attn_fwd_tcgen05_kernel; the schedule differs.  A CTA owns
// work items (256 query rows of one batch*head; see item_at for their order) and keeps
// two independent 128-row tiles in flight so the tensor core always has one tile's
// MMAs to run while the other tile's rows are in their softmax:
//
//   warps 0-3   softmax + epilogue of tile 0 (one query row per thread)
//   warps 4-7   softmax + epilogue of tile 1
//   warp  8     TMA producer: Q (both tiles) per item, K / V blocks in 2-stage rings
//               shared by both tiles (K and V are read once per 256 rows)
//   warp  10    one lane copies finished O tiles from a staging buffer in shared memory
//               to global memory (bulk tensor stores)
//   warp  11    idle (it completes the third warpgroup so that setmaxnreg can move
//               registers from it to the softmax warpgroups)
//   warp  9     issues tcgen05.mma (whole warp in the loop, one elected lane issuing) in the
//               order S0 = Q0 K(0)^T, S1 = Q1 K(0)^T, then per key block j:
//                 O0 += P0(j) V(j), S0 = Q0 K(j+1)^T, O1 += P1(j) V(j), S1 = Q1 K(j+1)^T
//               and, when the causal mask leaves tile 0 without a block in the item's last
//               step, the next item's S0 = Q0 K(0)^T in that slot (Q has one barrier pair
//               per tile for this)
//
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 columns each; P(j) overwrites
// the first 64 columns of its own S buffer as packed 16-bit pairs, so S(j+1) of a
// tile is issued only after that tile's P(j) V(j) MMA, which the in-order tensor
// pipe completes first.  Barriers carry running phase counters, so the rings keep
// turning across work items: the producer prefetches the next item's Q / K / V and
// the issuer starts its first S while the softmax warps still store the previous O.
#pragma once

#include "sm100.cuh"

namespace b200 {
namespace attn {
namespace pair {

using namespace sm100;

constexpr int TILE_M = 128;           // query rows per tile
constexpr int CTA_M = 2 * TILE_M;     // query rows per work item
constexpr int BLOCK_N = 128;          // keys per block
constexpr int KV_STAGES = 2;          // K ring
constexpr int V_STAGES = 2;           // V ring (a third stage was measured: no gain)
constexpr int THREADS = 384;  // 3 warpgroups: softmax 0, softmax 1, {producer, issuer, 2 idle}
constexpr int TMEM_COLS = 512;
constexpr int S_COLS = 128;
constexpr int O_COL0 = 2 * S_COLS;
constexpr float kRescaleThreshold = 8.0f;
#ifndef B200_ATTN_POLY_PAIRS
#define B200_ATTN_POLY_PAIRS 1  // pairs per group of 4 that take the polynomial exp2
#endif
// P is handed to the tensor core in two parts, so that the first part's P V MMAs run while
// the rest of the row is still being exponentiated.  Measured on causal [8,32,4096,128]: an
// even split (64 + 64 keys) 1160 TFLOP/s, 96 + 32 keys 1152.
#ifndef B200_ATTN_FIRST_KEYS
#define B200_ATTN_FIRST_KEYS 64
#endif
constexpr int kFirstKeys = B200_ATTN_FIRST_KEYS;  // multiple of 32 (a 16-column TMEM store)
#ifndef B200_ATTN_POLL_ONE
#define B200_ATTN_POLL_ONE 0
#endif

struct Params {
  int H, N, ZH;   // N = query rows per head
  int NK;          // keys per head; under the causal mask query row i sees keys <= i + NK - N
  int64_t lse_z, lse_h;  // element strides of lse over batch and head
  int kv_group;    // query heads per K / V head
  int wave_heads;  // (batch, head) pairs whose K / V are meant to share the L2 at one time
  float scale_log2;  // scale * log2(e)
  int causal;
  float *lse;
  uint32_t idesc_qk, idesc_pv;
  unsigned int *status;
};

template <int D> struct Smem {
  static constexpr int BOX_BYTES = 128 * 128;              // 128 rows x 128 B
  static constexpr int TILE_BYTES = (D / 64) * BOX_BYTES;  // one Q tile, K block or V block
  static constexpr int Q_OFF = 0;                          // two tiles
  static constexpr int K_OFF = 2 * TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int O_OFF = V_OFF + V_STAGES * TILE_BYTES;  // staging of one finished O tile
  static constexpr int BAR_OFF = O_OFF + TILE_BYTES;
  static constexpr int BYTES = BAR_OFF + 256 + 1024;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *tm, uint32_t bar,
                                            int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"((uint64_t)tm), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap *tm, uint32_t src, int x, int y,
                                             int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::
                   "l"((uint64_t)tm), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// packed pairs of fp32: one instruction for two lanes of the row
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)),
        "l"(*reinterpret_cast<unsigned long long *>(&c)));
  return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
  return *reinterpret_cast<float2 *>(&d);
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 fsub2(float2 a, float2 b) {
  unsigned long long d;
  asm("sub.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
  return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 fadd2_rm(float2 a, float2 b) {  // round towards -inf
  unsigned long long d;
  asm("add.rm.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
  return *reinterpret_cast<float2 *>(&d);
}
// 2^v for a pair, on the FMA / integer pipes instead of the special-function unit
// (which is the busiest pipe of this kernel): v = floor(v) + f, 2^f by a cubic with
// max relative error 8.6e-5 on [0,1) (below half an ulp of the 16-bit P it feeds),
// 2^floor(v) by adding floor(v) to the exponent field.  floor(v) comes out of the low
// mantissa bits of v + 1.5*2^23 rounded towards -inf.  Inputs below -127 (including
// the -inf of masked keys) give a value below 2^-126, which P rounds to zero.
__device__ __forceinline__ float2 exp2_poly2(float2 v) {
  const float kMagic = 12582912.0f;
  v.x = fmaxf(v.x, -127.0f);
  v.y = fmaxf(v.y, -127.0f);
  const float2 magic2 = make_float2(kMagic, kMagic);
  const float2 t = fadd2_rm(v, magic2);
  const float2 f = fsub2(v, fsub2(t, magic2));
  float2 p2 = ffma2(f, make_float2(0.07706635445356369f, 0.07706635445356369f),
                    make_float2(0.22764573991298676f, 0.22764573991298676f));
  p2 = ffma2(p2, f, make_float2(0.6951166391372681f, 0.6951166391372681f));
  p2 = ffma2(p2, f, make_float2(1.0f, 1.0f));
  return make_float2(__uint_as_float(__float_as_uint(p2.x) + (__float_as_uint(t.x) << 23)),
                     __uint_as_float(__float_as_uint(p2.y) + (__float_as_uint(t.y) << 23)));
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}

// One work item: 256 query rows of one (batch, head).
struct Item {
  int z, h, zh, m0;
  int nb[2];  // key blocks each tile visits
  int nb_max;
};

// The n-th step of this CTA's persistent loop.  Work is dealt out in units of two items
// of one (batch, head): the query block of rank r from the bottom and the one of rank r
// from the top.  Under the causal mask the pair visits num_qb + 1 key blocks whatever r
// is, so dealing units round-robin balances the CTAs to within one unit.  Units are
// ordered wave by wave (a wave = wave_heads heads, all of their units, pair rank by pair
// rank): the CTAs running at one time read the K / V of the same few heads, and a block
// fetched by one of them is an L2 hit for the others.
// Returns 0 past the end, 1 with `it` filled, 2 for the missing half of an odd middle.
__device__ __forceinline__ int item_at(int n, const Params &p, Item &it) {
  const int num_qb = (p.N + CTA_M - 1) / CTA_M;
  const int pairs = (num_qb + 1) / 2;
  const int u = (n >> 1) * (int)gridDim.x + (int)blockIdx.x;
  if (u >= pairs * p.ZH) return 0;
  const int per_wave = p.wave_heads * pairs;
  const int wave = u / per_wave, k = u - wave * per_wave;
  const int zh0 = wave * p.wave_heads;
  const int heads = min(p.wave_heads, p.ZH - zh0);
  const int r = k / heads;
  const int qb = (n & 1) ? r : num_qb - 1 - r;
  if ((n & 1) && r == num_qb - 1 - r) return 2;
  it.zh = zh0 + k % heads;
  it.z = it.zh / p.H;
  it.h = it.zh % p.H;
  it.m0 = qb * CTA_M;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int mt0 = it.m0 + t * TILE_M;
    if (mt0 >= p.N) {
      it.nb[t] = 0;
    } else {
      const int kv_len = p.causal ? min(p.NK, mt0 + TILE_M + (p.NK - p.N)) : p.NK;
      it.nb[t] = (kv_len + BLOCK_N - 1) / BLOCK_N;
    }
  }
  it.nb_max = max(it.nb[0], it.nb[1]);
  return 1;
}

template <typename T, int D>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_o, const Params p) {
  using L = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base + L::Q_OFF;
  const uint32_t k_smem = smem_base + L::K_OFF;
  const uint32_t v_smem = smem_base + L::V_OFF;
  const uint32_t o_stage = smem_base + L::O_OFF;
  const uint32_t bar0 = smem_base + L::BAR_OFF;
  auto q_full = [&](int t) { return bar0 + 8u * t; };           // one pair per tile, so that
  auto q_empty = [&](int t) { return bar0 + 8u * (27 + t); };   // tile 0 can move on alone
  auto k_full = [&](uint32_t s) { return bar0 + 8u * (2 + s); };
  auto k_empty = [&](uint32_t s) { return bar0 + 8u * (4 + s); };
  auto v_full = [&](uint32_t s) { return bar0 + 8u * (23 + s); };
  auto v_empty = [&](uint32_t s) { return bar0 + 8u * (23 + V_STAGES + s); };
  const uint32_t staged = bar0 + 8u * 21;      // a finished O tile sits in the staging buffer
  const uint32_t stage_free = bar0 + 8u * 22;  // its copy to global memory has read it
  auto s_full = [&](int t) { return bar0 + 8u * (10 + t); };
  auto p_full = [&](int t) { return bar0 + 8u * (12 + t); };
  auto o_full = [&](int t) { return bar0 + 8u * (14 + t); };
  auto o_empty = [&](int t) { return bar0 + 8u * (16 + t); };
  const uint32_t drain_bar = bar0 + 8u * 18;
  auto p2_full = [&](int t) { return bar0 + 8u * (19 + t); };  // second half of P
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + L::BAR_OFF + 8 * 29);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(q_full(t), 1);
      mbar_init(q_empty(t), 1);
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), TILE_M / 32);   // one arrival per softmax warp
      mbar_init(p2_full(t), TILE_M / 32);
      mbar_init(o_full(t), 1);
      mbar_init(o_empty(t), TILE_M / 32);
    }
    mbar_init(drain_bar, 1);
    mbar_init(staged, TILE_M / 32);
    mbar_init(stage_free, 1);
    *abort_flag = 0u;
    mbar_init_fence();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_o);
  }
  if (warp == 9) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Register budget: the softmax warpgroups hold a 128-wide fp32 row per thread, the
  // producer / issuer warpgroup needs little; setmaxnreg moves the difference.
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 8) {
    // ---------------------------------------------------------------- producer
    if (lane == 0) {
      uint32_t kv_it = 0, item_n = 0;
      uint32_t issued = 0, parity = 0;  // bit s: K stage, bit 2+s: V stage, bit 8+t: Q tile
      bool ok = true;
      for (int n = 0; ok; ++n) {
        Item it;
        const int step = item_at(n, p, it);
        if (step == 0) break;
        if (step == 2) continue;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!mbar_wait(q_empty(t), (item_n & 1u) ^ 1u, ctx, 1)) { ok = false; break; }
          mbar_arrive_expect_tx(q_full(t), L::TILE_BYTES);
#pragma unroll
          for (int b = 0; b < D / 64; ++b)
            tma_load_4d(q_smem + t * L::TILE_BYTES + b * L::BOX_BYTES, &tm_q, q_full(t), b * 64,
                        it.m0 + t * TILE_M, it.h, it.z);
          issued |= 256u << t;
          parity = (parity & ~(256u << t)) | ((item_n & 1u) << (8 + t));
        }
        if (!ok) break;
        for (int j = 0; j < it.nb_max; ++j, ++kv_it) {
          const uint32_t s = kv_it & 1u, ph = (kv_it >> 1) & 1u;
          if (!mbar_wait(k_empty(s), ph ^ 1u, ctx, 2)) { ok = false; break; }
          mbar_arrive_expect_tx(k_full(s), L::TILE_BYTES);
#pragma unroll
          for (int b = 0; b < D / 64; ++b)
            tma_load_4d(k_smem + s * L::TILE_BYTES + b * L::BOX_BYTES, &tm_k, k_full(s), b * 64,
                        j * BLOCK_N, it.h / p.kv_group, it.z);
          issued |= 1u << s;
          parity = (parity & ~(1u << s)) | (ph << s);
          const uint32_t vs = kv_it % V_STAGES, vph = (kv_it / V_STAGES) & 1u;
          if (!mbar_wait(v_empty(vs), vph ^ 1u, ctx, 3)) { ok = false; break; }
          mbar_arrive_expect_tx(v_full(vs), L::TILE_BYTES);
#pragma unroll
          for (int b = 0; b < D / 64; ++b)
            tma_load_4d(v_smem + vs * L::TILE_BYTES + b * L::BOX_BYTES, &tm_v, v_full(vs), b * 64,
                        j * BLOCK_N, it.h / p.kv_group, it.z);
          issued |= 4u << vs;
          parity = (parity & ~(4u << vs)) | (vph << (2 + vs));
        }
        ++item_n;
      }
      if (!ok) {
        // copies already issued still target this CTA's shared memory
        for (int t = 0; t < 2; ++t)
          if (issued & (256u << t)) mbar_wait_drain(q_full(t), (parity >> (8 + t)) & 1u);
        for (uint32_t s = 0; s < KV_STAGES; ++s)
          if (issued & (1u << s)) mbar_wait_drain(k_full(s), (parity >> s) & 1u);
        for (uint32_t s = 0; s < V_STAGES; ++s)
          if (issued & (4u << s)) mbar_wait_drain(v_full(s), (parity >> (2 + s)) & 1u);
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp runs this loop (uniform control flow keeps the descriptor
    // arithmetic cheap); one elected lane issues the MMAs and commits.
    const bool leader = elect_one();
    uint32_t kv_base = 0, item_n = 0;
    uint32_t blocks[2] = {0, 0};  // key blocks each tile has been through (barrier phases)
    uint32_t active[2] = {0, 0};  // items in which each tile had work (o_empty phase)
    bool ok = true;
    auto wait_all = [&](uint32_t bar, uint32_t parity, uint32_t site) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, site)) != 0;
    };
    // descriptor halves that never change: Q tiles, K / V stages
    constexpr uint32_t kHi = desc_hi_sw128(1024);
    const uint32_t q_lo0 = desc_lo_sw128(q_smem, 16);
    const uint32_t k_lo0 = desc_lo_sw128(k_smem, 16);
    const uint32_t v_lo0 = desc_lo_sw128(v_smem, L::BOX_BYTES);
    constexpr uint32_t kTileStep = L::TILE_BYTES >> 4;
    // S_t = Q_t K(s)^T
    auto issue_qk = [&](int t, uint32_t s) {
      const uint32_t d_tmem = tmem_base + (uint32_t)(t * S_COLS);
      const uint32_t a_lo = q_lo0 + (uint32_t)t * kTileStep;
      const uint32_t b_lo = k_lo0 + s * kTileStep;
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          constexpr uint32_t kBox = L::BOX_BYTES >> 4;
          const uint32_t off = (uint32_t)(kk / 4) * kBox + (uint32_t)(kk % 4) * 2u;
          mma_f16_ss(d_tmem, a_lo + off, kHi, b_lo + off, kHi, p.idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(s_full(t));
      }
    };
    // O_t += P_t V(s) over the key rows [0, kFirstKeys) (half 0) or [kFirstKeys, 128) (half 1)
    auto issue_pv_half = [&](int t, uint32_t s, bool first, int half) {
      const uint32_t o_tmem = tmem_base + (uint32_t)(O_COL0 + t * S_COLS);
      const uint32_t b_lo = v_lo0 + s * kTileStep;
      const uint32_t a_tmem = tmem_base + (uint32_t)(t * S_COLS);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
          if ((kk < kFirstKeys / 16) != (half == 0)) continue;
          mma_f16_ts(o_tmem, a_tmem + (uint32_t)(kk * 8), b_lo + (uint32_t)(kk * (2048 >> 4)), kHi,
                     p.idesc_pv, (!first || kk > 0) ? 1u : 0u);
        }
        if (half == 1) tc_commit(o_full(t));
      }
    };
    auto commit = [&](uint32_t bar) {
      if (leader) tc_commit(bar);
    };
    // the item after the current one is known one item ahead: when tile 0 runs out of key
    // blocks before tile 1 (causal mask), the next item's first S of tile 0 is issued in the
    // otherwise idle slot instead of waiting for tile 1's last block
    auto fetch = [&](int &n, Item &out) {
      for (;; ++n) {
        const int step = item_at(n, p, out);
        if (step == 0) return false;
        if (step == 1) { ++n; return true; }
      }
    };
    int n_next = 0;
    Item it, nx;
    bool has = fetch(n_next, it);
    bool early0 = false;  // S(0) of tile 0 of the current item was issued during the last one
    while (ok && has) {
      const bool has_nx = fetch(n_next, nx);
      bool early_next = false;
      {  // S(0) of both tiles
        const uint32_t s = kv_base & 1u, ph = (kv_base >> 1) & 1u;
        if (!early0) {
          if (!wait_all(q_full(0), item_n & 1u, 4)) { ok = false; break; }
          if (!wait_all(k_full(s), ph, 5)) { ok = false; break; }
          tc_fence_after_sync();
          if (it.nb[0] > 0) issue_qk(0, s);
          if (it.nb[0] <= 1) commit(q_empty(0));
        }
        if (!wait_all(q_full(1), item_n & 1u, 4)) { ok = false; break; }
        if (!wait_all(k_full(s), ph, 5)) { ok = false; break; }
        tc_fence_after_sync();
        if (it.nb[1] > 0) issue_qk(1, s);
        commit(k_empty(s));
        if (it.nb[1] <= 1) commit(q_empty(1));
      }
      for (int j = 0; ok && j < it.nb_max; ++j) {
        const uint32_t kv = kv_base + (uint32_t)j;
        const uint32_t s = kv & 1u, ph = (kv >> 1) & 1u;
        const uint32_t s1 = (kv + 1) & 1u, ph1 = ((kv + 1) >> 1) & 1u;
        const bool more = j + 1 < it.nb_max;
        const uint32_t vs = kv % V_STAGES, vph = (kv / V_STAGES) & 1u;
        if (!wait_all(v_full(vs), vph, 6)) { ok = false; break; }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < it.nb[t]) {
            // the previous item's O of this tile must have been read out
            if (j == 0 && !wait_all(o_empty(t), (active[t] & 1u) ^ 1u, 7)) { ok = false; break; }
            if (!wait_all(p_full(t), blocks[t] & 1u, 8)) { ok = false; break; }
            tc_fence_after_sync();
            issue_pv_half(t, vs, j == 0, 0);
            if (!wait_all(p2_full(t), blocks[t] & 1u, 13)) { ok = false; break; }
            tc_fence_after_sync();
            issue_pv_half(t, vs, j == 0, 1);
            ++blocks[t];
          } else if (t == 0 && !more && has_nx && nx.nb[0] > 0) {
            // tile 0 has no block j and nothing follows in this item
            const uint32_t kvn = kv_base + (uint32_t)it.nb_max;
            const uint32_t sn = kvn & 1u, phn = (kvn >> 1) & 1u;
            if (!wait_all(q_full(0), (item_n + 1u) & 1u, 4)) { ok = false; break; }
            if (!wait_all(k_full(sn), phn, 5)) { ok = false; break; }
            tc_fence_after_sync();
            issue_qk(0, sn);
            if (nx.nb[0] <= 1) commit(q_empty(0));
            early_next = true;
          }
          if (t == 1) commit(v_empty(vs));
          if (more) {
            if (t == 0 && !wait_all(k_full(s1), ph1, 9)) { ok = false; break; }
            tc_fence_after_sync();
            if (j + 1 < it.nb[t]) {
              issue_qk(t, s1);
              if (j + 2 == it.nb[t]) commit(q_empty(t));  // last S of this tile in this item
            }
            if (t == 1) commit(k_empty(s1));
          }
        }
      }
      kv_base += (uint32_t)it.nb_max;
      active[0] += it.nb[0] > 0 ? 1u : 0u;
      active[1] += it.nb[1] > 0 ? 1u : 0u;
      ++item_n;
      it = nx;
      has = has_nx;
      early0 = early_next;
    }
    if (leader) {
      tc_commit(drain_bar);
      mbar_wait_drain(drain_bar, 0);
    }
    __syncwarp();
  } else if (warp == 10) {
    // ---------------------------------------------------------------- O store
    // Finished O tiles reach global memory as bulk tensor copies out of the staging
    // buffer: the softmax warps fill it in the order tile 0, tile 1 of each item, one
    // lane here copies it out and hands it back.
    if (lane == 0) {
      uint32_t e = 0;  // tiles stored so far (barrier phases)
      bool ok = true;
      for (int n = 0; ok; ++n) {
        Item it;
        const int step = item_at(n, p, it);
        if (step == 0) break;
        if (step == 2) continue;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (it.nb[t] == 0) continue;
          if (!mbar_wait(staged, e & 1u, ctx, 17)) { ok = false; break; }
#pragma unroll
          for (int b = 0; b < D / 64; ++b)
            tma_store_4d(&tm_o, o_stage + b * L::BOX_BYTES, b * 64, it.m0 + t * TILE_M, it.h, it.z);
          tma_store_commit();
          tma_store_wait_read<0>();
          mbar_arrive(stage_free);
          ++e;
        }
      }
      tma_store_wait<0>();
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    // ---------------------------------------------------------------- softmax + epilogue
    const int t = warp >> 2;                          // tile of this warpgroup
    const int row_in_tile = (warp & 3) * 32 + lane;   // == TMEM lane of this thread
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_addr + (uint32_t)(t * S_COLS);
    const uint32_t o_tmem = tmem_base + lane_addr + (uint32_t)(O_COL0 + t * S_COLS);
    uint32_t blocks = 0;  // key blocks this tile has been through (barrier phases)
    uint32_t stored = 0;  // O tiles (of either tile) staged before the current item
    bool ok = true;
    // warp-uniform wait: the vote keeps the warp converged for the .sync.aligned
    // tensor-memory accesses that follow
    auto wait_all = [&](uint32_t bar, uint32_t parity, uint32_t site) {
#if B200_ATTN_POLL_ONE
      // one lane polls; the vote publishes its result and reconverges the warp
      bool done = true;
      if (lane == 0) done = mbar_wait(bar, parity, ctx, site);
      return __all_sync(0xffffffffu, done) != 0;
#else
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, site)) != 0;
#endif
    };
    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
    for (int n = 0; ok; ++n) {
      Item it;
      const int step = item_at(n, p, it);
      if (step == 0) break;
      if (step == 2) continue;
      const int nb = it.nb[t];
      // this tile's place in the order in which O tiles pass through the staging buffer
      const uint32_t e = stored + ((t == 1 && it.nb[0] > 0) ? 1u : 0u);
      stored += (it.nb[0] > 0 ? 1u : 0u) + (it.nb[1] > 0 ? 1u : 0u);
      if (nb == 0) continue;
      const int mt0 = it.m0 + t * TILE_M;
      const int row = mt0 + row_in_tile;
      float m_used = -INFINITY;  // running max in the scaled log2 domain
      float l = 0.f;
      for (int j = 0; j < nb; ++j, ++blocks) {
        if (!wait_all(s_full(t), blocks & 1u, 10)) { ok = false; break; }
        tc_fence_after_sync();
#ifdef B200_ATTN_SKIP_SOFTMAX
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) { mbar_arrive(p_full(t)); mbar_arrive(p2_full(t)); }
        continue;
#endif
        float x[BLOCK_N];
        uint32_t(&xr)[BLOCK_N] = reinterpret_cast<uint32_t(&)[BLOCK_N]>(x);
        // the row arrives in two halves; the max of the first half is taken while the
        // second half is still on its way from tensor memory
        tmem_ld_32x32b_x32(s_tmem, reinterpret_cast<uint32_t(&)[32]>(xr[0]));
        tmem_ld_32x32b_x32(s_tmem + 32, reinterpret_cast<uint32_t(&)[32]>(xr[32]));
        tmem_ld_wait();
        tmem_ld_32x32b_x32(s_tmem + 64, reinterpret_cast<uint32_t(&)[32]>(xr[64]));
        tmem_ld_32x32b_x32(s_tmem + 96, reinterpret_cast<uint32_t(&)[32]>(xr[96]));
        const int col0 = j * BLOCK_N;
        const bool diag = p.causal && (col0 + BLOCK_N - 1 > mt0 + (p.NK - p.N));
        const bool ragged = col0 + BLOCK_N > p.NK;
        const bool masked = diag || ragged;
        const int limit = min(p.causal ? row + (p.NK - p.N) : p.NK - 1, p.NK - 1) - col0;  // last kept column
        float mx0, mx1, mx2, mx3;
        {
          if (masked) {
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (i > limit) x[i] = -INFINITY;
          }
          mx0 = x[0]; mx1 = x[1]; mx2 = x[2]; mx3 = x[3];
#pragma unroll
          for (int i = 4; i < 60; i += 8) {
            mx0 = max3(mx0, x[i], x[i + 1]);
            mx1 = max3(mx1, x[i + 2], x[i + 3]);
            mx2 = max3(mx2, x[i + 4], x[i + 5]);
            mx3 = max3(mx3, x[i + 6], x[i + 7]);
          }
          mx0 = max3(mx0, x[60], x[61]);
          mx1 = max3(mx1, x[62], x[63]);
        }
        tmem_ld_wait();
        {
          if (masked) {
#pragma unroll
            for (int i = 64; i < BLOCK_N; ++i)
              if (i > limit) x[i] = -INFINITY;
          }
#pragma unroll
          for (int i = 64; i < BLOCK_N; i += 8) {
            mx0 = max3(mx0, x[i], x[i + 1]);
            mx1 = max3(mx1, x[i + 2], x[i + 3]);
            mx2 = max3(mx2, x[i + 4], x[i + 5]);
            mx3 = max3(mx3, x[i + 6], x[i + 7]);
          }
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
        // lazy rescale: the max used for exp2 is raised only when the true max
        // exceeds it by more than 2^kRescaleThreshold
        float alpha = 1.0f;
        bool raise = mx > m_used + kRescaleThreshold;
        if (j == 0) {
          m_used = mx;
          raise = false;
        }
        if (raise) {
          alpha = ex2(m_used - mx);
          m_used = mx;
        }
        if (j > 0 && __any_sync(0xffffffffu, raise)) {
          // O += P(j-1) V(j-1) must have landed before O is rescaled
          if (!wait_all(o_full(t), (blocks - 1u) & 1u, 11)) { ok = false; break; }
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(o_tmem + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x32(o_tmem + c * 32, r);
          }
          tmem_st_wait();
        }
        l *= alpha;
        const float2 negm2 = make_float2(-m_used, -m_used);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
        // P is handed over in two halves of 64 keys so that the first half of
        // O += P V runs while the second half is still being exponentiated.  In every
        // group of 8 keys one pair takes the polynomial exp2, three pairs the ex2 unit.
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          constexpr int kGroups0 = kFirstKeys / 8;
          uint32_t packed[kFirstKeys / 2 > 32 ? kFirstKeys / 2 : 32];  // one word per key pair
#pragma unroll
          for (int g8 = 0; g8 < BLOCK_N / 8; ++g8) {
            if ((g8 < kGroups0) != (half == 0)) continue;
            const int g = g8 - (half == 0 ? 0 : kGroups0);
            const int i = g8 * 8;
            const float2 va = ffma2(make_float2(x[i], x[i + 1]), scale2, negm2);
            const float2 vb = ffma2(make_float2(x[i + 2], x[i + 3]), scale2, negm2);
            const float2 vc = ffma2(make_float2(x[i + 4], x[i + 5]), scale2, negm2);
            const float2 vd = ffma2(make_float2(x[i + 6], x[i + 7]), scale2, negm2);
            const float2 ea = make_float2(ex2(va.x), ex2(va.y));
            const float2 eb = make_float2(ex2(vb.x), ex2(vb.y));
            const float2 ec = B200_ATTN_POLY_PAIRS >= 2 ? exp2_poly2(vc)
                                                        : make_float2(ex2(vc.x), ex2(vc.y));
            const float2 ed = B200_ATTN_POLY_PAIRS >= 1 ? exp2_poly2(vd)
                                                        : make_float2(ex2(vd.x), ex2(vd.y));
            sum_a = fadd2(sum_a, fadd2(ea, ec));
            sum_b = fadd2(sum_b, fadd2(eb, ed));
            packed[g * 4] = pack2<T>(ea.x, ea.y);
            packed[g * 4 + 1] = pack2<T>(eb.x, eb.y);
            packed[g * 4 + 2] = pack2<T>(ec.x, ec.y);
            packed[g * 4 + 3] = pack2<T>(ed.x, ed.y);
          }
          // packed words -> the columns of P: 16 columns (32 keys) per store
          constexpr int kCol0 = kFirstKeys / 2;
#pragma unroll
          for (int c = 0; c < BLOCK_N / 32; ++c) {
            if ((c < kFirstKeys / 32) != (half == 0)) continue;
            const int w0 = (c - (half == 0 ? 0 : kFirstKeys / 32)) * 16;
            tmem_st_32x32b_x16(s_tmem + (half == 0 ? 0 : kCol0) + w0,
                               reinterpret_cast<uint32_t(&)[16]>(packed[w0]));
          }
          tmem_st_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(half == 0 ? p_full(t) : p2_full(t));
        }
        l += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
      }
      if (!ok) break;
      // ---- epilogue of this tile: O / l, LSE
      if (!wait_all(o_full(t), (blocks - 1u) & 1u, 12)) { ok = false; break; }
      tc_fence_after_sync();
      uint32_t acc[D];
#pragma unroll
      for (int c = 0; c < D / 32; ++c)
        tmem_ld_32x32b_x32(o_tmem + c * 32, reinterpret_cast<uint32_t(&)[32]>(acc[c * 32]));
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_empty(t));  // O may be overwritten by the next item's first P V
      // the staging buffer is free once the copy of the tile before this one has read it
      if (e > 0 && !wait_all(stage_free, (e - 1u) & 1u, 16)) { ok = false; break; }
      {
        const float inv_l = 1.0f / l;
        // rows of 128 B in the 128-byte swizzle the tensor map expects: 16-byte chunk c of
        // row r sits at chunk c ^ (r % 8), so the 32 rows of a warp spread over all banks
        const uint32_t row_smem = o_stage + (uint32_t)row_in_tile * 128u;
        const uint32_t sw = (uint32_t)row_in_tile & 7u;
#pragma unroll
        for (int q = 0; q < D / 8; ++q) {
          const uint32_t x0 = pack2<T>(__uint_as_float(acc[q * 8 + 0]) * inv_l, __uint_as_float(acc[q * 8 + 1]) * inv_l);
          const uint32_t x1 = pack2<T>(__uint_as_float(acc[q * 8 + 2]) * inv_l, __uint_as_float(acc[q * 8 + 3]) * inv_l);
          const uint32_t x2 = pack2<T>(__uint_as_float(acc[q * 8 + 4]) * inv_l, __uint_as_float(acc[q * 8 + 5]) * inv_l);
          const uint32_t x3 = pack2<T>(__uint_as_float(acc[q * 8 + 6]) * inv_l, __uint_as_float(acc[q * 8 + 7]) * inv_l);
          const uint32_t addr = row_smem + (uint32_t)(q / 8) * L::BOX_BYTES + ((((uint32_t)q & 7u) ^ sw) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x0), "r"(x1), "r"(x2), "r"(x3) : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(staged);
        if (row < p.N && p.lse != nullptr)
          p.lse[it.z * p.lse_z + it.h * p.lse_h + row] = m_used * 0.6931471805599453f + logf(l);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <typename T, int D>
static int launch(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                  const CUtensorMap &to, const Params &p, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  auto kernel = attn_fwd_pair_kernel<T, D>;
  constexpr int smem = Smem<D>::BYTES;
  if (dev < 64 && !configured[dev]) {
    B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  const int num_qb = (p.N + CTA_M - 1) / CTA_M;
  const int units = ((num_qb + 1) / 2) * p.ZH;  // pairs of query blocks
  const int grid = units < sm_count() ? units : sm_count();
  Params pw = p;
  // heads per wave: about 8 MiB of K and V (measured on [8,32,4096,128]: 4 heads per wave
  // 1135 TFLOP/s causal, 16 heads 1122, 64 heads 1076; B200OPS_ATTN_WAVE overrides)
  static const int wave_env = getenv("B200OPS_ATTN_WAVE") ? atoi(getenv("B200OPS_ATTN_WAVE")) : 0;
  const int64_t kv_bytes = 2 * (int64_t)p.NK * D * (int64_t)sizeof(T);
  pw.wave_heads = wave_env > 0 ? wave_env : (int)((8 << 20) / kv_bytes);
  if (pw.wave_heads < 1) pw.wave_heads = 1;
  if (pw.wave_heads > p.ZH) pw.wave_heads = p.ZH;
  kernel<<<grid, THREADS, smem, stream>>>(tq, tk, tv, to, pw);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // namespace pair
}  // namespace attn
}  // namespace b200
