// Attention forward, two query tiles per CTA (256 query rows), persistent.
//
// Same arithmetic as attn_fwd_tcgen05_kernel; the schedule differs.  A CTA owns
// work items (256 query rows of one batch*head), heaviest first, and keeps two
// independent 128-row tiles in flight so the tensor core always has one tile's
// MMAs to run while the other tile's rows are in their softmax:
//
//   warps 0-3   softmax + epilogue of tile 0 (one query row per thread)
//   warps 4-7   softmax + epilogue of tile 1
//   warp  8     TMA producer: Q (both tiles) per item, K / V blocks in 2-stage rings
//               shared by both tiles (K and V are read once per 256 rows)
//   warps 10-11 idle (they complete the third warpgroup so that setmaxnreg can move
//               registers from it to the softmax warpgroups)
//   warp  9     one lane issues tcgen05.mma in the order
//                 S0 = Q0 K(0)^T, S1 = Q1 K(0)^T, then per key block j:
//                 O0 += P0(j) V(j), S0 = Q0 K(j+1)^T, O1 += P1(j) V(j), S1 = Q1 K(j+1)^T
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
constexpr int KV_STAGES = 2;
constexpr int THREADS = 384;  // 3 warpgroups: softmax 0, softmax 1, {producer, issuer, 2 idle}
constexpr int TMEM_COLS = 512;
constexpr int S_COLS = 128;
constexpr int O_COL0 = 2 * S_COLS;
constexpr float kRescaleThreshold = 8.0f;

struct Params {
  int H, N, ZH;
  float scale_log2;  // scale * log2(e)
  int causal;
  void *o;
  int64_t oz, oh, om;
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
  static constexpr int BAR_OFF = V_OFF + KV_STAGES * TILE_BYTES;
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

__device__ __forceinline__ Item decode_item(int item, const Params &p) {
  const int num_qb = (p.N + CTA_M - 1) / CTA_M;
  Item it;
  const int qb = num_qb - 1 - item / p.ZH;  // heaviest query blocks first
  it.zh = item % p.ZH;
  it.z = it.zh / p.H;
  it.h = it.zh % p.H;
  it.m0 = qb * CTA_M;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int mt0 = it.m0 + t * TILE_M;
    if (mt0 >= p.N) {
      it.nb[t] = 0;
    } else {
      const int kv_len = p.causal ? min(p.N, mt0 + TILE_M) : p.N;
      it.nb[t] = (kv_len + BLOCK_N - 1) / BLOCK_N;
    }
  }
  it.nb_max = max(it.nb[0], it.nb[1]);
  return it;
}

template <typename T, int D>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const Params p) {
  using L = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base + L::Q_OFF;
  const uint32_t k_smem = smem_base + L::K_OFF;
  const uint32_t v_smem = smem_base + L::V_OFF;
  const uint32_t bar0 = smem_base + L::BAR_OFF;
  const uint32_t q_full = bar0, q_empty = bar0 + 8;
  auto k_full = [&](uint32_t s) { return bar0 + 8u * (2 + s); };
  auto k_empty = [&](uint32_t s) { return bar0 + 8u * (4 + s); };
  auto v_full = [&](uint32_t s) { return bar0 + 8u * (6 + s); };
  auto v_empty = [&](uint32_t s) { return bar0 + 8u * (8 + s); };
  auto s_full = [&](int t) { return bar0 + 8u * (10 + t); };
  auto p_full = [&](int t) { return bar0 + 8u * (12 + t); };
  auto o_full = [&](int t) { return bar0 + 8u * (14 + t); };
  auto o_empty = [&](int t) { return bar0 + 8u * (16 + t); };
  const uint32_t drain_bar = bar0 + 8u * 18;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + L::BAR_OFF + 8 * 19);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};
  const int num_items = ((p.N + CTA_M - 1) / CTA_M) * p.ZH;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full(t), 1);
      mbar_init(p_full(t), TILE_M);
      mbar_init(o_full(t), 1);
      mbar_init(o_empty(t), TILE_M);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0u;
    mbar_init_fence();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
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
      uint32_t issued = 0, parity = 0;  // bit s: K stage, bit 2+s: V stage, bit 4: Q
      bool ok = true;
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x, ++item_n) {
        const Item it = decode_item(item, p);
        if (!mbar_wait(q_empty, (item_n & 1u) ^ 1u, ctx, 1)) { ok = false; break; }
        mbar_arrive_expect_tx(q_full, 2 * L::TILE_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int b = 0; b < D / 64; ++b)
            tma_load_4d(q_smem + t * L::TILE_BYTES + b * L::BOX_BYTES, &tm_q, q_full, b * 64,
                        it.m0 + t * TILE_M, it.h, it.z);
        issued |= 16u;
        parity = (parity & ~16u) | ((item_n & 1u) << 4);
        for (int j = 0; j < it.nb_max; ++j, ++kv_it) {
          const uint32_t s = kv_it & 1u, ph = (kv_it >> 1) & 1u;
          if (!mbar_wait(k_empty(s), ph ^ 1u, ctx, 2)) { ok = false; break; }
          mbar_arrive_expect_tx(k_full(s), L::TILE_BYTES);
#pragma unroll
          for (int b = 0; b < D / 64; ++b)
            tma_load_4d(k_smem + s * L::TILE_BYTES + b * L::BOX_BYTES, &tm_k, k_full(s), b * 64,
                        j * BLOCK_N, it.h, it.z);
          issued |= 1u << s;
          parity = (parity & ~(1u << s)) | (ph << s);
          if (!mbar_wait(v_empty(s), ph ^ 1u, ctx, 3)) { ok = false; break; }
          mbar_arrive_expect_tx(v_full(s), L::TILE_BYTES);
#pragma unroll
          for (int b = 0; b < D / 64; ++b)
            tma_load_4d(v_smem + s * L::TILE_BYTES + b * L::BOX_BYTES, &tm_v, v_full(s), b * 64,
                        j * BLOCK_N, it.h, it.z);
          issued |= 4u << s;
          parity = (parity & ~(4u << s)) | (ph << (2 + s));
        }
      }
      if (!ok) {
        // copies already issued still target this CTA's shared memory
        if (issued & 16u) mbar_wait_drain(q_full, (parity >> 4) & 1u);
        for (uint32_t s = 0; s < KV_STAGES; ++s) {
          if (issued & (1u << s)) mbar_wait_drain(k_full(s), (parity >> s) & 1u);
          if (issued & (4u << s)) mbar_wait_drain(v_full(s), (parity >> (2 + s)) & 1u);
        }
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t kv_base = 0, item_n = 0;
      uint32_t blocks[2] = {0, 0};  // key blocks each tile has been through (barrier phases)
      uint32_t active[2] = {0, 0};  // items in which each tile had work (o_empty phase)
      bool ok = true;
      auto issue_qk = [&](int t, uint32_t s) {
        const uint32_t d_tmem = tmem_base + (uint32_t)(t * S_COLS);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk / 4) * L::BOX_BYTES + (kk % 4) * 32);
          const uint64_t a_desc =
              make_smem_desc_sw128(q_smem + t * L::TILE_BYTES + off, 16, 1024);
          const uint64_t b_desc =
              make_smem_desc_sw128(k_smem + s * L::TILE_BYTES + off, 16, 1024);
          mma_f16_ss(d_tmem, a_desc, b_desc, p.idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(s_full(t));
      };
      auto issue_pv = [&](int t, uint32_t s, bool first) {
        const uint32_t o_tmem = tmem_base + (uint32_t)(O_COL0 + t * S_COLS);
#pragma unroll
        for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
          const uint64_t b_desc = make_smem_desc_sw128(
              v_smem + s * L::TILE_BYTES + kk * 2048, L::BOX_BYTES, 1024);
          const uint32_t a_tmem = tmem_base + (uint32_t)(t * S_COLS + kk * 8);
          mma_f16_ts(o_tmem, a_tmem, b_desc, p.idesc_pv, (!first || kk > 0) ? 1u : 0u);
        }
        tc_commit(o_full(t));
      };
      for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x, ++item_n) {
        const Item it = decode_item(item, p);
        if (!mbar_wait(q_full, item_n & 1u, ctx, 4)) { ok = false; break; }
        {  // S(0) of both tiles
          const uint32_t s = kv_base & 1u, ph = (kv_base >> 1) & 1u;
          if (!mbar_wait(k_full(s), ph, ctx, 5)) { ok = false; break; }
          tc_fence_after_sync();
          if (it.nb[0] > 0) issue_qk(0, s);
          if (it.nb[1] > 0) issue_qk(1, s);
          tc_commit(k_empty(s));
          if (it.nb_max == 1) tc_commit(q_empty);
        }
        for (int j = 0; ok && j < it.nb_max; ++j) {
          const uint32_t kv = kv_base + (uint32_t)j;
          const uint32_t s = kv & 1u, ph = (kv >> 1) & 1u;
          const uint32_t s1 = (kv + 1) & 1u, ph1 = ((kv + 1) >> 1) & 1u;
          const bool more = j + 1 < it.nb_max;
          if (!mbar_wait(v_full(s), ph, ctx, 6)) { ok = false; break; }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j < it.nb[t]) {
              // the previous item's O of this tile must have been read out
              if (j == 0 && !mbar_wait(o_empty(t), (active[t] & 1u) ^ 1u, ctx, 7)) { ok = false; break; }
              if (!mbar_wait(p_full(t), blocks[t] & 1u, ctx, 8)) { ok = false; break; }
              tc_fence_after_sync();
              issue_pv(t, s, j == 0);
              ++blocks[t];
            }
            if (t == 1) tc_commit(v_empty(s));
            if (more) {
              if (t == 0 && !mbar_wait(k_full(s1), ph1, ctx, 9)) { ok = false; break; }
              tc_fence_after_sync();
              if (j + 1 < it.nb[t]) issue_qk(t, s1);
              if (t == 1) {
                tc_commit(k_empty(s1));
                if (j + 2 == it.nb_max) tc_commit(q_empty);  // last S of this item issued
              }
            }
          }
        }
        kv_base += (uint32_t)it.nb_max;
        active[0] += it.nb[0] > 0 ? 1u : 0u;
        active[1] += it.nb[1] > 0 ? 1u : 0u;
      }
      tc_commit(drain_bar);
      mbar_wait_drain(drain_bar, 0);
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
    bool ok = true;
    // warp-uniform wait: the vote keeps the warp converged for the .sync.aligned
    // tensor-memory accesses that follow
    auto wait_all = [&](uint32_t bar, uint32_t parity, uint32_t site) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, site)) != 0;
    };
    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
    for (int item = blockIdx.x; ok && item < num_items; item += gridDim.x) {
      const Item it = decode_item(item, p);
      const int nb = it.nb[t];
      if (nb == 0) continue;
      const int mt0 = it.m0 + t * TILE_M;
      const int row = mt0 + row_in_tile;
      float m_used = -INFINITY;  // running max in the scaled log2 domain
      float l = 0.f;
      for (int j = 0; j < nb; ++j, ++blocks) {
        if (!wait_all(s_full(t), blocks & 1u, 10)) { ok = false; break; }
        tc_fence_after_sync();
        float x[BLOCK_N];
        {
          uint32_t(&r)[BLOCK_N] = reinterpret_cast<uint32_t(&)[BLOCK_N]>(x);
#pragma unroll
          for (int c = 0; c < BLOCK_N / 32; ++c)
            tmem_ld_32x32b_x32(s_tmem + c * 32, reinterpret_cast<uint32_t(&)[32]>(r[c * 32]));
          tmem_ld_wait();
        }
        const int col0 = j * BLOCK_N;
        const bool diag = p.causal && (col0 + BLOCK_N - 1 > mt0);
        const bool ragged = col0 + BLOCK_N > p.N;
        if (diag || ragged) {
          const int limit = min(p.causal ? row : p.N - 1, p.N - 1);  // last kept column
#pragma unroll
          for (int i = 0; i < BLOCK_N; ++i)
            if (col0 + i > limit) x[i] = -INFINITY;
        }
        float mx0 = x[0], mx1 = x[1], mx2 = x[2], mx3 = x[3];
#pragma unroll
        for (int i = 4; i < BLOCK_N; i += 4) {
          mx0 = fmaxf(mx0, x[i]);
          mx1 = fmaxf(mx1, x[i + 1]);
          mx2 = fmaxf(mx2, x[i + 2]);
          mx3 = fmaxf(mx3, x[i + 3]);
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
        uint32_t packed[BLOCK_N / 2];
#pragma unroll
        for (int i = 0; i < BLOCK_N; i += 4) {
          const float2 va = ffma2(make_float2(x[i], x[i + 1]), scale2, negm2);
          const float2 vb = ffma2(make_float2(x[i + 2], x[i + 3]), scale2, negm2);
          const float2 ea = make_float2(ex2(va.x), ex2(va.y));
          const float2 eb = make_float2(ex2(vb.x), ex2(vb.y));
          sum_a = fadd2(sum_a, ea);
          sum_b = fadd2(sum_b, eb);
          packed[i / 2] = pack2<T>(ea.x, ea.y);
          packed[i / 2 + 1] = pack2<T>(eb.x, eb.y);
        }
        l += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
#pragma unroll
        for (int c = 0; c < BLOCK_N / 64; ++c)
          tmem_st_32x32b_x32(s_tmem + c * 32,
                             reinterpret_cast<const uint32_t(&)[32]>(packed[c * 32]));
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(p_full(t));
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
      mbar_arrive(o_empty(t));  // the issuer may overwrite O with the next item's first P V
      if (row < p.N) {
        const float inv_l = 1.0f / l;
        T *orow = reinterpret_cast<T *>(p.o) + it.z * p.oz + it.h * p.oh + (int64_t)row * p.om;
#pragma unroll
        for (int q = 0; q < D / 8; ++q) {
          uint4 out;
          out.x = pack2<T>(__uint_as_float(acc[q * 8 + 0]) * inv_l, __uint_as_float(acc[q * 8 + 1]) * inv_l);
          out.y = pack2<T>(__uint_as_float(acc[q * 8 + 2]) * inv_l, __uint_as_float(acc[q * 8 + 3]) * inv_l);
          out.z = pack2<T>(__uint_as_float(acc[q * 8 + 4]) * inv_l, __uint_as_float(acc[q * 8 + 5]) * inv_l);
          out.w = pack2<T>(__uint_as_float(acc[q * 8 + 6]) * inv_l, __uint_as_float(acc[q * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4 *>(orow + q * 8) = out;
        }
        if (p.lse != nullptr)
          p.lse[(int64_t)it.zh * p.N + row] = m_used * 0.6931471805599453f + logf(l);
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
                  const Params &p, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  auto kernel = attn_fwd_pair_kernel<T, D>;
  constexpr int smem = Smem<D>::BYTES;
  if (dev < 64 && !configured[dev]) {
    B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  const int items = ((p.N + CTA_M - 1) / CTA_M) * p.ZH;
  const int grid = items < sm_count() ? items : sm_count();
  kernel<<<grid, THREADS, smem, stream>>>(tq, tk, tv, p);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // namespace pair
}  // namespace attn
}  // namespace b200
