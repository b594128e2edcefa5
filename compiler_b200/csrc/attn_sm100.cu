// Attention forward for sm_100a: S = Q K^T and O += P V on tcgen05 tensor
// cores with S / P / O in tensor memory and an online softmax between them.
//
// Semantics follow attn_fwd_causal_kernel (ops/suite/perf/attn_fwd_causal.py:
// 19-57): scores scaled by `scale`, keys n > m masked to -inf when causal, fp32
// max / exp / sum, out = softmax(scores) V; LSE is the natural log of the sum
// of exp of the scaled masked scores (ops/suite/dev/flash_varlen_fwd_kernel.py:
// 309, 318-320).  The reference program holds a whole key row block per query
// row; here keys are visited in blocks of 128 with a running max and sum.
//
// One CTA owns 128 query rows of one (batch, head):
//   warp 4   TMA producer: Q once, then K / V blocks into 2-stage rings
//   warp 5   one lane issues tcgen05.mma: S(j+1) = Q K(j+1)^T runs while the
//            softmax warps work on S(j); then O += P(j) V(j)
//   warps 0-3 one query row per thread: tcgen05.ld of the S row, scale, mask,
//            running max with lazy rescale of O, exp2, P written back as 16-bit
//            (tensor memory over the S columns, or shared memory), final
//            normalisation and store of O and LSE
// Every wait is bounded; an expired wait sets the status word and drains.
#include "attn_pair_sm100.cuh"
#include "attn_simt.cuh"
#include "sm100.cuh"

#include <stdlib.h>

namespace b200 {
namespace attn {

using namespace sm100;

constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 128;
constexpr int KV_STAGES = 2;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int S_COLS = 128;
constexpr int O_COL0 = 2 * S_COLS;
// lazy rescale: the running max used for exp2 is only raised when the true
// max exceeds it by more than this many powers of two
constexpr float kRescaleThreshold = 8.0f;

struct Params {
  int H, N;      // N = query rows per head
  int NK;        // keys per head; under the causal mask query row i sees keys <= i + NK - N
  int64_t lse_z, lse_h;  // element strides of lse over batch and head
  int kv_group;  // query heads per K / V head (1 = one K / V head per query head)
  float scale_log2;  // scale * log2(e)
  int causal;
  void *o;
  int64_t oz, oh, om;
  float *lse;
  uint32_t idesc_qk, idesc_pv;
  unsigned int *status;
};

template <int D> struct Smem {
  static constexpr int BOX_BYTES = BLOCK_N * 128;            // 128 rows x 128 B
  static constexpr int TILE_BYTES = (D / 64) * BOX_BYTES;    // Q, K or V tile
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE_BYTES;
  static constexpr int V_OFF = K_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int P_OFF = V_OFF + KV_STAGES * TILE_BYTES;
  static constexpr int P_BYTES = (BLOCK_N / 64) * BOX_BYTES;
  static constexpr int bar_off(bool p_tmem) { return P_OFF + (p_tmem ? 0 : P_BYTES); }
  static constexpr int bytes(bool p_tmem) { return bar_off(p_tmem) + 256 + 1024; }
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

template <typename T, int D, bool P_TMEM>
__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q,
                        const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const Params p) {
  using L = Smem<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_smem = smem_base + L::Q_OFF;
  const uint32_t k_smem = smem_base + L::K_OFF;
  const uint32_t v_smem = smem_base + L::V_OFF;
  const uint32_t p_smem = smem_base + L::P_OFF;
  const uint32_t bar0 = smem_base + L::bar_off(P_TMEM);
  // barrier slots
  const uint32_t q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (7 + s); };
  auto s_full = [&](int s) { return bar0 + 8u * (9 + s); };
  const uint32_t p_full = bar0 + 8u * 11;
  const uint32_t o_full = bar0 + 8u * 12;
  const uint32_t drain_bar = bar0 + 8u * 13;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_gen + L::bar_off(P_TMEM) + 8 * 14);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};

  const int num_q_blocks = (p.N + BLOCK_M - 1) / BLOCK_M;
  const int qb = num_q_blocks - 1 - (int)blockIdx.x;  // heaviest query blocks first
  const int zh = blockIdx.y;
  const int z = zh / p.H, h = zh % p.H;
  const int m0 = qb * BLOCK_M;
  const int kv_len = p.causal ? min(p.NK, m0 + BLOCK_M + (p.NK - p.N)) : p.NK;
  const int nblocks = (kv_len + BLOCK_N - 1) / BLOCK_N;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
    }
    mbar_init(p_full, 128);
    mbar_init(o_full, 1);
    mbar_init(drain_bar, 1);
    *abort_flag = 0u;
    mbar_init_fence();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 5) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // -------------------------------------------------------------- producer
    if (lane == 0) {
      uint32_t issued = 0;  // bit s: K stage s, bit 2+s: V stage s, bit 4: Q
      uint32_t parity = 0;
      mbar_arrive_expect_tx(q_full, L::TILE_BYTES);
#pragma unroll
      for (int b = 0; b < D / 64; ++b)
        tma_load_4d(q_smem + b * L::BOX_BYTES, &tm_q, q_full, b * 64, m0, h, z);
      issued |= 16u;
      bool ok = true;
      for (int j = 0; ok && j < nblocks; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (uint32_t)(j / KV_STAGES) & 1u;
        if (!mbar_wait(k_empty(s), ph ^ 1u, ctx, 1)) { ok = false; break; }
        mbar_arrive_expect_tx(k_full(s), L::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < D / 64; ++b)
          tma_load_4d(k_smem + s * L::TILE_BYTES + b * L::BOX_BYTES, &tm_k, k_full(s), b * 64,
                      j * BLOCK_N, h / p.kv_group, z);
        issued |= 1u << s;
        parity = (parity & ~(1u << s)) | (ph << s);
        if (!mbar_wait(v_empty(s), ph ^ 1u, ctx, 2)) { ok = false; break; }
        mbar_arrive_expect_tx(v_full(s), L::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < D / 64; ++b)
          tma_load_4d(v_smem + s * L::TILE_BYTES + b * L::BOX_BYTES, &tm_v, v_full(s), b * 64,
                      j * BLOCK_N, h / p.kv_group, z);
        issued |= 4u << s;
        parity = (parity & ~(4u << s)) | (ph << (2 + s));
      }
      if (!ok) {
        // copies in flight still target this CTA's shared memory
        if (issued & 16u) mbar_wait_drain(q_full, 0);
        for (int s = 0; s < KV_STAGES; ++s) {
          if (issued & (1u << s)) mbar_wait_drain(k_full(s), (parity >> s) & 1u);
          if (issued & (4u << s)) mbar_wait_drain(v_full(s), (parity >> (2 + s)) & 1u);
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0, ctx, 3);
      auto issue_qk = [&](int j) {
        const int s = j % KV_STAGES;
        const uint32_t d_tmem = tmem_base + (uint32_t)(s * S_COLS);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk / 4) * L::BOX_BYTES + (kk % 4) * 32);
          const uint64_t a_desc = make_smem_desc_sw128(q_smem + off, 16, 1024);
          const uint64_t b_desc =
              make_smem_desc_sw128(k_smem + s * L::TILE_BYTES + off, 16, 1024);
          mma_f16_ss(d_tmem, a_desc, b_desc, p.idesc_qk, kk > 0 ? 1u : 0u);
        }
        tc_commit(s_full(s));
        tc_commit(k_empty(s));
      };
      if (ok && nblocks > 0) {
        ok = mbar_wait(k_full(0), 0, ctx, 4);
        if (ok) {
          tc_fence_after_sync();
          issue_qk(0);
        }
      }
      for (int j = 0; ok && j < nblocks; ++j) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (uint32_t)(j / KV_STAGES) & 1u;
        if (j + 1 < nblocks) {
          const int s1 = (j + 1) % KV_STAGES;
          const uint32_t ph1 = (uint32_t)((j + 1) / KV_STAGES) & 1u;
          if (!mbar_wait(k_full(s1), ph1, ctx, 5)) { ok = false; break; }
          // S buffer s1 still holds S(j-1) / P(j-1) until PV(j-1) has completed
          if (j >= 1 && !mbar_wait(o_full, (uint32_t)(j - 1) & 1u, ctx, 6)) { ok = false; break; }
          tc_fence_after_sync();
          issue_qk(j + 1);
        }
        if (!mbar_wait(v_full(s), ph, ctx, 7)) { ok = false; break; }
        if (!mbar_wait(p_full, (uint32_t)j & 1u, ctx, 8)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t o_tmem = tmem_base + O_COL0;
#pragma unroll
        for (int kk = 0; kk < BLOCK_N / 16; ++kk) {
          // V tile: D/64 chunks of 64 columns (pitch = one box), 16 key rows per step
          const uint64_t b_desc = make_smem_desc_sw128(
              v_smem + s * L::TILE_BYTES + kk * 2048, L::BOX_BYTES, 1024);
          if (P_TMEM) {
            const uint32_t a_tmem = tmem_base + (uint32_t)(s * S_COLS + kk * 8);
            mma_f16_ts(o_tmem, a_tmem, b_desc, p.idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          } else {
            const uint32_t off = (uint32_t)((kk / 4) * L::BOX_BYTES + (kk % 4) * 32);
            const uint64_t a_desc = make_smem_desc_sw128(p_smem + off, 16, 1024);
            mma_f16_ss(o_tmem, a_desc, b_desc, p.idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          }
        }
        tc_commit(o_full);
        tc_commit(v_empty(s));
      }
      tc_commit(drain_bar);
      mbar_wait_drain(drain_bar, 0);
    }
  } else {
    // -------------------------------------------------------------- softmax + epilogue
    const int row = m0 + warp * 32 + lane;  // query row of this thread
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY;  // running max (log2 domain, scaled) used for exp2
    float l = 0.f;
    bool ok = true;
    // warp-uniform wait: the vote keeps the warp converged for the .sync.aligned
    // tensor-memory accesses that follow
    auto wait_all = [&](uint32_t bar, uint32_t parity, uint32_t site) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, site)) != 0;
    };
    for (int j = 0; ok && j < nblocks; ++j) {
      const int s = j % KV_STAGES;
      if (!wait_all(s_full(s), (uint32_t)(j / KV_STAGES) & 1u, 9)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t s_tmem = tmem_base + lane_addr + (uint32_t)(s * S_COLS);
      float x[BLOCK_N];
#pragma unroll
      for (int c = 0; c < BLOCK_N / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(s_tmem + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) x[c * 32 + i] = __uint_as_float(r[i]);
      }
      const int col0 = j * BLOCK_N;
      const bool diag = p.causal && (col0 + BLOCK_N - 1 > m0 + (p.NK - p.N));
      const bool ragged = col0 + BLOCK_N > p.NK;
      if (diag || ragged) {
        const int limit = min(p.causal ? row + (p.NK - p.N) : p.NK - 1, p.NK - 1);  // last kept column
#pragma unroll
        for (int i = 0; i < BLOCK_N; ++i)
          if (col0 + i > limit) x[i] = -INFINITY;
      }
      float mx = x[0];
#pragma unroll
      for (int i = 1; i < BLOCK_N; ++i) mx = fmaxf(mx, x[i]);
      mx *= p.scale_log2;
      // lazy rescale of the accumulator
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
      if (j > 0 && (!P_TMEM || __any_sync(0xffffffffu, raise))) {
        // PV(j-1) must have landed in O (and finished reading P from shared memory)
        if (!wait_all(o_full, (uint32_t)(j - 1) & 1u, 10)) { ok = false; break; }
        tc_fence_after_sync();
      }
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        const uint32_t o_tmem = tmem_base + lane_addr + O_COL0;
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
      const float neg_m = -m_used;
      float sum = 0.f;
      uint32_t packed[BLOCK_N / 2];
#pragma unroll
      for (int i = 0; i < BLOCK_N; i += 2) {
        const float e0 = ex2(fmaf(x[i], p.scale_log2, neg_m));
        const float e1 = ex2(fmaf(x[i + 1], p.scale_log2, neg_m));
        sum += e0 + e1;
        packed[i / 2] = pack2<T>(e0, e1);
      }
      l += sum;
      if (P_TMEM) {
#pragma unroll
        for (int c = 0; c < BLOCK_N / 64; ++c) {
          uint32_t r[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = packed[c * 32 + i];
          tmem_st_32x32b_x32(s_tmem + c * 32, r);
        }
        tmem_st_wait();
        tc_fence_before_sync();
      } else {
        // row-major 128-byte spans, 16-byte units XOR-swizzled by (row % 8)
        const int r_in = warp * 32 + lane;
#pragma unroll
        for (int u = 0; u < BLOCK_N / 8; ++u) {
          const int box = u / 8, unit = u % 8;
          const uint32_t addr = p_smem + box * L::BOX_BYTES + r_in * 128 +
                                (uint32_t)((unit ^ (r_in & 7)) * 16);
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                       "r"(packed[u * 4]), "r"(packed[u * 4 + 1]), "r"(packed[u * 4 + 2]),
                       "r"(packed[u * 4 + 3])
                       : "memory");
        }
        fence_proxy_async_smem();
      }
      mbar_arrive(p_full);
    }
    if (ok && nblocks > 0) ok = wait_all(o_full, (uint32_t)(nblocks - 1) & 1u, 11);
    if (ok && nblocks > 0) {
      tc_fence_after_sync();
      const float inv_l = 1.0f / l;
      const uint32_t o_tmem = tmem_base + lane_addr + O_COL0;
      T *orow = reinterpret_cast<T *>(p.o) + z * p.oz + h * p.oh + (int64_t)row * p.om;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(o_tmem + c * 32, r);
        tmem_ld_wait();
        if (row < p.N) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 out;
            out.x = pack2<T>(__uint_as_float(r[q * 8 + 0]) * inv_l, __uint_as_float(r[q * 8 + 1]) * inv_l);
            out.y = pack2<T>(__uint_as_float(r[q * 8 + 2]) * inv_l, __uint_as_float(r[q * 8 + 3]) * inv_l);
            out.z = pack2<T>(__uint_as_float(r[q * 8 + 4]) * inv_l, __uint_as_float(r[q * 8 + 5]) * inv_l);
            out.w = pack2<T>(__uint_as_float(r[q * 8 + 6]) * inv_l, __uint_as_float(r[q * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4 *>(orow + c * 32 + q * 8) = out;
          }
        }
      }
      if (p.lse != nullptr && row < p.N)
        p.lse[z * p.lse_z + h * p.lse_h + row] = m_used * 0.6931471805599453f + logf(l);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <typename T, int D, bool P_TMEM>
static int launch_tc(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                     const Params &p, int zh, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  auto kernel = attn_fwd_tcgen05_kernel<T, D, P_TMEM>;
  constexpr int smem = Smem<D>::bytes(P_TMEM);
  if (dev < 64 && !configured[dev]) {
    B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  dim3 grid((p.N + BLOCK_M - 1) / BLOCK_M, zh);
  kernel<<<grid, THREADS, smem, stream>>>(tq, tk, tv, p);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

static int encode_qkv(CUtensorMap *tm, const b200_tensor *t) {
  const size_t es = dtype_size(t->dtype);
  const uint64_t dims[4] = {(uint64_t)t->shape[3], (uint64_t)t->shape[2], (uint64_t)t->shape[1],
                            (uint64_t)t->shape[0]};
  const uint64_t strides[4] = {es, (uint64_t)t->stride[2] * es, (uint64_t)t->stride[1] * es,
                               (uint64_t)t->stride[0] * es};
  const uint32_t box[4] = {64, BLOCK_N, 1, 1};
  return encode_tensor_map(tm, t->dtype, t->data, 4, dims, strides, box);
}

// Where P (the 16-bit softmax numerators) is handed to the second MMA:
// B200OPS_ATTN_P=smem selects shared memory, anything else tensor memory.
static bool p_in_tmem() {
  const char *e = getenv("B200OPS_ATTN_P");
  return !(e != nullptr && e[0] == 's');
}

}  // namespace attn
}  // namespace b200

static int attn_fwd_impl(const b200_tensor *q, const b200_tensor *k, const b200_tensor *v,
                         b200_tensor *o, b200_tensor *lse, float scale, int causal,
                         const b200::attn::SimtModes &modes, void *stream) {
  using namespace b200;
  using namespace b200::attn;
  int st;
  const bool plain = modes.softcap == 0.f && modes.alibi == nullptr && !modes.local &&
                     modes.page_table == nullptr;
  if ((st = check_tensor(q, "q", 4)) || (st = check_tensor(k, "k", 4)) ||
      (st = check_tensor(v, "v", 4)) || (st = check_tensor(o, "o", 4)))
    return st;
  if (lse != nullptr && (st = check_tensor(lse, "lse", 3))) return st;
  B200_REQUIRE(is_float_io(q->dtype), "q: dtype %u is not f16/bf16/f32", q->dtype);
  B200_REQUIRE(k->dtype == q->dtype && v->dtype == q->dtype && o->dtype == q->dtype,
               "q/k/v/o dtypes differ");
  const int64_t Z = q->shape[0], H = q->shape[1], N = q->shape[2], D = q->shape[3];
  B200_REQUIRE(o->shape[0] == Z && o->shape[1] == H && o->shape[2] == N && o->shape[3] == D,
               "o must have q's shape");
  // K / V may have fewer heads: query head h reads K / V head h / (H / H_KV), the grouping
  // of gqa_kernel (ops/suite/dev/gqa.py:27-32)
  const int64_t HKV = k->shape[1];
  // ... and another length: N_K keys per head (one sequence of flash_varlen_fwd_kernel,
  // ops/suite/dev/flash_varlen_fwd_kernel.py).  The causal mask is then aligned to the last
  // key: row i sees keys <= i + N_K - N (:138, window_size_right = 0)
  const int64_t NK = k->shape[2];
  for (const b200_tensor *t : {k, v}) {
    B200_REQUIRE(t->shape[0] == Z && t->shape[1] == HKV && t->shape[2] == NK && t->shape[3] == D,
                 "k and v must both be [Z, H_KV, N_K, D]");
  }
  // (with the other modes a row that sees no key is defined: zeros and lse = +inf)
  B200_REQUIRE(!plain || !causal || NK >= N,
               "the causal mask needs at least as many keys as query rows");
  B200_REQUIRE(NK < (1 << 24), "N_K out of range");
  B200_REQUIRE(HKV > 0 ? H % HKV == 0 : H == 0, "query heads %lld are not a multiple of K/V heads %lld",
               (long long)H, (long long)HKV);
  const int kv_group = HKV > 0 ? (int)(H / HKV) : 1;
  B200_REQUIRE(q->stride[3] == 1 && k->stride[3] == 1 && v->stride[3] == 1 && o->stride[3] == 1,
               "last-dim stride must be 1");
  B200_REQUIRE(D >= 1 && D <= 512, "head_dim %lld out of range", (long long)D);
  B200_REQUIRE(Z * H < 65536 && N < (1 << 24), "batch*heads or N_CTX out of range");
  B200_REQUIRE(scale == scale && scale > 0.f, "scale must be positive");
  if (lse != nullptr) {
    B200_REQUIRE(lse->dtype == B200_DTYPE_FLOAT32, "lse must be f32");
    B200_REQUIRE(lse->shape[0] == Z && lse->shape[1] == H && lse->shape[2] == N &&
                 lse->stride[2] == 1, "lse must be [Z,H,N] with unit last stride");
  }
  if (Z * H == 0 || N == 0) return B200_OK;
  B200_REQUIRE(NK > 0, "N_K must be positive: softmax over no keys is undefined");
  cudaStream_t s = (cudaStream_t)stream;

  const size_t es = dtype_size(q->dtype);
  auto tma_ok = [&](const b200_tensor *t) {
    return (uintptr_t)t->data % 16 == 0 && (t->stride[0] * es) % 16 == 0 &&
           (t->stride[1] * es) % 16 == 0 && (t->stride[2] * es) % 16 == 0;
  };
  const bool tensor_core = plain && q->dtype != B200_DTYPE_FLOAT32 && (D == 64 || D == 128) &&
                           tma_ok(q) && tma_ok(k) && tma_ok(v) &&
                           (uintptr_t)o->data % 16 == 0 && (o->stride[0] * es) % 16 == 0 &&
                           (o->stride[1] * es) % 16 == 0 && (o->stride[2] * es) % 16 == 0;
  if (!tensor_core) {
    B200_REQUIRE(NK <= kSimtMaxKeys, "N_K %lld exceeds the CUDA-core path's limit %d",
                 (long long)NK, kSimtMaxKeys);
    const size_t smem = (size_t)(NK + D) * sizeof(float);
    dim3 grid((unsigned)N, (unsigned)(Z * H));
#define B200_ATTN_SIMT(T)                                                                    \
  attn_simt_kernel<T><<<grid, kSimtThreads, smem, s>>>(                                      \
      (const T *)q->data, (const T *)k->data, (const T *)v->data, (T *)o->data,              \
      lse ? (float *)lse->data : nullptr, lse ? lse->stride[0] : 0, lse ? lse->stride[1] : 0,   \
      (int)H, kv_group, (int)N, (int)NK, (int)D, q->stride[0], q->stride[1],                    \
      q->stride[2], k->stride[0], k->stride[1], k->stride[2], v->stride[0], v->stride[1],    \
      v->stride[2], o->stride[0], o->stride[1], o->stride[2], scale, causal ? 1 : 0, modes)
    if (q->dtype == B200_DTYPE_FLOAT32) B200_ATTN_SIMT(float);
    else if (q->dtype == B200_DTYPE_FLOAT16) B200_ATTN_SIMT(__half);
    else B200_ATTN_SIMT(__nv_bfloat16);
#undef B200_ATTN_SIMT
    B200_CUDA_OK(cudaGetLastError());
    return B200_OK;
  }

  CUtensorMap tq, tk, tv;
  if ((st = encode_qkv(&tq, q)) || (st = encode_qkv(&tk, k)) || (st = encode_qkv(&tv, v)))
    return st;
  Params p;
  p.H = (int)H;
  p.N = (int)N;
  p.NK = (int)NK;
  p.lse_z = lse ? lse->stride[0] : 0;
  p.lse_h = lse ? lse->stride[1] : 0;
  p.kv_group = kv_group;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal ? 1 : 0;
  p.o = o->data;
  p.oz = o->stride[0];
  p.oh = o->stride[1];
  p.om = o->stride[2];
  p.lse = lse ? (float *)lse->data : nullptr;
  const int fmt = q->dtype == B200_DTYPE_BFLOAT16 ? 1 : 0;
  p.idesc_qk = sm100::make_idesc_f16(BLOCK_M, BLOCK_N, fmt, 0, 0);
  p.idesc_pv = sm100::make_idesc_f16(BLOCK_M, (int)D, fmt, 0, 1);
  p.status = device_status_word();
  if (p.status == nullptr) return fail(B200_RESOURCE, "no status word on this device");
  // B200OPS_ATTN_KERNEL=single selects the one-tile-per-CTA kernel; the default is the
  // persistent two-tile kernel
  const char *which = getenv("B200OPS_ATTN_KERNEL");
  if (!(which != nullptr && which[0] == 's')) {
    pair::Params pp;
    pp.H = p.H; pp.N = p.N; pp.NK = p.NK; pp.ZH = (int)(Z * H); pp.kv_group = kv_group;
    pp.lse_z = p.lse_z; pp.lse_h = p.lse_h;
    pp.scale_log2 = p.scale_log2; pp.causal = p.causal;
    pp.lse = p.lse;
    pp.idesc_qk = p.idesc_qk; pp.idesc_pv = p.idesc_pv; pp.status = p.status;
    CUtensorMap to;
    if ((st = encode_qkv(&to, o))) return st;
    if (q->dtype == B200_DTYPE_BFLOAT16)
      return D == 128 ? pair::launch<__nv_bfloat16, 128>(tq, tk, tv, to, pp, s)
                      : pair::launch<__nv_bfloat16, 64>(tq, tk, tv, to, pp, s);
    return D == 128 ? pair::launch<__half, 128>(tq, tk, tv, to, pp, s)
                    : pair::launch<__half, 64>(tq, tk, tv, to, pp, s);
  }
  const bool pt = p_in_tmem();
  const int zh = (int)(Z * H);
#define B200_ATTN_TC(T, DD)                                                   \
  (pt ? launch_tc<T, DD, true>(tq, tk, tv, p, zh, s) : launch_tc<T, DD, false>(tq, tk, tv, p, zh, s))
  if (q->dtype == B200_DTYPE_BFLOAT16)
    return D == 128 ? B200_ATTN_TC(__nv_bfloat16, 128) : B200_ATTN_TC(__nv_bfloat16, 64);
  return D == 128 ? B200_ATTN_TC(__half, 128) : B200_ATTN_TC(__half, 64);
#undef B200_ATTN_TC
}

extern "C" int b200_attn_fwd(const b200_tensor *q, const b200_tensor *k, const b200_tensor *v,
                             b200_tensor *o, b200_tensor *lse, float scale, int causal,
                             void *stream) {
  const b200::attn::SimtModes none{0.f, nullptr, 0, 0, 0, 0, nullptr, 0, 1, 0};
  return attn_fwd_impl(q, k, v, o, lse, scale, causal, none, stream);
}

extern "C" int b200_attn_fwd_modes(const b200_tensor *q, const b200_tensor *k,
                                   const b200_tensor *v, b200_tensor *o, b200_tensor *lse,
                                   float scale, int causal, float softcap,
                                   const b200_tensor *alibi_slopes, int window_left,
                                   int window_right, const b200_tensor *page_table,
                                   int block_size, int64_t page_stride, void *stream) {
  using namespace b200;
  attn::SimtModes modes{0.f, nullptr, 0, 0, 0, 0, nullptr, 0, 1, 0};
  B200_REQUIRE(softcap == softcap && softcap >= 0.f, "softcap must be >= 0 (0: off)");
  modes.softcap = softcap;
  if (alibi_slopes != nullptr) {
    int st;
    if (q == nullptr) return fail(B200_USAGE, "null argument");
    const int dims = alibi_slopes->ndim;
    if ((st = check_tensor(alibi_slopes, "alibi_slopes", dims == 2 ? 2 : 1))) return st;
    B200_REQUIRE(alibi_slopes->dtype == B200_DTYPE_FLOAT32, "alibi_slopes must be f32");
    const int64_t heads = q->shape[1];
    B200_REQUIRE(alibi_slopes->shape[dims - 1] == heads && alibi_slopes->stride[dims - 1] == 1 &&
                 (dims == 1 || alibi_slopes->shape[0] == q->shape[0]),
                 "alibi_slopes must be [H] or [Z, H] with unit last stride");
    modes.alibi = static_cast<const float *>(alibi_slopes->data);
    modes.alibi_z = dims == 2 ? alibi_slopes->stride[0] : 0;
  }
  if (window_left >= 0 || window_right >= 0) {
    B200_REQUIRE(window_left >= 0 && window_right >= 0,
                 "a local window needs both sides (negative on both: no window)");
    modes.local = 1;
    modes.window_left = window_left;
    modes.window_right = window_right;
  }
  if (page_table != nullptr) {
    int st;
    if ((st = check_tensor(page_table, "page_table", 2))) return st;
    if (q == nullptr || k == nullptr) return fail(B200_USAGE, "null argument");
    B200_REQUIRE(page_table->dtype == B200_DTYPE_INT32 && page_table->stride[1] == 1 &&
                 page_table->shape[0] == q->shape[0],
                 "page_table must be int32 [Z, pages] with unit last stride");
    B200_REQUIRE(block_size > 0 && page_stride > 0, "block_size and page_stride must be positive");
    B200_REQUIRE(page_table->shape[1] * (int64_t)block_size >= k->shape[2],
                 "the page table covers %lld keys, N_K is %lld",
                 (long long)(page_table->shape[1] * (int64_t)block_size), (long long)k->shape[2]);
    modes.page_table = static_cast<const int *>(page_table->data);
    modes.page_table_z = page_table->stride[0];
    modes.block_size = block_size;
    modes.page_stride = page_stride;
  }
  return attn_fwd_impl(q, k, v, o, lse, scale, causal, modes, stream);
}

