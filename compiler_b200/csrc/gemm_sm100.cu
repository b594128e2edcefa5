// C = act(A @ B + bias) for sm_100a: TMA-fed tcgen05.mma tiles with the
// accumulator in tensor memory and the epilogue fused behind it.
//
// Semantics follow matmul_kernel (ops/suite/perf/matmul.py:20-38) and
// linear_act_kernel (ops/suite/perf/triton_linear_activation.py:27-49):
// A [M,K] row-major, B [K,N] row-major, 16-bit operands, fp32 accumulation,
// bias add and activation in fp32, one rounding at the store.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 4   producer: TMA loads of A (128x64, K-major) and B (64x256, four
//            64-column boxes, N-major) into a 4-stage shared-memory ring
//   warp 5   one elected lane issues tcgen05.mma 128x256x16 into one of two
//            256-column TMEM accumulators and commits stage / tile barriers
//   warps 0-3 epilogue: tcgen05.ld the finished accumulator (one row per
//            thread), bias + activation, convert, 16-byte global stores
// so the epilogue of tile i overlaps the main loop of tile i+1.  Out-of-range
// rows / columns / K are zero-filled by TMA on load and predicated on store;
// no out-of-range address is ever formed.
#include "sm100.cuh"

#include <algorithm>
#include <map>
#include <mutex>

namespace b200 {

// ------------------------------------------------------------ tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_entry() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  });
  return fn;
}

int encode_tensor_map(CUtensorMap *out, uint32_t dtype, const void *base, int rank,
                      const uint64_t *dims, const uint64_t *strides_bytes,
                      const uint32_t *box) {
  EncodeTiledFn fn = encode_tiled_entry();
  if (fn == nullptr) return fail(B200_RESOURCE, "cuTensorMapEncodeTiled is not available");
  CUtensorMapDataType dt;
  switch (dtype) {
    case B200_DTYPE_BFLOAT16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case B200_DTYPE_FLOAT16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case B200_DTYPE_FLOAT32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: return fail(B200_UNSUPPORTED, "no tensor map for dtype %u", dtype);
  }
  cuuint64_t gdims[5], gstrides[5];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i];
  }
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void *>(base), gdims, gstrides, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B200_REJECTED, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return B200_OK;
}

namespace gemm {

using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 256;  // accumulator columns per tile (two 128-column halves when DUAL)
constexpr int BK = 64;   // 64 16-bit elements = one 128-byte swizzle span
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;                     // stages of a full-width (256-column) ring
constexpr int MAX_STAGES = 8;                 // a narrower B operand leaves room for more
constexpr int A_STAGE_BYTES = BM * BK * 2;    // 16 KiB
constexpr int B_BOX_BYTES = BK * 64 * 2;      // one 64(K) x 64(N) box: 8 KiB
constexpr int B_STAGE_BYTES = 4 * B_BOX_BYTES;  // 32 KiB
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 192;

constexpr int kActLogSoftmax = 100;  // internal epilogue code: row log-softmax (N <= 256)
constexpr int kActGroupNormMin = 101;  // internal: group norm over column groups, row minimum

// Group normalisation over groups of `group` consecutive columns followed by the minimum of
// each row, merged into mins[] with an atomic minimum (the epilogue of
// fused_gemm_gn_min_kernel, ops/suite/dev/fused_gemm_gn_min_kernel.py:45-59).
struct GroupNormMin {
  const void *gamma, *beta;  // [N], kind = dtype code
  int kind;
  int group;                 // 8, 16, 32 or 64 columns
  float eps;
  float *mins;               // [M], holds the running minimum (start it at +inf)
};

struct Params {
  int M, N, K;
  int act;
  int bias_kind;  // 0 none, B200_DTYPE_* otherwise
  const void *bias;
  void *c;
  int64_t ldc;
  uint32_t idesc;
  int vector_store;  // rows of C are 16-byte aligned and N % 8 == 0 (N % 4 for f32)
  unsigned int *status;
  uint32_t b_lbo, b_sbo;  // B-operand descriptor pitches (bytes)
  uint32_t b_kstep;       // descriptor advance per UMMA_K step, in 16-byte units
  int b_kmajor;           // B is given as [N, K] (rows of K): one 64(K) x 256(N) box per stage
  const float *row_scale; // optional [M] factors applied to the accumulator rows before the bias
  GroupNormMin gn;        // used with kActGroupNormMin
  // Row scatter for the tensor-parallel MLP: when scatter_rows > 0 the row block
  // [k * scatter_rows, (k+1) * scatter_rows) of C is not written to `c` but to slot
  // `scatter_slot` of c_rank[k] -- the memory of the rank that owns those rows (a peer
  // GPU's buffer mapped into this process, or this GPU's own for k == this rank).
  void *c_rank[8];
  int scatter_rows;
  int scatter_slot;
  int group_m;  // m-blocks per raster group
  // One-CTA kernel: the ring holds `stages` stages of A_STAGE_BYTES + b_stage_bytes.  A single
  // column block narrower than the tile loads only the B columns that exist (b_boxes boxes of
  // 64 columns for B as [K,N]; one box of b_stage_bytes / 128 rows for B as [N,K]), so a
  // product that only streams A keeps eight stages of A in flight instead of four.
  int stages;
  int b_stage_bytes;
  int b_boxes;
  // CTA-pair kernel, split of the last partial wave along K.  When the tiles do not fill a
  // whole number of waves of SM pairs, the last `tail_tiles` tiles are not dealt out whole:
  // each is cut into `tail_slices` (2 or 4) ranges of k-blocks, one range per pair, so the
  // last wave takes 1 / tail_slices of a tile's time.  The slices then share the tile's columns:
  // every slice stores the raw fp32 accumulator columns that are not its own to `tail_ws`,
  // counts up a flag in `tail_flags`, waits (bounded) for the others, adds their partials of its
  // own columns into its accumulator in tensor memory and runs the epilogue on those columns.
  // Every column is summed by one slice in a fixed order: repeated launches give the same bits.
  int tail_tiles;    // 0: no split
  int tail_slices;
  float *tail_ws;    // [tail_tiles][tail_slices][2 CTAs][256 columns][128 rows]
  unsigned int *tail_flags;  // [tail_tiles][2 CTAs][4 warps][arrived, done], zero between launches
  // CTA-pair kernel, progress per raster group (a block of group_m x 128 rows of C): when
  // `progress` is set every epilogue warp, after the stores of its part of a tile (fenced at
  // system scope), adds one to progress[group of the tile].  A kernel launched behind this one
  // as its programmatic dependent -- the all-reduce of the tensor-parallel MLP -- starts while
  // this one runs and takes a block of rows as soon as the block's count is complete, instead
  // of waiting for the last tile of the product.  The kernel also releases its dependents
  // (griddepcontrol.launch_dependents) as soon as its CTAs are set up.
  unsigned int *progress;
};

// What a launch with progress counters tells its caller (host memory): the count each block
// of rows reaches when all its tiles are stored.
struct Progress {
  unsigned int *counters;   // device, one per block of rows, zero before the launch
  int64_t rows_per_block;   // a multiple of 256
  unsigned int *targets;    // host, [max_blocks]
  int max_blocks;
  int *blocks;              // host: number of blocks
};

__device__ __forceinline__ float gelu_tanh_fast(float z) {
  const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * z * (1.0f + t);
}
__device__ __forceinline__ float gelu_tanh_exact(float z) {
  const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  return 0.5f * z * (1.0f + tanhf(u));
}
__device__ __forceinline__ float gelu_erf(float z) {
  return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
}

template <typename OutT, int ACT> __device__ __forceinline__ float activate(float z) {
  if constexpr (ACT == B200_ACT_GELU_ERF) return gelu_erf(z);
  if constexpr (ACT == B200_ACT_GELU_TANH)
    return sizeof(OutT) == 2 ? gelu_tanh_fast(z) : gelu_tanh_exact(z);
  if constexpr (ACT == B200_ACT_LEAKY_RELU) return z >= 0.f ? z : 0.01f * z;
  return z;
}
__device__ __forceinline__ float silu(float z) { return z / (1.0f + __expf(-z)); }

__device__ __forceinline__ float load_bias(const void *bias, int kind, int col) {
  if (kind == B200_DTYPE_FLOAT32) return ((const float *)bias)[col];
  if (kind == B200_DTYPE_BFLOAT16) return __bfloat162float(((const __nv_bfloat16 *)bias)[col]);
  return __half2float(((const __half *)bias)[col]);
}

// bias values of 32 consecutive columns starting at col0 (same for every thread
// of the warp: the loads are broadcasts served by L1)
__device__ __forceinline__ void load_bias_chunk(const void *bias, int kind, int col0, int n,
                                                float (&b)[32]) {
  if (kind == 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) b[j] = 0.f;
    return;
  }
  if (col0 + 32 <= n && ((uintptr_t)bias & 15) == 0) {
    if (kind == B200_DTYPE_FLOAT32) {
      const float4 *src = reinterpret_cast<const float4 *>((const float *)bias + col0);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 t = __ldg(src + q);
        b[4 * q] = t.x; b[4 * q + 1] = t.y; b[4 * q + 2] = t.z; b[4 * q + 3] = t.w;
      }
    } else {
      const uint4 *src = reinterpret_cast<const uint4 *>((const uint16_t *)bias + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 t = __ldg(src + q);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (kind == B200_DTYPE_BFLOAT16) {
            b[8 * q + 2 * i] = __uint_as_float(w[i] << 16);
            b[8 * q + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
          } else {
            const __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            b[8 * q + 2 * i] = __low2float(h);
            b[8 * q + 2 * i + 1] = __high2float(h);
          }
        }
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) b[j] = col0 + j < n ? load_bias(bias, kind, col0 + j) : 0.f;
  }
}

// convert and store 32 consecutive columns of one row
template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT *crow, int col0, int n, bool vector_ok,
                                            const float (&v)[32]) {
  if (vector_ok && col0 + 32 <= n) {
    constexpr int PER = 16 / (int)sizeof(OutT);
#pragma unroll
    for (int q = 0; q < 32 / PER; ++q) {
      vec16<OutT> o;
#pragma unroll
      for (int j = 0; j < PER; ++j) o.e[j] = io<OutT>::store(v[q * PER + j]);
      *reinterpret_cast<uint4 *>(crow + col0 + q * PER) = o.raw;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < n) crow[col0 + j] = io<OutT>::store(v[j]);
  }
}

// bias + activation + store of one 32-column chunk held in registers
template <typename OutT, int ACT>
__device__ __forceinline__ void finish_chunk(const uint32_t (&r)[32], const Params &p, OutT *crow,
                                             int col0, bool row_ok, float row_mul) {
  if (col0 >= p.N) return;  // warp-uniform
  float b[32], v[32];
  load_bias_chunk(p.bias, p.bias_kind, col0, p.N, b);
#pragma unroll
  for (int j = 0; j < 32; ++j)
    v[j] = activate<OutT, ACT>(fmaf(__uint_as_float(r[j]), row_mul, b[j]));
  if (row_ok) store_chunk<OutT>(crow, col0, p.N, p.vector_store != 0, v);
}

// Epilogue of one 128 x 256 accumulator for one warp (32 rows): the TMEM load of
// chunk c+1 is in flight while chunk c is converted and stored.
// Chunks [c0, c1) of 32 columns (an even count): the whole tile, or one slice's share of a
// tile of the split last wave.
template <typename OutT, int ACT>
__device__ __forceinline__ void epilogue_tile(uint32_t t_row, const Params &p, OutT *crow,
                                              int col_base, bool row_ok, float row_mul,
                                              int c0 = 0, int c1 = BN / 32) {
  uint32_t ra[32], rb[32];
  tmem_ld_32x32b_x32(t_row + (uint32_t)(c0 * 32), ra);
#pragma unroll 1
  for (int chunk = c0; chunk < c1; chunk += 2) {
    tmem_ld_wait();
    tmem_ld_32x32b_x32(t_row + (uint32_t)((chunk + 1) * 32), rb);
    finish_chunk<OutT, ACT>(ra, p, crow, col_base + chunk * 32, row_ok, row_mul);
    tmem_ld_wait();
    if (chunk + 2 < c1) tmem_ld_32x32b_x32(t_row + (uint32_t)((chunk + 2) * 32), ra);
    finish_chunk<OutT, ACT>(rb, p, crow, col_base + (chunk + 1) * 32, row_ok, row_mul);
  }
}

// Row log-softmax over the N <= 256 columns of the one column block (the epilogue of
// log_softmax_linear_kernel, ops/suite/perf/log_softmax_linear.py:32-35): the thread that
// owns a row reads its accumulator three times from tensor memory -- max, sum of
// exponentials, y = z - max - log(sum) -- instead of keeping 256 values in registers.
template <typename OutT>
__device__ __forceinline__ void epilogue_tile_log_softmax(uint32_t t_row, const Params &p,
                                                          OutT *crow, bool row_ok) {
  const int chunks = (p.N + 31) / 32;
  float mx = -INFINITY;
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + (uint32_t)(c * 32), r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (c * 32 + j < p.N) mx = fmaxf(mx, __uint_as_float(r[j]));
  }
  float sum = 0.f;
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + (uint32_t)(c * 32), r);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (c * 32 + j < p.N) sum += expf(__uint_as_float(r[j]) - mx);
  }
  const float shift = mx + logf(sum);
  for (int c = 0; c < chunks; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + (uint32_t)(c * 32), r);
    tmem_ld_wait();
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) - shift;
    if (row_ok) store_chunk<OutT>(crow, c * 32, p.N, p.vector_store != 0, v);
  }
}

// minimum of floats through integer atomics: non-negative values order like ints, negative
// ones in reverse like unsigned ints
__device__ __forceinline__ void atomic_min_float(float *addr, float v) {
  if (v >= 0.f) atomicMin(reinterpret_cast<int *>(addr), __float_as_int(v));
  else atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

// group norm + row minimum over W = max(GS, 32) columns held in registers
template <int GS, int W>
__device__ __forceinline__ float gn_min_block(const float (&z)[W], const Params &p, int col0) {
  float lowest = INFINITY;
#pragma unroll
  for (int g = 0; g < W / GS; ++g) {
    float mean = 0.f;
#pragma unroll
    for (int j = 0; j < GS; ++j) mean += z[g * GS + j];
    mean *= 1.0f / GS;
    float var = 0.f;
#pragma unroll
    for (int j = 0; j < GS; ++j) {
      const float d = z[g * GS + j] - mean;
      var = fmaf(d, d, var);
    }
    const float rstd = rsqrtf(var * (1.0f / GS) + p.gn.eps);
#pragma unroll
    for (int j = 0; j < GS; ++j) {
      const int col = col0 + g * GS + j;
      const float out = (z[g * GS + j] - mean) * rstd * load_bias(p.gn.gamma, p.gn.kind, col) +
                        load_bias(p.gn.beta, p.gn.kind, col);
      lowest = fminf(lowest, out);
    }
  }
  return lowest;
}

// Epilogue of fused_gemm_gn_min_kernel: bias, group norm over groups of GS columns (a group
// lies inside one thread's row, so the statistics are plain per-thread arithmetic), row
// minimum, one atomic minimum per row and column block.  N % GS == 0.
template <int GS>
__device__ __forceinline__ void epilogue_tile_gn_min(uint32_t t_row, const Params &p, int row,
                                                     int col_base, bool row_ok) {
  constexpr int W = GS > 32 ? GS : 32;
  float lowest = INFINITY;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += W) {
    if (col_base + c0 >= p.N) break;  // warp-uniform
    float z[W];
#pragma unroll
    for (int part = 0; part < W / 32; ++part) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_row + (uint32_t)(c0 + part * 32), r);
      tmem_ld_wait();
      float b[32];
      load_bias_chunk(p.bias, p.bias_kind, col_base + c0 + part * 32, p.N, b);
#pragma unroll
      for (int j = 0; j < 32; ++j) z[part * 32 + j] = __uint_as_float(r[j]) + b[j];
    }
    lowest = fminf(lowest, gn_min_block<GS, W>(z, p, col_base + c0));
  }
  if (row_ok) atomic_min_float(p.gn.mins + row, lowest);
}

// DUAL: columns [0,128) hold x Wg, [128,256) hold x Wu; out = silu(g) * u
template <typename OutT>
__device__ __forceinline__ void epilogue_tile_dual(uint32_t t_row, const Params &p, OutT *crow,
                                                   int col_base, bool row_ok, int c0 = 0,
                                                   int c1 = BN / 64) {
#pragma unroll 1
  for (int chunk = c0; chunk < c1; ++chunk) {
    const int col0 = col_base + chunk * 32;
    uint32_t r[32], r2[32];
    tmem_ld_32x32b_x32(t_row + (uint32_t)(chunk * 32), r);
    tmem_ld_32x32b_x32(t_row + (uint32_t)(BN / 2 + chunk * 32), r2);
    tmem_ld_wait();
    if (col0 >= p.N) continue;  // warp-uniform
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = silu(__uint_as_float(r[j])) * __uint_as_float(r2[j]);
    if (row_ok) store_chunk<OutT>(crow, col0, p.N, p.vector_store != 0, v);
  }
}

// Epilogue of one accumulator for one warp: one straight-line body per activation, chosen per
// tile and not per element.
// [c0, c1): the 32-column chunks of the OUTPUT tile to finish (8 per tile, 4 with two B
// operands); anything but the whole tile only for the plain and activation epilogues.
template <typename OutT, bool DUAL>
__device__ __forceinline__ void run_epilogue(uint32_t t_row, const Params &p, OutT *crow, int row,
                                             int col_base, bool row_ok, float row_mul, int c0 = 0,
                                             int c1 = DUAL ? BN / 64 : BN / 32) {
  if constexpr (DUAL) {
    epilogue_tile_dual<OutT>(t_row, p, crow, col_base, row_ok, c0, c1);
  } else {
    switch (p.act) {
      case kActLogSoftmax:
        epilogue_tile_log_softmax<OutT>(t_row, p, crow, row_ok);
        break;
      case kActGroupNormMin:
        if (p.gn.group == 8) epilogue_tile_gn_min<8>(t_row, p, row, col_base, row_ok);
        else if (p.gn.group == 16) epilogue_tile_gn_min<16>(t_row, p, row, col_base, row_ok);
        else if (p.gn.group == 32) epilogue_tile_gn_min<32>(t_row, p, row, col_base, row_ok);
        else epilogue_tile_gn_min<64>(t_row, p, row, col_base, row_ok);
        break;
      case B200_ACT_GELU_TANH:
        epilogue_tile<OutT, B200_ACT_GELU_TANH>(t_row, p, crow, col_base, row_ok, row_mul, c0, c1);
        break;
      case B200_ACT_GELU_ERF:
        epilogue_tile<OutT, B200_ACT_GELU_ERF>(t_row, p, crow, col_base, row_ok, row_mul, c0, c1);
        break;
      case B200_ACT_LEAKY_RELU:
        epilogue_tile<OutT, B200_ACT_LEAKY_RELU>(t_row, p, crow, col_base, row_ok, row_mul, c0, c1);
        break;
      default:
        epilogue_tile<OutT, B200_ACT_NONE>(t_row, p, crow, col_base, row_ok, row_mul, c0, c1);
    }
  }
}

// tile index -> block coordinates, grouped so that concurrently running CTAs
// share A row-blocks and B column-blocks in L2
__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int group_m,
                                            int &mb, int &nb) {
  const int per_group = group_m * n_blocks;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int rows = min(group_m, m_blocks - first_m);
  const int in_group = tile - group * per_group;
  mb = first_m + in_group % rows;
  nb = in_group / rows;
}

template <typename OutT, bool DUAL>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a,
                    const __grid_constant__ CUtensorMap tm_b,
                    const __grid_constant__ CUtensorMap tm_b2, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int stages = p.stages;
  const uint32_t b_stage_bytes = (uint32_t)p.b_stage_bytes;
  const uint32_t ring_bytes = (uint32_t)stages * (A_STAGE_BYTES + b_stage_bytes);
  const uint32_t a_smem = smem_base;
  const uint32_t b_smem = smem_base + (uint32_t)stages * A_STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_gen + ring_bytes);
  // barrier slots: full[MAX_STAGES], empty[MAX_STAGES], acc_full[2], acc_empty[2], drain
  const uint32_t bar0 = smem_base + ring_bytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (MAX_STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * MAX_STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * MAX_STAGES + 2 + a); };
  const uint32_t drain_bar = bar0 + 8u * (2 * MAX_STAGES + 4);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * MAX_STAGES + 5);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx ctx{abort_flag, p.status};

  // output tile width in columns of C
  constexpr int TILE_N = DUAL ? BN / 2 : BN;
  const int m_blocks = (p.M + BM - 1) / BM;
  const int n_blocks = (p.N + TILE_N - 1) / TILE_N;
  const int num_tiles = m_blocks * n_blocks;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0u;
    mbar_init_fence();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    if (DUAL) tma_prefetch_desc(&tm_b2);
  }
  if (warp == 5) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, issued_parity = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, ctx, 1)) { ok = false; break; }
          mbar_arrive_expect_tx(full_bar(stage), A_STAGE_BYTES + b_stage_bytes);
          tma_load_2d(a_smem + stage * A_STAGE_BYTES, &tm_a, full_bar(stage), kb * BK, mb * BM);
          const uint32_t bdst = b_smem + (uint32_t)stage * b_stage_bytes;
          if (DUAL) {
            const int n0 = nb * TILE_N;
            tma_load_2d(bdst, &tm_b, full_bar(stage), n0, kb * BK);
            tma_load_2d(bdst + B_BOX_BYTES, &tm_b, full_bar(stage), n0 + 64, kb * BK);
            tma_load_2d(bdst + 2 * B_BOX_BYTES, &tm_b2, full_bar(stage), n0, kb * BK);
            tma_load_2d(bdst + 3 * B_BOX_BYTES, &tm_b2, full_bar(stage), n0 + 64, kb * BK);
          } else if (p.b_kmajor) {
            // B rows are rows of K: one box of 64 (K) x up to 256 (N), laid out like the A tile
            tma_load_2d(bdst, &tm_b, full_bar(stage), kb * BK, nb * TILE_N);
          } else {
            const int n0 = nb * TILE_N;
            for (int j = 0; j < p.b_boxes; ++j)
              tma_load_2d(bdst + j * B_BOX_BYTES, &tm_b, full_bar(stage), n0 + 64 * j, kb * BK);
          }
          issued_mask |= 1u << stage;
          issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // copies already issued still target this CTA's shared memory: wait for
        // them (bounded) before the CTA is allowed to exit
        for (int s = 0; s < stages; ++s)
          if (issued_mask & (1u << s)) mbar_wait_drain(full_bar(s), (issued_parity >> s) & 1u);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop (uniform control flow keeps the descriptor
    // arithmetic cheap); one elected lane issues the MMAs and commits.
    const bool leader = elect_one();
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    auto wait_all = [&](uint32_t bar, uint32_t parity, uint32_t site) {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, site)) != 0;
    };
    // descriptor halves: only the low word moves, by constants
    const uint32_t a_lo0 = desc_lo_sw128(a_smem, 16);
    const uint32_t b_lo0 = desc_lo_sw128(b_smem, p.b_lbo);
    constexpr uint32_t a_hi = desc_hi_sw128(1024);
    const uint32_t b_hi = desc_hi_sw128(p.b_sbo);
    const uint32_t b_kstep = p.b_kstep;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      if (!wait_all(acc_empty_bar(acc), acc_phase ^ 1u, 2)) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!wait_all(full_bar(stage), phase, 3)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t a_lo = a_lo0 + (uint32_t)stage * (A_STAGE_BYTES >> 4);
        const uint32_t b_lo = b_lo0 + (uint32_t)stage * (b_stage_bytes >> 4);
        if (leader) {
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // A: +32 bytes along K inside the swizzle span; B: +16 K-rows of 128 bytes when
            // its rows are rows of N, +32 bytes like A when they are rows of K
            mma_f16_ss(d_tmem, a_lo + (uint32_t)(k * ((UMMA_K * 2) >> 4)), a_hi,
                       b_lo + (uint32_t)k * b_kstep, b_hi, p.idesc,
                       (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));  // stage reusable once these MMAs retire
        }
        if (++stage == stages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (leader) tc_commit(acc_full_bar(acc));  // accumulator complete
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    // every MMA issued above must retire before shared / tensor memory go away
    if (leader) {
      tc_commit(drain_bar);
      mbar_wait_drain(drain_bar, 0);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    OutT *c = reinterpret_cast<OutT *>(p.c);
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, m_blocks, n_blocks, p.group_m, mb, nb);
      // the vote keeps the warp converged for the .sync.aligned TMEM loads below
      if (!__all_sync(0xffffffffu, mbar_wait(acc_full_bar(acc), acc_phase, ctx, 4))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row = mb * BM + warp * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * BN);
      OutT *crow = c + (int64_t)row * p.ldc;
      if (p.scatter_rows > 0) {
        // a tile never straddles two owners: scatter_rows is a multiple of the tile height
        const int owner = (mb * BM) / p.scatter_rows;
        const int local = row - owner * p.scatter_rows;
        crow = reinterpret_cast<OutT *>(p.c_rank[owner]) +
               ((int64_t)p.scatter_slot * p.scatter_rows + local) * p.ldc;
      }
      const int col_base = nb * TILE_N;
      const float row_mul = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f;
      run_epilogue<OutT, DUAL>(t_row, p, crow, row, col_base, row_ok, row_mul);
      // this warp has drained its quarter of the accumulator
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------ CTA-pair kernel
// The same persistent pipeline for a cluster of two CTAs that share one 256 x 256 tile of C:
// each CTA loads its 128 rows of A and its 128 of the 256 columns of B, the even CTA issues
// tcgen05.mma.cta_group::2 (M = 256), and each CTA's tensor memory receives the 256 columns of
// its own 128 rows.  Per tile and SM the operand bytes read from shared memory and brought in
// from L2 drop by a third against the one-CTA kernel (B is not duplicated in the two SMs).
// Barriers: full[s] lives in the even CTA and counts the bytes of both CTAs' copies; empty[s]
// and acc_full[a] exist in both CTAs and get one commit each; acc_empty[a] lives in the even
// CTA and takes the arrivals of the eight epilogue warps of the pair.
// One unit of work of a CTA pair: a tile and the k-blocks [kb0, kb1) of it.
struct PairWork {
  int tile;
  int kb0, kb1;
  int slice;   // 0: owns the tile (runs its epilogue)
  int slices;  // 1: the whole tile
  int tail;    // index among the split tiles
};

// The it-th unit of the pair that starts at tile `first` and strides by `step`: whole tiles
// while they last, then at most one slice of a split tile.
template <bool TAIL>
__device__ __forceinline__ bool pair_work(const Params &p, int it, int first, int step,
                                          int num_tiles, int num_kb, PairWork &w) {
  if constexpr (!TAIL) {
    w.tile = first + it * step;
    w.kb0 = 0; w.kb1 = num_kb; w.slice = 0; w.slices = 1; w.tail = 0;
    return w.tile < num_tiles;
  }
  const int main_tiles = num_tiles - p.tail_tiles;
  const int tile = first + it * step;
  if (tile < main_tiles) {
    w.tile = tile; w.kb0 = 0; w.kb1 = num_kb; w.slice = 0; w.slices = 1; w.tail = 0;
    return true;
  }
  if (p.tail_tiles == 0) return false;
  const int mine = first < main_tiles ? (main_tiles - first + step - 1) / step : 0;
  if (it != mine || first >= p.tail_tiles * p.tail_slices) return false;
  w.tail = first / p.tail_slices;
  w.slice = first - w.tail * p.tail_slices;
  w.slices = p.tail_slices;
  w.tile = main_tiles + w.tail;
  w.kb0 = (int)((int64_t)num_kb * w.slice / p.tail_slices);
  w.kb1 = (int)((int64_t)num_kb * (w.slice + 1) / p.tail_slices);
  return true;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr int PAIR_STAGES = 6;
constexpr int PAIR_B_STAGE_BYTES = 2 * B_BOX_BYTES;                      // 16 KiB
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_B_STAGE_BYTES;     // 32 KiB per CTA
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;

// TAIL: the instantiation that can cut the last partial wave along K (Params::tail_*); the
// plain one carries none of that code, so launches without a split run the kernel as it was.
// Registers: the 16-bit instantiations stay at 184 per thread (the split one is held there by
// __maxnreg__, without spills), because that decides what can run BESIDE this kernel: the six
// warps of a CTA sit on four SM sub-partitions of 16 K registers each, two of which hold two
// of them, so a 128-thread CTA of another kernel (one warp per sub-partition) fits only while
// 2 x this + its own registers per thread stay within 512.  Measured: beside the 248-register
// form a 128-thread kernel on a second stream started only when this one had ended; beside the
// 184-register form it ran concurrently (the all-reduce of the tensor-parallel MLP does).
template <typename OutT, bool DUAL, bool TAIL>
__global__ void __cluster_dims__(2, 1, 1) __maxnreg__(TAIL ? 184 : 255)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a,
                 const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_b2, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t a_smem = smem_base;
  const uint32_t b_smem = smem_base + PAIR_STAGES * A_STAGE_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_gen + PAIR_STAGES * PAIR_STAGE_BYTES);
  const uint32_t bar0 = smem_base + PAIR_STAGES * PAIR_STAGE_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (PAIR_STAGES + s); };
  auto acc_full_bar = [&](int a) { return bar0 + 8u * (2 * PAIR_STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bar0 + 8u * (2 * PAIR_STAGES + 2 + a); };
  const uint32_t drain_bar = bar0 + 8u * (2 * PAIR_STAGES + 4);
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * PAIR_STAGES + 5);
  volatile uint32_t *abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0: issues the MMAs of the pair
  const WaitCtx ctx{abort_flag, p.status};

  // DUAL: the even CTA holds the 128 columns of the first B operand, the odd CTA those of the
  // second, so every accumulator row has x Wg in columns [0,128) and x Wu in [128,256)
  constexpr int TILE_N = DUAL ? BN / 2 : BN;
  const int m_pairs = (p.M + 2 * BM - 1) / (2 * BM);
  const int n_blocks = (p.N + TILE_N - 1) / TILE_N;
  const int num_tiles = m_pairs * n_blocks;
  const int num_kb = (p.K + BK - 1) / BK;
  const int first_tile = (int)(blockIdx.x >> 1);
  const int tile_step = (int)(gridDim.x >> 1);
  const int group_pairs = (p.group_m + 1) / 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 8);
    }
    mbar_init(drain_bar, 1);
    *abort_flag = 0u;
    mbar_init_fence();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(DUAL && rank == 1 ? &tm_b2 : &tm_b);
  }
  if (warp == 5) tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  // the peer's barriers must be initialised before anything of this CTA reaches them
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // a programmatic dependent may start now: it reads nothing of this kernel's output before
  // the progress counters say so
  if (p.progress != nullptr) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 4) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued_mask = 0, issued_parity = 0;
      bool ok = true;
      PairWork w;
      for (int it = 0; ok && pair_work<TAIL>(p, it, first_tile, tile_step, num_tiles, num_kb, w); ++it) {
        int mp, nb;
        tile_coords(w.tile, m_pairs, n_blocks, group_pairs, mp, nb);
        const int row0 = (mp * 2 + (int)rank) * BM;
        const int col0 = DUAL ? nb * TILE_N : nb * BN + (int)rank * (BN / 2);
        const CUtensorMap *bmap = (DUAL && rank == 1) ? &tm_b2 : &tm_b;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, ctx, 1)) { ok = false; break; }
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * PAIR_STAGE_BYTES);
          const uint32_t full0 = map_to_cta(full_bar(stage), 0);
          tma_load_2d_pair(a_smem + stage * A_STAGE_BYTES, &tm_a, full0, kb * BK, row0);
          const uint32_t bdst = b_smem + stage * PAIR_B_STAGE_BYTES;
          if (p.b_kmajor) {
            // B rows are rows of K: this CTA's 128 of the tile's 256 columns as one box of
            // 64 (K) x 128 (N), laid out like the A tile
            tma_load_2d_pair(bdst, bmap, full0, kb * BK, col0);
          } else {
            tma_load_2d_pair(bdst, bmap, full0, col0, kb * BK);
            tma_load_2d_pair(bdst + B_BOX_BYTES, bmap, full0, col0 + 64, kb * BK);
          }
          issued_mask |= 1u << stage;
          issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && rank == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s)
          if (issued_mask & (1u << s)) mbar_wait_drain(full_bar(s), (issued_parity >> s) & 1u);
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ MMA issuer (even CTA)
    if (rank == 0) {
      const bool leader = elect_one();
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      auto wait_all = [&](uint32_t bar, uint32_t parity, uint32_t site) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, site)) != 0;
      };
      const uint32_t a_lo0 = desc_lo_sw128(a_smem, 16);
      const uint32_t b_lo0 = desc_lo_sw128(b_smem, p.b_lbo);
      constexpr uint32_t hi = desc_hi_sw128(1024);
      const uint32_t b_kstep = p.b_kstep;
      const uint32_t peer_bar0 = map_to_cta(bar0, 1);
      PairWork w;
      for (int it = 0; ok && pair_work<TAIL>(p, it, first_tile, tile_step, num_tiles, num_kb, w); ++it) {
        if (!wait_all(acc_empty_bar(acc), acc_phase ^ 1u, 2)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!wait_all(full_bar(stage), phase, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + (uint32_t)stage * (A_STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + (uint32_t)stage * (PAIR_B_STAGE_BYTES >> 4);
          if (leader) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              mma_f16_ss_pair(d_tmem, a_lo + (uint32_t)(k * ((UMMA_K * 2) >> 4)), hi,
                              b_lo + (uint32_t)k * b_kstep, hi, p.idesc,
                              (kb > w.kb0 || k > 0) ? 1u : 0u);
            // the stage is reusable in both CTAs once these MMAs retire
            tc_commit_pair(empty_bar(stage));
            tc_commit_pair(peer_bar0 + (empty_bar(stage) - bar0));
          }
          if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (leader) {
          tc_commit_pair(acc_full_bar(acc));
          tc_commit_pair(peer_bar0 + (acc_full_bar(acc) - bar0));
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (leader) {
        tc_commit_pair(drain_bar);
        mbar_wait_drain(drain_bar, 0);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    OutT *c = reinterpret_cast<OutT *>(p.c);
    const uint32_t acc_empty0 = map_to_cta(acc_empty_bar(0), 0);
    PairWork w;
    for (int it = 0; ok && pair_work<TAIL>(p, it, first_tile, tile_step, num_tiles, num_kb, w); ++it) {
      int mp, nb;
      tile_coords(w.tile, m_pairs, n_blocks, group_pairs, mp, nb);
      if (!__all_sync(0xffffffffu, mbar_wait(acc_full_bar(acc), acc_phase, ctx, 4))) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int mb = mp * 2 + (int)rank;
      const int row = mb * BM + warp * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * BN);
      int c0 = 0, c1 = DUAL ? BN / 64 : BN / 32;  // output chunks this pair finishes
      if (TAIL && w.slices > 1) {
        // A slice of a split tile.  Output chunks [c0, c1) are this slice's; with two B
        // operands output chunk c is accumulator chunks c (x Wg) and c + 4 (x Wu).  Partials
        // travel as [column][row] floats: 32 consecutive rows per warp access.
        const int S = w.slices;
        const int per = (DUAL ? BN / 64 : BN / 32) / S;
        c0 = w.slice * per;
        c1 = c0 + per;
        auto mine = [&](int a) {
          const int o = DUAL ? (a & 3) : a;
          return o >= c0 && o < c1;
        };
        unsigned int *flag = p.tail_flags + (size_t)((w.tail * 2 + (int)rank) * 4 + warp) * 2;
        const size_t part = (size_t)BN * BM;  // floats of one CTA's accumulator
        float *tile_ws = p.tail_ws + (size_t)w.tail * S * 2 * part + (size_t)rank * part +
                         (size_t)(warp * 32 + lane);
        float *own = tile_ws + (size_t)w.slice * 2 * part;
#pragma unroll 1
        for (int a = 0; a < BN / 32; ++a) {
          if (mine(a)) continue;  // warp-uniform
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + (uint32_t)(a * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) own[(size_t)(a * 32 + j) * BM] = __uint_as_float(r[j]);
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(flag, 1u);
        bool arrived = true;
        {
          const uint64_t t0 = globaltimer_ns();
          for (uint32_t spin = 0; ld_acquire_gpu(flag) < (unsigned int)S; ++spin) {
            if ((spin & 0x3f) == 0x3f && globaltimer_ns() - t0 > kWaitLimitNs) {
              arrived = false;
              break;
            }
          }
        }
        if (!__all_sync(0xffffffffu, arrived)) {
          if (lane == 0) atomicOr(p.status, (unsigned)B200_TIMEOUT | (5u << 8));
        } else {
          // Two slices: 32 columns at a time, one array of the other slice's partials; four
          // slices: 16 columns at a time, three arrays -- 64 values live either way (the
          // register count of this instantiation decides what fits beside it on an SM).
          // This slice's own partial first, then the others' in slice order: a fixed order, so
          // repeated launches give the same bits.
#pragma unroll 1
          for (int a = 0; a < BN / 32; ++a) {
            if (!mine(a)) continue;
            if (S == 2) {
              uint32_t r[32];
              tmem_ld_32x32b_x32(t_row + (uint32_t)(a * 32), r);
              const float *src = tile_ws + (size_t)(1 - w.slice) * 2 * part;
              float other[32];  // every load is issued before the first sum needs one
#pragma unroll
              for (int j = 0; j < 32; ++j) other[j] = __ldcg(src + (size_t)(a * 32 + j) * BM);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + other[j]);
              tmem_st_32x32b_x32(t_row + (uint32_t)(a * 32), r);
              continue;
            }
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
              const int col = a * 32 + h * 16;
              uint32_t r[16];
              tmem_ld_32x32b_x16(t_row + (uint32_t)col, r);
              float other[3][16];
#pragma unroll
              for (int k = 0; k < 3; ++k) {
                const int sl = k + (k >= w.slice ? 1 : 0);  // the other slices, in slice order
                const float *src = tile_ws + (size_t)sl * 2 * part;
#pragma unroll
                for (int j = 0; j < 16; ++j) other[k][j] = __ldcg(src + (size_t)(col + j) * BM);
              }
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 3; ++k) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  r[j] = __float_as_uint(__uint_as_float(r[j]) + other[k][j]);
              }
              tmem_st_32x32b_x16(t_row + (uint32_t)col, r);
            }
          }
          tmem_st_wait();
        }
        __syncwarp();
        // the last of the S readers puts both counters back to zero for the next launch
        if (lane == 0 && atomicAdd(flag + 1, 1u) == (unsigned int)(S - 1)) {
          flag[0] = 0u;
          flag[1] = 0u;
        }
      }
      OutT *crow = c + (int64_t)row * p.ldc;
      if (p.scatter_rows > 0) {
        const int owner = (mb * BM) / p.scatter_rows;
        const int local = row - owner * p.scatter_rows;
        crow = reinterpret_cast<OutT *>(p.c_rank[owner]) +
               ((int64_t)p.scatter_slot * p.scatter_rows + local) * p.ldc;
      }
      const int col_base = nb * TILE_N;
      const float row_mul = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f;
      if constexpr (TAIL)
        run_epilogue<OutT, DUAL>(t_row, p, crow, row, col_base, row_ok, row_mul, c0, c1);
      else
        run_epilogue<OutT, DUAL>(t_row, p, crow, row, col_base, row_ok, row_mul);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_empty0 + 8u * (uint32_t)acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      if (p.progress != nullptr) {
        // this warp's rows of the tile are stored: visible to every GPU before the count is
        __threadfence_system();
        __syncwarp();
        if (lane == 0) atomicAdd(p.progress + mp / group_pairs, 1u);
      }
    }
  }

  // neither CTA may leave while the pair's MMAs can still read its shared memory or write
  // its tensor memory: the even CTA has drained them before it arrives here
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------ CUDA-core path
// Any dtype, any stride alignment: 32x32 tiles through shared memory, fp32 FMA
// accumulation (IEEE for fp32 operands).  Serves shapes the tensor-core path
// rejects (row pitch not a multiple of 16 bytes, fp32 operands).
template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const InT *__restrict__ a, int64_t lda, const InT *__restrict__ b, int64_t ldb_k,
                 int64_t ldb_n, const InT *__restrict__ b2, OutT *__restrict__ c, int64_t ldc, int M, int N,
                 int K, const void *bias, int bias_kind, int act, const float *row_scale,
                 GroupNormMin gn) {
  __shared__ float sa[32][33];
  __shared__ float sb[32][33];
  __shared__ float sb2[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int m0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k0 = 0; k0 < K; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty + 8 * i;
      const int am = m0 + r, ak = k0 + tx;
      sa[r][tx] = (am < M && ak < K) ? io<InT>::load(a[(int64_t)am * lda + ak]) : 0.f;
      const int bk = k0 + r, bn = n0 + tx;
      const bool bok = bk < K && bn < N;
      sb[r][tx] = bok ? io<InT>::load(b[(int64_t)bk * ldb_k + (int64_t)bn * ldb_n]) : 0.f;
      if (b2 != nullptr)
        sb2[r][tx] = bok ? io<InT>::load(b2[(int64_t)bk * ldb_k + (int64_t)bn * ldb_n]) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < 32; ++k) {
      const float bv = sb[k][tx];
      const float bv2 = b2 != nullptr ? sb2[k][tx] : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float av = sa[ty + 8 * i][k];
        acc[i] = fmaf(av, bv, acc[i]);
        acc2[i] = fmaf(av, bv2, acc2[i]);
      }
    }
    __syncthreads();
  }
  const int n = n0 + tx;
  if (n >= N) return;
  const float bias_v = bias_kind ? load_bias(bias, bias_kind, n) : 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 8 * i;
    if (m >= M) continue;
    float z;
    if (act == B200_ACT_SWIGLU) {
      z = acc[i] / (1.0f + expf(-acc[i])) * acc2[i];
    } else {
      z = fmaf(acc[i], row_scale != nullptr ? row_scale[m] : 1.0f, bias_v);
      switch (act) {
        case B200_ACT_GELU_ERF: z = gelu_erf(z); break;
        case B200_ACT_GELU_TANH: z = gelu_tanh_exact(z); break;
        case B200_ACT_LEAKY_RELU: z = z >= 0.f ? z : 0.01f * z; break;
        default: break;
      }
    }
    if (gn.mins != nullptr) {
      // a 32-column tile is one group (gn.group == 32, N % 32 == 0): the lanes of this warp
      // hold the group's 32 values of row m
      const float mean = warp_sum(z) * (1.0f / 32);
      const float d = z - mean;
      const float rstd = rsqrtf(warp_sum(d * d) * (1.0f / 32) + gn.eps);
      const float out = d * rstd * load_bias(gn.gamma, gn.kind, n) + load_bias(gn.beta, gn.kind, n);
      const float lowest = -warp_max(-out);
      if (tx == 0) atomic_min_float(gn.mins + m, lowest);
      continue;
    }
    c[(int64_t)m * ldc + n] = io<OutT>::store(z);
  }
}

template <typename InT, typename OutT>
static int launch_simt(const b200_tensor *a, const b200_tensor *b, const b200_tensor *b2,
                       const b200_tensor *bias, b200_tensor *c, int act, cudaStream_t stream,
                       const float *row_scale = nullptr, const GroupNormMin *gn = nullptr,
                       bool b_rows_are_n = false) {
  const int M = (int)a->shape[0], K = (int)a->shape[1], N = (int)b->shape[b_rows_are_n ? 0 : 1];
  GroupNormMin gn_args = {nullptr, nullptr, 0, 0, 0.f, nullptr};
  if (gn != nullptr) {
    B200_REQUIRE(gn->group == 32 && N % 32 == 0,
                 "the CUDA-core path takes groups of exactly 32 columns");
    gn_args = *gn;
  }
  dim3 grid((N + 31) / 32, (M + 31) / 32);
  B200_REQUIRE(grid.y <= 65535, "M too large for the CUDA-core path");
  gemm_simt_kernel<InT, OutT><<<grid, 256, 0, stream>>>(
      (const InT *)a->data, a->stride[0], (const InT *)b->data,
      b_rows_are_n ? (int64_t)1 : b->stride[0], b_rows_are_n ? b->stride[0] : (int64_t)1,
      b2 ? (const InT *)b2->data : nullptr, (OutT *)c->data, c->stride[0], M, N, K,
      bias ? bias->data : nullptr, bias ? (int)bias->dtype : 0, act, row_scale, gn_args);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

template <typename OutT, bool DUAL>
static int launch_tc(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tb2,
                     const Params &p, cudaStream_t stream) {
  static bool configured[64] = {false};
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  auto kernel = gemm_tcgen05_kernel<OutT, DUAL>;
  if (dev < 64 && !configured[dev]) {
    B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      227 * 1024));
    configured[dev] = true;
  }
  constexpr int TILE_N = DUAL ? BN / 2 : BN;
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + TILE_N - 1) / TILE_N);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  const int smem = p.stages * (A_STAGE_BYTES + p.b_stage_bytes) + 1024 + 256;
  kernel<<<grid, THREADS, smem, stream>>>(ta, tb, tb2, p);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

// Scratch of the split last wave: at most one partial per SM pair (256 KiB each) and twelve
// flags per split tile, per (device, stream); allocated at the first launch that needs it and
// kept until the stream is destroyed through the library (release_gemm_scratch).
constexpr int kTailMinKb = 16;  // k-blocks of 64 a slice has at least (below that the exchange of partials costs what the split saves: 4096 x 4096 x 1792 measured 47.2 against 46.2 us)
struct TailScratch {
  float *ws;
  unsigned int *flags;
};
static std::mutex g_tail_lock;
static std::map<std::pair<int, cudaStream_t>, TailScratch> g_tail_scratch;

static bool tail_scratch(int pairs, cudaStream_t stream, TailScratch &out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> guard(g_tail_lock);
  auto key = std::make_pair(dev, stream);
  auto found = g_tail_scratch.find(key);
  if (found != g_tail_scratch.end()) {
    out = found->second;
    return true;
  }
  const size_t ws_bytes = (size_t)pairs * 2 * BN * BM * sizeof(float);
  const size_t flag_bytes = (size_t)pairs * 16 * sizeof(unsigned int);
  void *ws = nullptr, *flags = nullptr;
  if (cudaMalloc(&ws, ws_bytes) != cudaSuccess || cudaMalloc(&flags, flag_bytes) != cudaSuccess ||
      cudaMemset(flags, 0, flag_bytes) != cudaSuccess) {
    (void)cudaGetLastError();
    if (ws) cudaFree(ws);
    if (flags) cudaFree(flags);
    return false;
  }
  out = TailScratch{static_cast<float *>(ws), static_cast<unsigned int *>(flags)};
  g_tail_scratch[key] = out;
  return true;
}

template <typename OutT, bool DUAL>
static int launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tb2,
                       const Params &p_in, cudaStream_t stream,
                       const Progress *progress = nullptr) {
  Params p = p_in;
  p.progress = nullptr;
  static bool configured[64] = {false};
  static int max_clusters[64] = {0};
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  auto kernel = gemm_pair_kernel<OutT, DUAL, false>;
  auto kernel_tail = gemm_pair_kernel<OutT, DUAL, true>;
  if (dev >= 64) return fail(B200_RESOURCE, "device index %d out of range", dev);
  if (!configured[dev]) {
    B200_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PAIR_SMEM_BYTES));
    B200_CUDA_OK(cudaFuncSetAttribute(kernel_tail, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      PAIR_SMEM_BYTES));
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3((unsigned)sm_count());
    probe.blockDim = dim3(THREADS);
    probe.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    probe.attrs = &attr;
    probe.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &probe) != cudaSuccess) {
      (void)cudaGetLastError();
      n = 0;
    }
    max_clusters[dev] = n > 0 ? n : sm_count() / 2;
    configured[dev] = true;
  }
  constexpr int TILE_N = DUAL ? BN / 2 : BN;
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + TILE_N - 1) / TILE_N);
  const int clusters = tiles < max_clusters[dev] ? tiles : max_clusters[dev];
  // the last partial wave, cut along K when that makes it shorter (B200OPS_GEMM_TAIL=0: never)
  p.tail_tiles = 0;
  p.tail_slices = 1;
  p.tail_ws = nullptr;
  p.tail_flags = nullptr;
  static const int tail_env =
      getenv("B200OPS_GEMM_TAIL") ? atoi(getenv("B200OPS_GEMM_TAIL")) : 1;
  const int rest = tiles % clusters;
  const int num_kb = (p.K + BK - 1) / BK;
  // (not for the group-norm epilogue, which needs whole rows of a tile in one thread)
  if (tail_env != 0 && tiles > clusters && rest > 0 && p.act != kActGroupNormMin) {
    int slices = rest * 4 <= clusters ? 4 : (rest * 2 <= clusters ? 2 : 1);
    while (slices > 1 && num_kb / slices < kTailMinKb) slices /= 2;
    // the instantiation with the split runs its whole waves about 2 % slower (measured): with
    // many waves that costs more than the shorter last wave gives back
    const int waves = tiles / clusters;
    if ((slices == 4 && waves > 24) || (slices == 2 && waves > 12)) slices = 1;
    TailScratch scratch;
    if (slices >= 2 && tail_scratch(max_clusters[dev], stream, scratch)) {
      p.tail_tiles = rest;
      p.tail_slices = slices;
      p.tail_ws = scratch.ws;
      p.tail_flags = scratch.flags;
    }
  }
  if (progress != nullptr) {
    // per block of rows (= raster group): eight epilogue warps count once per whole tile and
    // once per slice of a split tile; the split tiles are the last ones in raster order
    const int m_pairs = (p.M + 2 * BM - 1) / (2 * BM);
    const int n_blocks = (p.N + TILE_N - 1) / TILE_N;
    const int group_pairs = (p.group_m + 1) / 2;
    const int groups = (m_pairs + group_pairs - 1) / group_pairs;
    if (groups > progress->max_blocks)
      return fail(B200_REJECTED, "%d blocks of rows, room for %d", groups, progress->max_blocks);
    for (int g = 0; g < groups; ++g) {
      const int pairs = std::min(group_pairs, m_pairs - g * group_pairs);
      const int first = g * group_pairs * n_blocks, last = first + pairs * n_blocks;
      const int split_from = std::max(first, tiles - p.tail_tiles);
      const int split = last > split_from ? last - split_from : 0;
      progress->targets[g] = 8u * (unsigned)((last - first - split) + split * p.tail_slices);
    }
    *progress->blocks = groups;
    p.progress = progress->counters;
  }
  if (p.tail_tiles > 0)
    kernel_tail<<<2 * clusters, THREADS, PAIR_SMEM_BYTES, stream>>>(ta, tb, tb2, p);
  else
    kernel<<<2 * clusters, THREADS, PAIR_SMEM_BYTES, stream>>>(ta, tb, tb2, p);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // namespace gemm

// Called by b200_stream_destroy: frees the split-wave scratch kept for (current device, stream).
void release_gemm_scratch(cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  gemm::TailScratch scratch{nullptr, nullptr};
  {
    std::lock_guard<std::mutex> guard(gemm::g_tail_lock);
    auto found = gemm::g_tail_scratch.find(std::make_pair(dev, stream));
    if (found == gemm::g_tail_scratch.end()) return;
    scratch = found->second;
    gemm::g_tail_scratch.erase(found);
  }
  (void)cudaStreamSynchronize(stream);
  (void)cudaFree(scratch.ws);
  (void)cudaFree(scratch.flags);
}
}  // namespace b200

namespace b200 {
namespace gemm {
struct Scatter {
  void *const *c_rank;  // device pointers, one per rank
  int world, slot;
  int64_t rows;         // rows of C owned by each rank
};
}  // namespace gemm
}  // namespace b200

// y[row] = log_softmax(x[row] . w[n], n < N) for operands the tensor-core path does not take
// (fp32, unaligned rows): one CTA per row, thread n owns output n.
namespace b200 {
namespace gemm {
template <typename T, typename OutT>
__global__ void __launch_bounds__(256)
linear_log_softmax_simt_kernel(const T *__restrict__ x, const T *__restrict__ w,
                               OutT *__restrict__ y, int N, int K, int64_t ldx, int64_t ldw,
                               int64_t ldy) {
  __shared__ float red[8];
  const int row = blockIdx.x, n = threadIdx.x;
  const T *xr = x + (int64_t)row * ldx;
  float z = 0.f;
  if (n < N) {
    const T *wr = w + (int64_t)n * ldw;
    for (int k = 0; k < K; ++k) z = fmaf(io<T>::load(xr[k]), io<T>::load(wr[k]), z);
  }
  float mx = warp_max(n < N ? z : -INFINITY);
  if ((n & 31) == 0) red[n >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = warp_sum(n < N ? expf(z - mx) : 0.f);
  if ((n & 31) == 0) red[n >> 5] = sum;
  __syncthreads();
  sum = 0.f;
  for (int i = 0; i < 8; ++i) sum += red[i];
  if (n < N) y[(int64_t)row * ldy + n] = io<OutT>::store(z - mx - logf(sum));
}
}  // namespace gemm
}  // namespace b200

// b_rows_are_n: B is given as [N, K] (the weight layout of a linear layer) instead of [K, N].
static int gemm_impl(const b200_tensor *a, const b200_tensor *b, const b200_tensor *b2,
                     const b200_tensor *bias, b200_tensor *c, int act, void *stream,
                     const b200::gemm::Scatter *scatter, bool b_rows_are_n = false,
                     const float *row_scale = nullptr,
                     const b200::gemm::GroupNormMin *gn = nullptr,
                     const b200::gemm::Progress *progress = nullptr) {
  using namespace b200;
  using namespace b200::gemm;
  int st;
  if ((st = check_tensor(a, "a", 2)) || (st = check_tensor(b, "b", 2)) ||
      (st = check_tensor(c, "c", 2)))
    return st;
  if ((act < B200_ACT_NONE || act > B200_ACT_SWIGLU) && act != kActLogSoftmax &&
      act != kActGroupNormMin)
    return fail(B200_USAGE, "act %d is not a b200_act value", act);
  if (bias != nullptr && (st = check_tensor(bias, "bias", 1))) return st;
  if (act == B200_ACT_SWIGLU) {
    if (b2 == nullptr) return fail(B200_USAGE, "B200_ACT_SWIGLU needs the second B operand");
    if ((st = check_tensor(b2, "b2", 2))) return st;
    B200_REQUIRE(bias == nullptr, "B200_ACT_SWIGLU takes no bias");
  } else if (b2 != nullptr) {
    return fail(B200_USAGE, "b2 is only used with B200_ACT_SWIGLU");
  }
  B200_REQUIRE(is_float_io(a->dtype), "a: dtype %u is not f16/bf16/f32", a->dtype);
  B200_REQUIRE(b->dtype == a->dtype, "a/b dtypes differ (%u/%u)", a->dtype, b->dtype);
  // a 16-bit product may be stored in the other 16-bit type (float16 partials of bfloat16
  // operands keep three more mantissa bits at the same size)
  B200_REQUIRE(c->dtype == a->dtype || c->dtype == B200_DTYPE_FLOAT32 ||
               (a->dtype != B200_DTYPE_FLOAT32 && is_float_io(c->dtype)),
               "c dtype %u must be a's dtype, the other 16-bit type or f32", c->dtype);
  const int64_t M = a->shape[0], K = a->shape[1], N = b->shape[b_rows_are_n ? 0 : 1];
  B200_REQUIRE(b->shape[b_rows_are_n ? 1 : 0] == K, "a is [%lld,%lld] but b has K = %lld",
               (long long)M, (long long)K, (long long)b->shape[b_rows_are_n ? 1 : 0]);
  if (act == kActLogSoftmax)
    B200_REQUIRE(N >= 1 && N <= BN && bias == nullptr && b2 == nullptr && scatter == nullptr,
                 "the row log-softmax epilogue takes 1..%d output columns, no bias", BN);
  B200_REQUIRE(c->shape[0] == M && c->shape[1] == N, "c shape is not [M,N]");
  B200_REQUIRE(a->stride[1] == 1 && b->stride[1] == 1 && c->stride[1] == 1,
               "a/b/c need unit column stride (row-major)");
  B200_REQUIRE(a->stride[0] >= K && b->stride[0] >= (b_rows_are_n ? K : N) && c->stride[0] >= N,
               "row stride below row width");
  B200_REQUIRE(M < (1 << 30) && N < (1 << 30) && K < (1 << 30), "extent out of range");
  if (b2 != nullptr) {
    B200_REQUIRE(b2->dtype == b->dtype && b2->shape[0] == K && b2->shape[1] == N &&
                 b2->stride[1] == 1 && b2->stride[0] == b->stride[0],
                 "b2 must match b in dtype, shape and strides");
  }
  if (bias != nullptr) {
    B200_REQUIRE(bias->shape[0] == N && bias->stride[0] == 1, "bias must be contiguous [N]");
    B200_REQUIRE(bias->dtype == B200_DTYPE_FLOAT32 || bias->dtype == a->dtype,
                 "bias dtype %u must be f32 or a's dtype", bias->dtype);
  }
  if (M == 0 || N == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;

  const size_t es = dtype_size(a->dtype);
  const bool tensor_core =
      K > 0 && a->dtype != B200_DTYPE_FLOAT32 && (a->stride[0] * es) % 16 == 0 &&
      (b->stride[0] * es) % 16 == 0 && (uintptr_t)a->data % 16 == 0 &&
      (uintptr_t)b->data % 16 == 0 && (b2 == nullptr || (uintptr_t)b2->data % 16 == 0);
  if (scatter != nullptr) {
    B200_REQUIRE(tensor_core, "the row-scatter epilogue exists only on the tensor-core path "
                              "(16-bit operands, 16-byte aligned row pitches)");
    B200_REQUIRE(scatter->world >= 1 && scatter->world <= 8 && scatter->slot >= 0 &&
                 scatter->slot < scatter->world, "world %d / slot %d out of range",
                 scatter->world, scatter->slot);
    B200_REQUIRE(scatter->rows > 0 && scatter->rows % BM == 0 &&
                 scatter->rows * scatter->world >= M,
                 "rows per rank (%lld) must be a multiple of %d and cover M", 
                 (long long)scatter->rows, BM);
    B200_REQUIRE(c->stride[0] == N, "scattered C slots are contiguous [rows, N]");
    for (int r = 0; r < scatter->world; ++r)
      B200_REQUIRE(scatter->c_rank[r] != nullptr && (uintptr_t)scatter->c_rank[r] % 16 == 0,
                   "destination pointer of rank %d is null or unaligned", r);
  }
  if (!tensor_core)
    B200_REQUIRE(c->dtype == a->dtype || c->dtype == B200_DTYPE_FLOAT32,
                 "the CUDA-core paths store c in a's dtype or f32 (got %u)", c->dtype);
  if (!tensor_core && act == kActLogSoftmax) {
    B200_REQUIRE(b_rows_are_n, "the CUDA-core log-softmax path takes B as [N, K]");
#define B200_LLS(T, OutT)                                                                   \
  linear_log_softmax_simt_kernel<T, OutT><<<(unsigned)M, 256, 0, s>>>(                      \
      (const T *)a->data, (const T *)b->data, (OutT *)c->data, (int)N, (int)K, a->stride[0], \
      b->stride[0], c->stride[0])
    if (a->dtype == B200_DTYPE_FLOAT32) B200_LLS(float, float);
    else if (a->dtype == B200_DTYPE_FLOAT16 && c->dtype == B200_DTYPE_FLOAT32) B200_LLS(__half, float);
    else if (a->dtype == B200_DTYPE_FLOAT16) B200_LLS(__half, __half);
    else if (c->dtype == B200_DTYPE_FLOAT32) B200_LLS(__nv_bfloat16, float);
    else B200_LLS(__nv_bfloat16, __nv_bfloat16);
#undef B200_LLS
    B200_CUDA_OK(cudaGetLastError());
    return B200_OK;
  }
  if (!tensor_core) {
    const bool t = b_rows_are_n;
    if (a->dtype == B200_DTYPE_FLOAT32) return launch_simt<float, float>(a, b, b2, bias, c, act, s, row_scale, gn, t);
    if (a->dtype == B200_DTYPE_FLOAT16) {
      return c->dtype == B200_DTYPE_FLOAT32
                 ? launch_simt<__half, float>(a, b, b2, bias, c, act, s, row_scale, gn, t)
                 : launch_simt<__half, __half>(a, b, b2, bias, c, act, s, row_scale, gn, t);
    }
    return c->dtype == B200_DTYPE_FLOAT32
               ? launch_simt<__nv_bfloat16, float>(a, b, b2, bias, c, act, s, row_scale, gn, t)
               : launch_simt<__nv_bfloat16, __nv_bfloat16>(a, b, b2, bias, c, act, s, row_scale, gn, t);
  }

  // CTA pairs (256-row tiles) when the pair tiles fill at least one wave of SM pairs (a pair
  // always multiplies 256 columns: not for outputs of at most half a tile, nor for the row
  // log-softmax, whose epilogue needs the whole row in one CTA); B200OPS_GEMM_PAIR=0 / 1
  // forces the choice.
  const bool dual = act == B200_ACT_SWIGLU;
  bool use_pair;
  {
    static const int pair_env =
        getenv("B200OPS_GEMM_PAIR") ? atoi(getenv("B200OPS_GEMM_PAIR")) : -1;
    const int tile_n = dual ? BN / 2 : BN;
    const int64_t pair_tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + tile_n - 1) / tile_n);
    use_pair = act != kActLogSoftmax &&
               (pair_env >= 0 ? pair_env != 0 : pair_tiles >= sm_count() / 2 && N > tile_n / 2);
  }

  CUtensorMap ta, tb, tb2;
  {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    const uint64_t strides[2] = {es, (uint64_t)a->stride[0] * es};
    const uint32_t box[2] = {BK, BM};
    if ((st = encode_tensor_map(&ta, a->dtype, a->data, 2, dims, strides, box))) return st;
  }
  // one column block narrower than the tile (one-CTA kernel): load only the columns that exist
  const bool narrow = !dual && !use_pair && N < BN && act != kActGroupNormMin;
  const int n_mma = narrow ? (int)((N + 15) / 16 * 16) : BN;
  if (b_rows_are_n) {
    const uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    const uint64_t strides[2] = {es, (uint64_t)b->stride[0] * es};
    const uint32_t box[2] = {BK, (uint32_t)(use_pair ? BN / 2 : n_mma)};
    if ((st = encode_tensor_map(&tb, b->dtype, b->data, 2, dims, strides, box))) return st;
    tb2 = tb;
  } else {
    const uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    const uint64_t strides[2] = {es, (uint64_t)b->stride[0] * es};
    const uint32_t box[2] = {64, BK};
    if ((st = encode_tensor_map(&tb, b->dtype, b->data, 2, dims, strides, box))) return st;
    tb2 = tb;
    if (b2 != nullptr &&
        (st = encode_tensor_map(&tb2, b2->dtype, b2->data, 2, dims, strides, box)))
      return st;
  }
  Params p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.act = act;
  p.bias_kind = bias ? (int)bias->dtype : 0;
  p.bias = bias ? bias->data : nullptr;
  p.c = c->data;
  p.ldc = c->stride[0];
  p.idesc = sm100::make_idesc_f16(BM, BN, a->dtype == B200_DTYPE_BFLOAT16 ? 1 : 0, 0,
                                  b_rows_are_n ? 0 : 1);
  const size_t cs = dtype_size(c->dtype);
  p.vector_store = ((c->stride[0] * cs) % 16 == 0 && (uintptr_t)c->data % 16 == 0) ? 1 : 0;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(B200_RESOURCE, "no status word on this device");
  p.row_scale = row_scale;
  p.gn = gn != nullptr ? *gn : GroupNormMin{nullptr, nullptr, 0, 0, 0.f, nullptr};
  p.b_kmajor = b_rows_are_n ? 1 : 0;
  p.b_lbo = b_rows_are_n ? 16 : B_BOX_BYTES;  // [K,N]: pitch between 64-column chunks of the tile
  p.b_sbo = 1024;                             // pitch between groups of 8 rows
  p.b_kstep = b_rows_are_n ? (UMMA_K * 2) >> 4 : (UMMA_K * 128) >> 4;
  p.scatter_rows = 0;
  p.scatter_slot = 0;
  p.b_boxes = narrow ? (int)((N + 63) / 64) : 4;
  p.b_stage_bytes = b_rows_are_n ? n_mma * BK * 2 : p.b_boxes * B_BOX_BYTES;
  p.stages = (227 * 1024 - 1024 - 256) / (A_STAGE_BYTES + p.b_stage_bytes);
  if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
  {
    // Raster groups: as many m-blocks as keep a group's rows of A (group_m x 128 x K)
    // within about 40 MiB, the part of the L2 that was seen to hold a panel while B streams
    // past it; the groups are evened out.  8192^3: 4 groups of 16 m-blocks;
    // 4097 x 11008 x 4096: one group, A read from memory once (1330 -> 1370 TFLOP/s).
    static const int group_env =
        getenv("B200OPS_GEMM_GROUP_M") ? atoi(getenv("B200OPS_GEMM_GROUP_M")) : 0;
    const int m_blocks = (int)((M + BM - 1) / BM);
    const int64_t block_bytes = (int64_t)BM * K * (int64_t)dtype_size(a->dtype);
    int gmax = (int)(((int64_t)40 << 20) / (block_bytes > 0 ? block_bytes : 1));
    if (gmax < 4) gmax = 4;
    const int groups = (m_blocks + gmax - 1) / gmax;
    p.group_m = group_env > 0 ? group_env : (m_blocks + groups - 1) / (groups > 0 ? groups : 1);
    if (p.group_m < 1) p.group_m = 1;
  }
  p.progress = nullptr;
  if (progress != nullptr) {
    B200_REQUIRE(use_pair && b2 == nullptr && scatter == nullptr,
                 "progress counters exist on the CTA-pair kernel with one B operand");
    B200_REQUIRE(progress->counters != nullptr && progress->targets != nullptr &&
                 progress->blocks != nullptr && progress->rows_per_block > 0 &&
                 progress->rows_per_block % (2 * BM) == 0,
                 "rows per block must be a positive multiple of %d", 2 * BM);
    p.group_m = (int)(progress->rows_per_block / BM);  // a block of rows is a raster group
  }
  for (int r = 0; r < 8; ++r) p.c_rank[r] = nullptr;
  if (scatter != nullptr) {
    p.scatter_rows = (int)scatter->rows;
    p.scatter_slot = scatter->slot;
    for (int r = 0; r < scatter->world; ++r) p.c_rank[r] = scatter->c_rank[r];
  }

  if (narrow) {
    // the MMAs take only the columns that exist (rounded up to the instruction's granule of
    // 16) instead of 256 -- a [65536, 4096] x [4096, 64] product is then bound by reading x,
    // not by the tensor pipe
    p.idesc = sm100::make_idesc_f16(BM, n_mma, a->dtype == B200_DTYPE_BFLOAT16 ? 1 : 0, 0,
                                    b_rows_are_n ? 0 : 1);
  }
  if (use_pair) {
    Params q = p;
    q.idesc = sm100::make_idesc_f16(2 * BM, BN, a->dtype == B200_DTYPE_BFLOAT16 ? 1 : 0, 0,
                                    b_rows_are_n ? 0 : 1);
    if (c->dtype == B200_DTYPE_FLOAT32)
      return dual ? launch_pair<float, true>(ta, tb, tb2, q, s)
                  : launch_pair<float, false>(ta, tb, tb2, q, s, progress);
    if (c->dtype == B200_DTYPE_FLOAT16)
      return dual ? launch_pair<__half, true>(ta, tb, tb2, q, s)
                  : launch_pair<__half, false>(ta, tb, tb2, q, s, progress);
    return dual ? launch_pair<__nv_bfloat16, true>(ta, tb, tb2, q, s)
                : launch_pair<__nv_bfloat16, false>(ta, tb, tb2, q, s, progress);
  }
  if (c->dtype == B200_DTYPE_FLOAT32)
    return dual ? launch_tc<float, true>(ta, tb, tb2, p, s) : launch_tc<float, false>(ta, tb, tb2, p, s);
  if (c->dtype == B200_DTYPE_FLOAT16)
    return dual ? launch_tc<__half, true>(ta, tb, tb2, p, s) : launch_tc<__half, false>(ta, tb, tb2, p, s);
  return dual ? launch_tc<__nv_bfloat16, true>(ta, tb, tb2, p, s)
              : launch_tc<__nv_bfloat16, false>(ta, tb, tb2, p, s);
}

extern "C" int b200_gemm_bias_act(const b200_tensor *a, const b200_tensor *b,
                                  const b200_tensor *b2, const b200_tensor *bias,
                                  b200_tensor *c, int act, void *stream) {
  return gemm_impl(a, b, b2, bias, c, act, stream, nullptr);
}

extern "C" int b200_linear_bias_act(const b200_tensor *x, const b200_tensor *w,
                                    const b200_tensor *bias, b200_tensor *y, int act,
                                    void *stream) {
  if (act == B200_ACT_SWIGLU)
    return b200::fail(B200_USAGE, "B200_ACT_SWIGLU takes two [K,N] operands: b200_gemm_bias_act");
  return gemm_impl(x, w, nullptr, bias, y, act, stream, nullptr, true);
}

extern "C" int b200_gemm_scatter_rows(const b200_tensor *a, const b200_tensor *b,
                                      const b200_tensor *c_like, void *const *c_rank, int world,
                                      int slot, int64_t rows_per_rank, void *stream) {
  using namespace b200;
  if (c_rank == nullptr || c_like == nullptr) return fail(B200_USAGE, "null argument");
  b200_tensor c = *c_like;
  if (world >= 1 && world <= 8 && slot >= 0 && slot < world) c.data = c_rank[slot];
  const gemm::Scatter scatter{c_rank, world, slot, rows_per_rank};
  return gemm_impl(a, b, nullptr, nullptr, &c, B200_ACT_NONE, stream, &scatter);
}

extern "C" int b200_gemm_progress(const b200_tensor *a, const b200_tensor *b, b200_tensor *c,
                                  int64_t rows_per_block, unsigned int *counters,
                                  unsigned int *targets, int max_blocks, int *blocks,
                                  void *stream) {
  using namespace b200;
  if (counters == nullptr || targets == nullptr || blocks == nullptr || max_blocks < 1)
    return fail(B200_USAGE, "null argument");
  const gemm::Progress progress{counters, rows_per_block, targets, max_blocks, blocks};
  return gemm_impl(a, b, nullptr, nullptr, c, B200_ACT_NONE, stream, nullptr, false, nullptr,
                   nullptr, &progress);
}

extern "C" int b200_linear_log_softmax(const b200_tensor *x, const b200_tensor *w, b200_tensor *y,
                                       void *stream) {
  return gemm_impl(x, w, nullptr, nullptr, y, b200::gemm::kActLogSoftmax, stream, nullptr, true);
}

// ---- RMS-normalised matmul ----------------------------------------------------------
namespace b200 {
namespace gemm {

// rinv[row] = rsqrt(mean(x[row]^2) + eps)
template <typename T>
__global__ void __launch_bounds__(256)
row_rinv_kernel(const T *__restrict__ x, int64_t ldx, int K, float eps, float *__restrict__ rinv) {
  __shared__ float red[8];
  const T *xr = x + (int64_t)blockIdx.x * ldx;
  float sum = 0.f;
  constexpr int PER = 16 / (int)sizeof(T);
  if ((ldx * (int64_t)sizeof(T)) % 16 == 0 && (uintptr_t)x % 16 == 0) {
    const int vecs = K / PER;
    for (int i = threadIdx.x; i < vecs; i += 256) {
      vec16<T> v;
      v.raw = ld_stream16(xr + i * PER);
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const float f = io<T>::load(v.e[j]);
        sum = fmaf(f, f, sum);
      }
    }
    for (int k = vecs * PER + threadIdx.x; k < K; k += 256) {
      const float f = io<T>::load(xr[k]);
      sum = fmaf(f, f, sum);
    }
  } else {
    for (int k = threadIdx.x; k < K; k += 256) {
      const float f = io<T>::load(xr[k]);
      sum = fmaf(f, f, sum);
    }
  }
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < 8; ++i) total += red[i];
    rinv[blockIdx.x] = rsqrtf(total / (float)K + eps);
  }
}

// out[k, n] = g[k] * w[k, n], one rounding
template <typename T>
__global__ void __launch_bounds__(256)
scale_rows_kernel(const T *__restrict__ w, int64_t ldw, const T *__restrict__ g, T *__restrict__ out,
                  int64_t ldo, int K, int N) {
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    const float gk = io<T>::load(g[k]);
    for (int n = blockIdx.x * 256 + threadIdx.x; n < N; n += gridDim.x * 256)
      out[(int64_t)k * ldo + n] = io<T>::store(gk * io<T>::load(w[(int64_t)k * ldw + n]));
  }
}

// the same on 16-byte vectors (rows of w and out 16-byte aligned, N a multiple of the vector)
template <typename T>
__global__ void __launch_bounds__(256)
scale_rows_vec_kernel(const T *__restrict__ w, int64_t ldw, const T *__restrict__ g,
                      T *__restrict__ out, int64_t ldo, int K, int nvec) {
  constexpr int PER = 16 / (int)sizeof(T);
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    const float gk = io<T>::load(g[k]);
    for (int v = blockIdx.x * 256 + threadIdx.x; v < nvec; v += gridDim.x * 256) {
      vec16<T> a, o;
      a.raw = ld_stream16(w + (int64_t)k * ldw + (int64_t)v * PER);
#pragma unroll
      for (int j = 0; j < PER; ++j) o.e[j] = io<T>::store(gk * io<T>::load(a.e[j]));
      *reinterpret_cast<uint4 *>(out + (int64_t)k * ldo + (int64_t)v * PER) = o.raw;
    }
  }
}

template <typename T>
static int rms_matmul_prepare(const b200_tensor *x, const b200_tensor *g, const b200_tensor *w,
                              b200_tensor *scaled_w, float *rinv, float eps, cudaStream_t s) {
  const int M = (int)x->shape[0], K = (int)x->shape[1], N = (int)w->shape[1];
  row_rinv_kernel<T><<<M, 256, 0, s>>>((const T *)x->data, x->stride[0], K, eps, rinv);
  B200_CUDA_OK(cudaGetLastError());
  constexpr int PER = 16 / (int)sizeof(T);
  const bool vec_ok = N % PER == 0 && w->stride[0] % PER == 0 && scaled_w->stride[0] % PER == 0 &&
                      (uintptr_t)w->data % 16 == 0 && (uintptr_t)scaled_w->data % 16 == 0;
  if (vec_ok) {
    const int nvec = N / PER;
    dim3 grid((unsigned)((nvec + 255) / 256 < 16 ? (nvec + 255) / 256 : 16),
              (unsigned)(K < 2048 ? K : 2048));
    scale_rows_vec_kernel<T><<<grid, 256, 0, s>>>((const T *)w->data, w->stride[0],
                                                  (const T *)g->data, (T *)scaled_w->data,
                                                  scaled_w->stride[0], K, nvec);
  } else {
    dim3 grid((unsigned)((N + 255) / 256 < 64 ? (N + 255) / 256 : 64), (unsigned)(K < 4096 ? K : 4096));
    scale_rows_kernel<T><<<grid, 256, 0, s>>>((const T *)w->data, w->stride[0], (const T *)g->data,
                                              (T *)scaled_w->data, scaled_w->stride[0], K, N);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // namespace gemm
}  // namespace b200

extern "C" int b200_rms_matmul(const b200_tensor *x, const b200_tensor *g, const b200_tensor *w,
                               b200_tensor *out, float eps, b200_tensor *scratch_w,
                               b200_tensor *scratch_rinv, void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(x, "x", 2)) || (st = check_tensor(g, "g", 1)) ||
      (st = check_tensor(w, "w", 2)) || (st = check_tensor(out, "out", 2)) ||
      (st = check_tensor(scratch_w, "scratch_w", 2)) ||
      (st = check_tensor(scratch_rinv, "scratch_rinv", 1)))
    return st;
  B200_REQUIRE(is_float_io(x->dtype) && w->dtype == x->dtype && g->dtype == x->dtype &&
               scratch_w->dtype == x->dtype, "x, g, w and scratch_w must share one float type");
  const int64_t M = x->shape[0], K = x->shape[1], N = w->shape[1];
  B200_REQUIRE(w->shape[0] == K && g->shape[0] == K && g->stride[0] == 1, "g must be contiguous [K], w [K,N]");
  B200_REQUIRE(x->stride[1] == 1 && w->stride[1] == 1 && x->stride[0] >= K && w->stride[0] >= N,
               "x and w need unit column stride");
  B200_REQUIRE(scratch_w->shape[0] == K && scratch_w->shape[1] == N && scratch_w->stride[1] == 1 &&
               scratch_w->stride[0] >= N, "scratch_w must be [K,N]");
  B200_REQUIRE(scratch_rinv->dtype == B200_DTYPE_FLOAT32 && scratch_rinv->shape[0] >= M &&
               scratch_rinv->stride[0] == 1, "scratch_rinv must be f32 [>= M]");
  B200_REQUIRE(eps == eps && eps >= 0.f, "eps must be non-negative");
  B200_REQUIRE(K > 0, "K must be positive");
  if (M == 0 || N == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  float *rinv = (float *)scratch_rinv->data;
  if (x->dtype == B200_DTYPE_FLOAT32) st = gemm::rms_matmul_prepare<float>(x, g, w, scratch_w, rinv, eps, s);
  else if (x->dtype == B200_DTYPE_FLOAT16) st = gemm::rms_matmul_prepare<__half>(x, g, w, scratch_w, rinv, eps, s);
  else st = gemm::rms_matmul_prepare<__nv_bfloat16>(x, g, w, scratch_w, rinv, eps, s);
  if (st) return st;
  return gemm_impl(x, scratch_w, nullptr, nullptr, out, B200_ACT_NONE, stream, nullptr, false, rinv);
}

extern "C" int b200_gemm_groupnorm_rowmin(const b200_tensor *x, const b200_tensor *w,
                                          const b200_tensor *bias, const b200_tensor *gamma,
                                          const b200_tensor *beta, b200_tensor *mins,
                                          int group_size, float eps, void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(x, "x", 2)) || (st = check_tensor(w, "w", 2)) ||
      (st = check_tensor(gamma, "gamma", 1)) || (st = check_tensor(beta, "beta", 1)) ||
      (st = check_tensor(mins, "mins", 1)))
    return st;
  const int64_t M = x->shape[0], N = w->shape[1];
  B200_REQUIRE(group_size == 8 || group_size == 16 || group_size == 32 || group_size == 64,
               "group_size %d is not 8, 16, 32 or 64", group_size);
  B200_REQUIRE(N % group_size == 0, "N %lld is not a multiple of the group size %d",
               (long long)N, group_size);
  B200_REQUIRE(gamma->shape[0] == N && beta->shape[0] == N && gamma->stride[0] == 1 &&
               beta->stride[0] == 1 && gamma->dtype == beta->dtype &&
               (gamma->dtype == B200_DTYPE_FLOAT32 || gamma->dtype == x->dtype),
               "gamma and beta must be contiguous [N] in f32 or x's type");
  B200_REQUIRE(mins->dtype == B200_DTYPE_FLOAT32 && mins->shape[0] == M && mins->stride[0] == 1,
               "mins must be contiguous f32 [M]");
  B200_REQUIRE(eps == eps && eps >= 0.f, "eps must be non-negative");
  gemm::GroupNormMin gn = {gamma->data, beta->data, (int)gamma->dtype, group_size, eps,
                           (float *)mins->data};
  // the product is never stored: this descriptor only carries the shape and an f32 type
  b200_tensor c = {};
  c.data = mins->data;
  c.ndim = 2;
  c.dtype = B200_DTYPE_FLOAT32;
  c.shape[0] = M; c.shape[1] = N;
  c.stride[0] = N; c.stride[1] = 1;
  return gemm_impl(x, w, nullptr, bias, &c, b200::gemm::kActGroupNormMin, stream, nullptr, false,
                   nullptr, &gn);
}
