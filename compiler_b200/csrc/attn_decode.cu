// Decode-side attention: one query row per (batch, head) against that head's K / V cache.
//
// Native form of flash_decode_kernel (ops/suite/perf/flash_decode.py:21-49):
//   out[b] = softmax(scale * K[b / group] q[b]) V[b / group]
// with q / out [B, D] and K / V [B / group, N, D]; `group` > 1 is the grouped-query
// layout of ops/suite/dev/gqa.py:29 (query head b reads K / V head b / group).
//
// The operator reads K and V once and does two flops per byte, so it is bound by HBM
// (2 * N * D elements per query row).  Layout of the fast kernel:
//   * a key row of D elements is LPK = D * sizeof(T) / 16 lanes wide, one 16-byte streaming
//     load per lane; a warp load covers 32 / LPK consecutive keys, fully coalesced;
//   * every group of LPK lanes keeps its own online-softmax state (running max in the log2
//     domain, sum, D / LPK accumulator columns) over the keys it has seen, so the loop has
//     no cross-key synchronisation: per key one partial dot product, log2(LPK) shuffles,
//     one exp2, one scaled accumulate; four K and four V loads are in flight per lane;
//   * the states merge at the end of a row segment: across the lane groups of a warp by
//     shuffles, across the 8 warps of a CTA through shared memory;
//   * work is dealt in equal byte ranges, not rows (see decode_stream_kernel): one wave of
//     resident CTAs streams the whole launch, whether it has 8 rows of 32768 keys or 2048
//     rows of 1024; rows cut between CTAs are finished by a small fix-up kernel from states
//     parked in a scratch buffer that belongs to the launching stream (a few hundred KiB,
//     allocated the first time a stream is used and kept).
// Anything the fast kernel does not take (head sizes other than 16/32/64/128, rows that are
// not 16-byte aligned) runs decode_generic_kernel: one CTA per row, scores kept in shared
// memory -- still on the GPU.
#include <cooperative_groups.h>

#include <stdlib.h>

#include <map>
#include <type_traits>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace b200 {
namespace decode {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int UNROLL = 4;         // K loads (and V loads) in flight per lane
// resident CTAs per SM the register budget is held to: 8 elements per lane need about 80
// registers, 4 elements about 64
template <typename T> constexpr int ctas_per_sm() { return sizeof(T) == 4 ? 4 : 3; }
constexpr int kGenericMaxKeys = 48 * 1024;  // scores of one row in shared memory

struct Params {
  const void *q, *k, *v;
  void *out;
  int64_t q_row, o_row;            // element strides of q / out rows
  int64_t k_head, k_row, v_head, v_row;
  int N, group;
  float scale;                     // multiplies q k
  int64_t units, units_per_row;    // streaming kernel: work units (UNIT_KEYS keys of one row)
  float *scratch;                  // [ctas][2][D + 2] softmax states of rows cut between CTAs
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x: the approximate unit is below half an ulp of a 16-bit output; fp32 outputs take exp2f
template <typename T> __device__ __forceinline__ float pow2(float x) { return ex2f(x); }
template <> __device__ __forceinline__ float pow2<float>(float x) { return exp2f(x); }

// 16 bytes -> floats.  16-bit pairs are widened with one shift / mask (bf16) or one packed
// conversion (f16) per word.
template <typename T, int VEC>
__device__ __forceinline__ void unpack(const uint4 &raw, float (&f)[VEC]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(w[i]);
  } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 pair = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
      f[2 * i] = pair.x;
      f[2 * i + 1] = pair.y;
    }
  }
}

// merge (m_b, l_b, acc_b) into (m, l, acc); either side may be empty (m = -inf, l = 0)
template <typename T, int VEC>
__device__ __forceinline__ void merge_state(float &m, float &l, float (&acc)[VEC], float m_b,
                                            float l_b, const float (&acc_b)[VEC]) {
  const float m_n = fmaxf(m, m_b);
  const float fa = (m == -INFINITY) ? 0.f : pow2<T>(m - m_n);
  const float fb = (m_b == -INFINITY) ? 0.f : pow2<T>(m_b - m_n);
  l = l * fa + l_b * fb;
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = acc[i] * fa + acc_b[i] * fb;
  m = m_n;
}

// Work decomposition of the streaming kernel: the key axis of every row is cut into units
// of UNIT_KEYS keys, all units of all rows form one sequence, and CTA c of G takes the
// contiguous range [c*U/G, (c+1)*U/G) of it -- every CTA streams the same number of bytes
// whatever the number of rows, and one wave of resident CTAs covers the whole launch.  A
// range is walked row by row ("segments").  A segment that is a whole row is finished on the
// spot; a range that starts or ends inside a row leaves that segment's softmax state
// (max, sum, D accumulators) in the scratch slot (c, 0) resp. (c, 1), and the fix-up kernel
// merges the pieces of every row that was cut -- at most two per CTA.
constexpr int UNIT_KEYS = 128;

__host__ __device__ inline int64_t range_begin(int64_t c, int64_t units, int64_t ctas) {
  return c * units / ctas;
}

template <typename T, int D>
__global__ void __launch_bounds__(THREADS, ctas_per_sm<T>())
decode_stream_kernel(const Params p) {
  constexpr int VEC = 16 / (int)sizeof(T);   // elements per lane
  constexpr int LPK = D / VEC;               // lanes per key row
  constexpr int KPL = 32 / LPK;              // keys per warp load
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head size");
  __shared__ float warp_state[WARPS][D + 2];  // per warp: m, l, acc[D]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int part = lane % LPK;   // which 16 bytes of the row
  const int sub = lane / LPK;    // which key of a warp load
  const int64_t u_begin = range_begin(blockIdx.x, p.units, gridDim.x);
  const int64_t u_end = range_begin(blockIdx.x + 1, p.units, gridDim.x);

  for (int64_t u = u_begin; u < u_end;) {
    const int b = (int)(u / p.units_per_row);
    const int64_t row_u0 = (int64_t)b * p.units_per_row;
    const int64_t seg_end = min(u_end, row_u0 + p.units_per_row);
    const int key0 = (int)(u - row_u0) * UNIT_KEYS;
    const int key1 = min(p.N, (int)(seg_end - row_u0) * UNIT_KEYS);
    const bool from_row_start = u == row_u0;
    const bool whole_row = from_row_start && seg_end == row_u0 + p.units_per_row;
    const int kv = b / p.group;
    const T *q = reinterpret_cast<const T *>(p.q) + (int64_t)b * p.q_row;
    const T *kbase = reinterpret_cast<const T *>(p.k) + (int64_t)kv * p.k_head;
    const T *vbase = reinterpret_cast<const T *>(p.v) + (int64_t)kv * p.v_head;

    float qf[VEC];
    {
      const uint4 raw = *reinterpret_cast<const uint4 *>(q + part * VEC);
      unpack<T, VEC>(raw, qf);
      const float s = p.scale * 1.4426950408889634f;  // scores in the log2 domain
#pragma unroll
      for (int i = 0; i < VEC; ++i) qf[i] *= s;
    }
    float m = -INFINITY, l = 0.f, acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;

    // The loop is software-pipelined: the K loads of step i+1 are issued as soon as the
    // dot products of step i have consumed the K registers, the V loads of step i+1 as soon
    // as the accumulation has consumed the V registers, so loads are in flight during all of
    // the arithmetic.
    constexpr int STEP = UNROLL * KPL;  // keys per warp per step
    uint4 kr[UNROLL], vr[UNROLL];
    auto load_rows = [&](const T *rows, int64_t pitch, int base, uint4 (&dst)[UNROLL]) {
#pragma unroll
      for (int t = 0; t < UNROLL; ++t) {
        const int key = base + t * KPL + sub;
        dst[t] = key < key1 ? ld_stream16(rows + (int64_t)key * pitch + part * VEC)
                            : make_uint4(0, 0, 0, 0);
      }
    };
    int base = key0 + warp * STEP;
    if (base < key1) {
      load_rows(kbase, p.k_row, base, kr);
      load_rows(vbase, p.v_row, base, vr);
    }
    for (; base < key1; base += WARPS * STEP) {
      const int next = base + WARPS * STEP;
      float s[UNROLL];
#pragma unroll
      for (int t = 0; t < UNROLL; ++t) {
        float kf[VEC];
        unpack<T, VEC>(kr[t], kf);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) dot = fmaf(qf[i], kf[i], dot);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        s[t] = (base + t * KPL + sub < key1) ? dot : -INFINITY;
      }
      if (next < key1) load_rows(kbase, p.k_row, next, kr);
      float m_n = m;
#pragma unroll
      for (int t = 0; t < UNROLL; ++t) m_n = fmaxf(m_n, s[t]);
      if (m_n > -INFINITY) {  // at least one key so far
        const float alpha = (m == -INFINITY) ? 0.f : pow2<T>(m - m_n);
        l *= alpha;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] *= alpha;
#pragma unroll
        for (int t = 0; t < UNROLL; ++t) {
          const float pt = pow2<T>(s[t] - m_n);  // 0 for a key past the end
          float vf[VEC];
          unpack<T, VEC>(vr[t], vf);
          l += pt;
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc[i] = fmaf(pt, vf[i], acc[i]);
        }
        m = m_n;
      }
      if (next < key1) load_rows(vbase, p.v_row, next, vr);
    }

    // lane groups of the warp: afterwards every lane group holds the warp's state for its
    // own VEC columns
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
      const float m_b = __shfl_xor_sync(0xffffffffu, m, o);
      const float l_b = __shfl_xor_sync(0xffffffffu, l, o);
      float acc_b[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc_b[i] = __shfl_xor_sync(0xffffffffu, acc[i], o);
      merge_state<T, VEC>(m, l, acc, m_b, l_b, acc_b);
    }
    if (sub == 0) {
      if (part == 0) {
        warp_state[warp][0] = m;
        warp_state[warp][1] = l;
      }
#pragma unroll
      for (int i = 0; i < VEC; ++i) warp_state[warp][2 + part * VEC + i] = acc[i];
    }
    __syncthreads();
    // warps of the CTA: thread d < D owns column d
    const int d = threadIdx.x;
    if (d < D) {
      float cm = -INFINITY, cl = 0.f, cacc[1] = {0.f};
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float acc_b[1] = {warp_state[w][2 + d]};
        merge_state<T, 1>(cm, cl, cacc, warp_state[w][0], warp_state[w][1], acc_b);
      }
      if (whole_row) {
        T *out = reinterpret_cast<T *>(p.out) + (int64_t)b * p.o_row;
        out[d] = io<T>::store(cacc[0] / cl);
      } else {
        float *slot = p.scratch + ((int64_t)blockIdx.x * 2 + (from_row_start ? 1 : 0)) * (D + 2);
        slot[2 + d] = cacc[0];
        if (d == 0) {
          slot[0] = cm;
          slot[1] = cl;
        }
      }
    }
    __syncthreads();  // warp_state is rewritten by the next segment
    u = seg_end;
  }
}

// Rows that were cut between CTAs: the CTA in whose range such a row starts merges its own
// slot 1 with slot 0 of every following CTA that continues the row, and writes the row.
template <typename T, int D>
__global__ void __launch_bounds__(D < 32 ? 32 : D)
decode_fixup_kernel(const Params p, int ctas) {
  const int c = (int)blockIdx.x, d = (int)threadIdx.x;
  const int64_t u_begin = range_begin(c, p.units, ctas), u_end = range_begin(c + 1, p.units, ctas);
  if (u_end <= u_begin || d >= D) return;
  const int b = (int)((u_end - 1) / p.units_per_row);        // the row this range ends in
  const int64_t row_u0 = (int64_t)b * p.units_per_row, row_u1 = row_u0 + p.units_per_row;
  if (u_end >= row_u1 || row_u0 < u_begin) return;          // not cut here / started earlier
  const float *slot = p.scratch + ((int64_t)c * 2 + 1) * (D + 2);
  float m = slot[0], l = slot[1], acc[1] = {slot[2 + d]};
  for (int n = c + 1; n < ctas && range_begin(n, p.units, ctas) < row_u1; ++n) {
    if (range_begin(n + 1, p.units, ctas) <= range_begin(n, p.units, ctas)) continue;
    const float *next = p.scratch + (int64_t)n * 2 * (D + 2);
    const float acc_b[1] = {next[2 + d]};
    merge_state<T, 1>(m, l, acc, next[0], next[1], acc_b);
  }
  T *out = reinterpret_cast<T *>(p.out) + (int64_t)b * p.o_row;
  out[d] = io<T>::store(acc[0] / l);
}

// One CTA per row, any head size: scores of the row in shared memory, then the weighted
// sum with one thread per output column.
template <typename T>
__global__ void __launch_bounds__(THREADS)
decode_generic_kernel(const Params p, int D) {
  extern __shared__ float scores[];  // N scores + 32 floats of reduction scratch
  float *scratch = scores + p.N;
  const int b = (int)blockIdx.x, kv = b / p.group;
  const T *q = reinterpret_cast<const T *>(p.q) + (int64_t)b * p.q_row;
  const T *kbase = reinterpret_cast<const T *>(p.k) + (int64_t)kv * p.k_head;
  const T *vbase = reinterpret_cast<const T *>(p.v) + (int64_t)kv * p.v_head;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float mx = -INFINITY;
  for (int key = threadIdx.x; key < p.N; key += THREADS) {
    const T *kr = kbase + (int64_t)key * p.k_row;
    float dot = 0.f;
    for (int i = 0; i < D; ++i) dot = fmaf(io<T>::load(q[i]), io<T>::load(kr[i]), dot);
    dot *= p.scale;
    scores[key] = dot;
    mx = fmaxf(mx, dot);
  }
  mx = warp_max(mx);
  if (lane == 0) scratch[warp] = mx;
  __syncthreads();
  mx = scratch[0];
  for (int w = 1; w < WARPS; ++w) mx = fmaxf(mx, scratch[w]);
  __syncthreads();
  float sum = 0.f;
  for (int key = threadIdx.x; key < p.N; key += THREADS) {
    const float e = expf(scores[key] - mx);
    scores[key] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) scratch[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < WARPS; ++w) sum += scratch[w];
  T *out = reinterpret_cast<T *>(p.out) + (int64_t)b * p.o_row;
  for (int d = threadIdx.x; d < D; d += THREADS) {
    float acc = 0.f;
    for (int key = 0; key < p.N; ++key)
      acc = fmaf(scores[key], io<T>::load(vbase[(int64_t)key * p.v_row + d]), acc);
    out[d] = io<T>::store(acc / sum);
  }
}

// Softmax states of rows cut between CTAs: [ctas][2][D + 2] floats, at most
// kMaxResident * 2 * 130.  One buffer per (device, stream), allocated the first time that
// stream launches a decode and kept: launches on one stream are ordered, so they can share
// it; launches on different streams never do.
constexpr int kMaxResident = 4 * 160;
static std::mutex g_scratch_lock;
static std::map<std::pair<int, cudaStream_t>, float *> g_scratch;

static float *stream_scratch(cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> guard(g_scratch_lock);
  auto key = std::make_pair(dev, stream);
  auto found = g_scratch.find(key);
  if (found != g_scratch.end()) return found->second;
  void *ptr = nullptr;
  if (cudaMalloc(&ptr, (size_t)kMaxResident * 2 * (128 + 2) * sizeof(float)) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  g_scratch[key] = reinterpret_cast<float *>(ptr);
  return g_scratch[key];
}

template <typename T, int D>
static int launch_stream(const Params &p, int rows, cudaStream_t stream) {
  Params ps = p;
  ps.units_per_row = (p.N + UNIT_KEYS - 1) / UNIT_KEYS;
  ps.units = ps.units_per_row * rows;
  const int64_t resident = (int64_t)ctas_per_sm<T>() * sm_count();
  int ctas = (int)(ps.units < resident ? ps.units : resident);
  if (ctas > kMaxResident) ctas = kMaxResident;
  ps.scratch = stream_scratch(stream);
  if (ps.scratch == nullptr) return fail(B200_RESOURCE, "no scratch for the decode kernel");
  decode_stream_kernel<T, D><<<ctas, THREADS, 0, stream>>>(ps);
  cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess && ctas > 1) {
    decode_fixup_kernel<T, D><<<ctas, D < 32 ? 32 : D, 0, stream>>>(ps, ctas);
    err = cudaGetLastError();
  }
  B200_CUDA_OK(err);
  return B200_OK;
}

template <typename T>
static int launch_typed(const Params &p, int rows, int D, bool aligned, cudaStream_t stream) {
  const bool fast = aligned && (D == 16 || D == 32 || D == 64 || D == 128) &&
                    D * (int)sizeof(T) <= 512 && D * (int)sizeof(T) >= 16;
  if (!fast) {
    B200_REQUIRE(p.N <= kGenericMaxKeys, "N_CTX %d exceeds the generic decode path's limit %d",
                 p.N, kGenericMaxKeys);
    const size_t smem = (size_t)(p.N + 32) * sizeof(float);
    static bool configured[64] = {false};
    int dev = 0;
    B200_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
      B200_CUDA_OK(cudaFuncSetAttribute(decode_generic_kernel<T>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)((kGenericMaxKeys + 32) * sizeof(float))));
      configured[dev] = true;
    }
    decode_generic_kernel<T><<<rows, THREADS, smem, stream>>>(p, D);
    B200_CUDA_OK(cudaGetLastError());
    return B200_OK;
  }
  switch (D) {
    case 16: return launch_stream<T, 16>(p, rows, stream);
    case 32: return launch_stream<T, 32>(p, rows, stream);
    case 64: return launch_stream<T, 64>(p, rows, stream);
    default: return launch_stream<T, 128>(p, rows, stream);
  }
}

}  // namespace decode

// Called by b200_stream_destroy before the stream goes away: the decode scratch kept for
// (current device, stream) is freed, so streams created per use do not accumulate buffers and
// a later stream that gets the same handle value starts without one.
void release_stream_scratch(cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return;
  float *ptr = nullptr;
  {
    std::lock_guard<std::mutex> guard(decode::g_scratch_lock);
    auto found = decode::g_scratch.find(std::make_pair(dev, stream));
    if (found == decode::g_scratch.end()) return;
    ptr = found->second;
    decode::g_scratch.erase(found);
  }
  (void)cudaStreamSynchronize(stream);  // its last decode may still be reading the buffer
  (void)cudaFree(ptr);
}
}  // namespace b200

extern "C" int b200_attn_decode(const b200_tensor *q, const b200_tensor *k, const b200_tensor *v,
                                b200_tensor *out, float scale, void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(q, "q", 2)) || (st = check_tensor(k, "k", 3)) ||
      (st = check_tensor(v, "v", 3)) || (st = check_tensor(out, "out", 2)))
    return st;
  B200_REQUIRE(is_float_io(q->dtype), "q: dtype %u is not f16/bf16/f32", q->dtype);
  B200_REQUIRE(k->dtype == q->dtype && v->dtype == q->dtype && out->dtype == q->dtype,
               "q/k/v/out dtypes differ");
  const int64_t B = q->shape[0], D = q->shape[1], BK = k->shape[0], N = k->shape[1];
  B200_REQUIRE(out->shape[0] == B && out->shape[1] == D, "out must be [B, D] like q");
  B200_REQUIRE(k->shape[2] == D && v->shape[0] == BK && v->shape[1] == N && v->shape[2] == D,
               "k and v must both be [B / group, N, D]");
  B200_REQUIRE(BK > 0 ? B % BK == 0 : B == 0, "query rows %lld are not a multiple of K/V heads %lld",
               (long long)B, (long long)BK);
  B200_REQUIRE(q->stride[1] == 1 && k->stride[2] == 1 && v->stride[2] == 1 && out->stride[1] == 1,
               "last-dim stride must be 1");
  B200_REQUIRE(D >= 1 && D <= 512, "head_dim %lld out of range", (long long)D);
  B200_REQUIRE(B < 65536 && N < (1 << 30), "rows or N_CTX out of range");
  B200_REQUIRE(scale == scale && scale > 0.f, "scale must be positive");
  if (B == 0) return B200_OK;
  B200_REQUIRE(N > 0, "N_CTX must be positive: softmax over no keys is undefined");

  decode::Params p;
  p.q = q->data; p.k = k->data; p.v = v->data; p.out = out->data;
  p.q_row = q->stride[0]; p.o_row = out->stride[0];
  p.k_head = k->stride[0]; p.k_row = k->stride[1];
  p.v_head = v->stride[0]; p.v_row = v->stride[1];
  p.N = (int)N; p.group = (int)(B / BK); p.scale = scale;
  p.units = 0; p.units_per_row = 0; p.scratch = nullptr;
  const size_t es = dtype_size(q->dtype);
  auto aligned16 = [&](const void *ptr, std::initializer_list<int64_t> strides) {
    if ((uintptr_t)ptr % 16 != 0) return false;
    for (int64_t s : strides)
      if ((s * (int64_t)es) % 16 != 0) return false;
    return true;
  };
  const bool aligned = aligned16(q->data, {q->stride[0]}) &&
                       aligned16(k->data, {k->stride[0], k->stride[1]}) &&
                       aligned16(v->data, {v->stride[0], v->stride[1]});
  cudaStream_t s = (cudaStream_t)stream;
  if (q->dtype == B200_DTYPE_FLOAT32) return decode::launch_typed<float>(p, (int)B, (int)D, aligned, s);
  if (q->dtype == B200_DTYPE_FLOAT16) return decode::launch_typed<__half>(p, (int)B, (int)D, aligned, s);
  return decode::launch_typed<__nv_bfloat16>(p, (int)B, (int)D, aligned, s);
}
