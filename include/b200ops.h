/* b200ops.h -- the C ABI of the sm_100a operator library (libb200ops.so).
 *
 * This is the single declaration of everything that crosses between the
 * Python host (ctypes) and the CUDA kernels.  It plays the role that
 * a100c/runtime/a100rt.h:1-218 plays between the a100c runtime and its
 * generated operator programs: one header, plain C types, layout pins.
 *
 * Conventions
 *   - every entry point validates its descriptors and RETURNS a status; it
 *     never aborts, traps or launches a kernel on a rejected descriptor
 *     (the "rejected bundle is never written" rule of
 *     a100c/runtime/bundle.c:1-9);
 *   - the caller owns all memory; `data` pointers are DEVICE pointers unless
 *     a function says otherwise; strides are in ELEMENTS;
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous
 *     and no entry point synchronises unless it says so;
 *   - tensor-core kernels bound every device-side wait; when a wait expires
 *     the kernel records B200_TIMEOUT in the library's per-device status
 *     word, which b200_last_device_status() returns after the stream drains.
 */
#ifndef B200OPS_H
#define B200OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

/* Status codes.  0..6 keep the numbering of the a100c process exit codes
 * (a100c/runtime/a100rt.h:49-55); 7.. are additions of this library. */
enum b200_status {
  B200_OK = 0,
  B200_USAGE = 2,           /* argument outside the contract (null, bad enum) */
  B200_REJECTED = 3,        /* descriptor violates a precondition */
  B200_RESOURCE = 4,        /* allocation / CUDA runtime failure */
  B200_REPEAT_MISMATCH = 5, /* repeats produced different outputs */
  B200_SYNC = 6,            /* stream / device synchronisation failed */
  B200_TIMEOUT = 7,         /* a bounded device-side wait expired */
  B200_UNSUPPORTED = 8      /* valid request this build has no kernel for */
};

/* dtype codes: the a100rt_dtype numbering (a100c/runtime/a100rt.h:58-72). */
enum b200_dtype {
  B200_DTYPE_BOOL = 1,
  B200_DTYPE_INT8 = 2,
  B200_DTYPE_UINT8 = 3,
  B200_DTYPE_INT16 = 4,
  B200_DTYPE_UINT16 = 5,
  B200_DTYPE_INT32 = 6,
  B200_DTYPE_UINT32 = 7,
  B200_DTYPE_INT64 = 8,
  B200_DTYPE_UINT64 = 9,
  B200_DTYPE_FLOAT16 = 10,
  B200_DTYPE_BFLOAT16 = 11,
  B200_DTYPE_FLOAT32 = 12,
  B200_DTYPE_FLOAT64 = 13
};

/* One tensor argument (the role of struct a100rt_view,
 * a100c/runtime/a100rt.h:79-92).  Dimensions beyond ndim are ignored. */
typedef struct b200_tensor {
  void *data;
  int64_t shape[4];
  int64_t stride[4]; /* in elements */
  uint32_t dtype;    /* enum b200_dtype */
  uint32_t ndim;
} b200_tensor;

typedef struct b200_device_props {
  char name[64];
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int32_t l2_bytes;
  int64_t hbm_bytes;
  int32_t smem_per_block_optin;
  int32_t clock_khz;
} b200_device_props;

/* GEMM epilogue selector */
enum b200_act {
  B200_ACT_NONE = 0,
  B200_ACT_GELU_ERF = 1,  /* 0.5 z (1 + erf(z / sqrt 2)), triton_linear_activation.py:46 */
  B200_ACT_GELU_TANH = 2, /* 0.5 z (1 + tanh(0.79788456 (z + 0.044715 z^3))), geglu_tanh_triton.py:32-36 */
  B200_ACT_LEAKY_RELU = 3,/* z >= 0 ? z : 0.01 z, matmul_triton2.py:77 */
  B200_ACT_SWIGLU = 4     /* silu(a@b) * (a@b2): two B operands, swiglu_fwd.py:34-36 over two matmuls */
};

enum b200_mask {
  B200_MASK_NONE = 0,
  B200_MASK_CAUSAL_MOD = 1 /* keep col <= (row_offset + row) % n_cols, -inf elsewhere */
};

/* ---- library / device ------------------------------------------------- */
int b200_abi_version(void);
/* Text for a status code (the role of a100rt_reject_reason,
 * a100c/runtime/bundle.c:59-88). */
const char *b200_status_string(int status);
/* Detail of the most recent non-OK return on this host thread. */
const char *b200_last_error(void);
/* Replaces the device discovery of ops/harness/opslib/devices/cuda.py:329-345. */
int b200_device_query(int device, b200_device_props *out);
int b200_set_device(int device);
/* Reads (and clears) the per-device status word that kernels with bounded
 * waits write; synchronises `stream` first. */
int b200_last_device_status(void *stream);

/* CUDA graphs: launches enqueued on `stream` between begin and end are recorded instead of
 * run, and the instantiated graph replays them with one call -- for loops of short kernels
 * whose cost is launch latency (the reference has no counterpart: its runtime launches one
 * program per process).  `stream` must come from b200_stream_create.  Other streams join a
 * capture through b200_event_record on the capturing stream + b200_stream_wait_event on
 * theirs, and must be joined back the same way before the capture ends.  Every operator
 * used inside a capture must have run once on this device before -- b200_attn_decode and the
 * GEMM entry points once on the capturing stream, with the shapes of the capture: their scratch
 * (decode: softmax states of rows cut between CTAs; GEMM: partial sums of a last wave that is
 * split along K) is kept per stream -- (first calls set kernel attributes and allocate the
 * status word / scratch, which a capture forbids); the entry
 * points that synchronise (memcpy with NULL stream, *_sync, b200_last_device_status,
 * b200_allclose_f32) cannot be captured. */
int b200_stream_wait_event(void *stream, void *event);
int b200_graph_begin_capture(void *stream);
int b200_graph_end_capture(void *stream, void **graph_exec);
int b200_graph_launch(void *graph_exec, void *stream);
int b200_graph_destroy(void *graph_exec);

/* Self-test of the bounded device-side wait: launches one CTA whose two waiters wait on a
 * barrier that nothing completes.  The wait expires after its limit (about 2 s), records
 * B200_TIMEOUT in the status word, and the kernel returns normally.  *gave_up = 1 when both
 * waiters gave up as they must; the next b200_last_device_status() then reports
 * B200_TIMEOUT (site 31) and clears it.  No reference counterpart (the reference's runtime
 * has no device-side waits); it exists so that the failure path can be exercised without a
 * fault. */
int b200_wait_selftest(unsigned int *gave_up, void *stream);

/* ---- memory, streams, events (torch-free Device plumbing; replaces the
 *      cudaMalloc / pinned staging / event timer of
 *      ops/harness/opslib/devices/cuda.py:71-123, 138-167, 186-262) -------- */
int b200_malloc(void **out, size_t bytes);
int b200_free(void *ptr);
/* Page-locked host memory.  It is addressable from the device under unified addressing, so
 * the row-wise and elementwise entry points also take it as operand memory: the kernel then
 * loads and stores over PCIe with no staging copy (tensor-map operands -- GEMM, attention --
 * must be in device memory). */
int b200_malloc_host(void **out, size_t bytes);
int b200_free_host(void *ptr);
int b200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream);
int b200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream);
int b200_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream);
int b200_memset(void *dst, int value, size_t bytes, void *stream);
int b200_stream_create(void **out);
int b200_stream_destroy(void *stream);
int b200_stream_sync(void *stream);
int b200_device_sync(void);
int b200_event_create(void **out);
int b200_event_destroy(void *event);
int b200_event_record(void *event, void *stream);
int b200_event_elapsed_ms(void *start, void *stop, float *ms); /* syncs stop */

/* ---- operators -------------------------------------------------------- */

/* RMSNorm forward.  Replaces rms_layernorm_forward_kernel
 * (ops/suite/perf/fast_rms_layernorm.py:19-44): per row
 * inv = rsqrt(mean(x^2) + eps); y = x * inv * w; rinv[row] = inv.
 * x,y: [rows, cols] with unit column stride; w: [cols]; rinv: [rows] or NULL.
 * x/y/w/rinv share one dtype (f32, f16 or bf16); accumulation is fp32. */
int b200_rmsnorm_fwd(const b200_tensor *x, const b200_tensor *w,
                     b200_tensor *y, b200_tensor *rinv, float eps,
                     void *stream);

/* The same with the weight taken as (w + gamma_offset): gamma_offset = 1 is the
 * zero-centred gamma of rmsnorm_fwd_loop_kernel (ops/suite/dev/rmsnorm_fwd_loop_kernel.py:10-34). */
int b200_rmsnorm_fwd_ex(const b200_tensor *x, const b200_tensor *w, b200_tensor *y,
                        b200_tensor *rinv, float eps, float gamma_offset, void *stream);

/* Row softmax with an optional index-computed mask.  Replaces softmax_kernel
 * (ops/suite/perf/softmax.py:20-31) and, with B200_MASK_CAUSAL_MOD, the
 * masking expression of ops/suite/perf/attn_fwd_causal.py:46-47 applied to a
 * row softmax.  x,y: contiguous [rows, cols], same dtype (f32/f16/bf16);
 * max and sum are fp32.  row_offset is the global index of local row 0 so a
 * row shard masks by its global row. */
int b200_softmax_fwd(const b200_tensor *x, b200_tensor *y, int mask_kind,
                     int64_t row_offset, void *stream);

/* Softmax variants over contiguous [rows, cols]: with `mul`, y = softmax(x) * mul
 * (softmax_mul_kernel, ops/suite/perf/softmax_mul.py:21-32); with log_input, y =
 * softmax(log x) and a NaN in log x makes its row NaN (softmax_log_kernel,
 * ops/suite/perf/softmax_log.py:20-40).  mul may be NULL. */
int b200_softmax_variant(const b200_tensor *x, const b200_tensor *mul, b200_tensor *y,
                         int log_input, void *stream);

/* y[row, p] = x[row, p / repeat] - logsumexp over p in [0, y.cols)
 * (fused_repeat_interleave_log_softmax_kernel,
 * ops/suite/perf/fused_repeat_interleave_log_softmax.py:19-31). */
int b200_repeat_log_softmax(const b200_tensor *x, b200_tensor *y, int repeat, void *stream);

/* Flat elementwise operators of the GELU family; a, b, out are 1-D contiguous. */
enum b200_ewise {
  B200_EW_GELU_ERF = 1,             /* gelu_kernel, ops/suite/perf/gelu.py:21-27 */
  B200_EW_ADD_GELU_ERF = 2,         /* gelu(a + p0 * b): add_gelu_kernel, ops/suite/perf/add_gelu.py:21-30 */
  B200_EW_GEGLU_TANH = 3,           /* gelu_tanh(a) * b: geglu_tanh_forward_kernel, ops/suite/perf/geglu_tanh_triton.py:19-37 */
  B200_EW_BIAS_SCALE_CLAMP_GELU = 4 /* gelu(clamp((a + b[i % len(b)]) * p0, p1, p2)): epilogue_kernel, ops/suite/dev/epilogue_kernel.py:24-32 */
};
int b200_elementwise(int op, const b200_tensor *a, const b200_tensor *b, b200_tensor *out,
                     float p0, float p1, float p2, void *stream);

/* C = act(A @ B + bias).  Replaces matmul_kernel (ops/suite/perf/matmul.py:20-38)
 * and linear_act_kernel (ops/suite/perf/triton_linear_activation.py:27-49).
 * A [M,K] row-major, B [K,N] row-major, C [M,N] row-major; A/B are f16 or
 * bf16 (same type), accumulation fp32, C is A's type or f32; bias [N] may be
 * NULL and is f32 or A's type.  b2 is the second B operand of
 * B200_ACT_SWIGLU (NULL otherwise).  Shapes whose row pitches are not
 * multiples of 16 bytes take a CUDA-core kernel instead of the tensor-core
 * path; nothing is computed on the host. */
int b200_gemm_bias_act(const b200_tensor *a, const b200_tensor *b,
                       const b200_tensor *b2, const b200_tensor *bias,
                       b200_tensor *c, int act, void *stream);

/* y = act(x @ w^T + bias) with the weight given as [N, K] rows of K -- the layout of a linear
 * layer's weight, and of a B operand passed with stride_bk = 1 (the "general strides" of
 * matmul_kernel, ops/suite/perf/matmul_triton2.py:27-30, and the transposed weight of
 * linear_act_kernel, ops/suite/perf/triton_linear_activation.py:28-30).  Same epilogues and
 * tensor-core kernels as b200_gemm_bias_act (the weight is fed as a K-major operand, nothing
 * is transposed in memory); B200_ACT_SWIGLU is not available here. */
int b200_linear_bias_act(const b200_tensor *x, const b200_tensor *w, const b200_tensor *bias,
                         b200_tensor *y, int act, void *stream);

/* mins[m] = min(mins[m], min_n GroupNorm(x @ w + bias)[m, n]): a GEMM whose epilogue
 * normalises groups of group_size consecutive columns (mean / variance inside the group,
 * gamma, beta) and keeps only the minimum of each row.  Replaces fused_gemm_gn_min_kernel
 * (ops/suite/dev/fused_gemm_gn_min_kernel.py:26-59).  x [M,K], w [K,N], bias / gamma / beta
 * [N] (bias may be NULL), mins f32 [M] (set it to +inf first: the kernel merges with an
 * atomic minimum, as the reference does); group_size 8 / 16 / 32 / 64 dividing N (32 only on
 * the CUDA-core path that fp32 operands take).  The [M,N] product is never written. */
int b200_gemm_groupnorm_rowmin(const b200_tensor *x, const b200_tensor *w,
                               const b200_tensor *bias, const b200_tensor *gamma,
                               const b200_tensor *beta, b200_tensor *mins, int group_size,
                               float eps, void *stream);

/* out[k,n] = b[k,n] * scale[n]: int8 weights to floats.  Replaces dequantize_kernel
 * (ops/suite/perf/dequantize_matmul.py:27-40).  b int8 [K,N], scale [N] and out [K,N] in one
 * float type, unit column strides. */
int b200_dequantize_cols(const b200_tensor *b, const b200_tensor *scale, b200_tensor *out,
                         void *stream);

/* out = rsqrt(mean(x^2, row) + eps) * ((x * g) @ w): RMS normalisation folded into a matmul.
 * Replaces rms_matmul_rbe_kernel (ops/suite/dev/rms_matmul_rbe.py:18-63).  x [M,K], g [K], w [K,N], out [M,N] (x's type or
 * f32).  Two small kernels write rinv[M] (f32) and g-scaled weights into caller-provided
 * scratch (scratch_w [K,N] in x's type, scratch_rinv f32 [>= M]); the tensor-core GEMM then
 * runs x @ scratch_w and multiplies each accumulator row by rinv in its epilogue, so the
 * normalised activations are never written. */
int b200_rms_matmul(const b200_tensor *x, const b200_tensor *g, const b200_tensor *w,
                    b200_tensor *out, float eps, b200_tensor *scratch_w,
                    b200_tensor *scratch_rinv, void *stream);

/* y = log_softmax(x @ w^T) over the output columns.  Replaces log_softmax_linear_kernel
 * (ops/suite/perf/log_softmax_linear.py:19-35): x [M,K], w [N,K] (a linear layer's weight:
 * rows of K), y [M,N] in x's type or f32, 1 <= N <= 256.  16-bit operands with 16-byte
 * aligned rows run the tensor-core GEMM with w fed as a K-major operand and the row
 * log-softmax done in the epilogue on the accumulator (no intermediate [M,N] matrix);
 * other operands take a CUDA-core kernel. */
int b200_linear_log_softmax(const b200_tensor *x, const b200_tensor *w, b200_tensor *y,
                            void *stream);

/* Attention forward.  Replaces attn_fwd_causal_kernel
 * (ops/suite/perf/attn_fwd_causal.py:19-57).  q,o: [Z,H,N,D], k,v: [Z,H_KV,N_K,D]
 * with unit last stride; H_KV divides H and query head h reads K / V head
 * h / (H / H_KV) (H_KV == H for the kernels above; fewer K / V heads is gqa_kernel,
 * ops/suite/dev/gqa.py:19-58).  N_K may differ from N (one sequence of
 * flash_varlen_fwd_kernel, ops/suite/dev/flash_varlen_fwd_kernel.py); the causal mask then
 * needs N_K >= N and is aligned to the last key: row i sees keys <= i + N_K - N (:138).  lse: [Z,H,N] f32 with unit last stride (any batch / head
 * strides) or NULL, natural log of the sum of
 * exp of the scaled masked scores (ops/suite/dev/flash_varlen_fwd_kernel.py:309). */
int b200_attn_fwd(const b200_tensor *q, const b200_tensor *k,
                  const b200_tensor *v, b200_tensor *o, b200_tensor *lse,
                  float scale, int causal, void *stream);

/* The same with the further modes of flash_varlen_fwd_kernel
 * (ops/suite/dev/flash_varlen_fwd_kernel.py), applied to the raw score S = q.k before the
 * softmax scale: soft-cap S = tanh(S * softcap) (:121-124; softcap 0: off); ALiBi (:76-81,
 * :125-133) with one f32 slope per head ([H]) or per batch and head ([Z,H]) or NULL -- causal:
 * S += slope / scale * (j - N_K + 1), otherwise S -= slope / scale * |j - N_K + N - i|; local
 * window (:56-61, :137-146; both sides >= 0, negative on both sides: off): row i sees keys
 * max(0, i + N_K - N - left) .. min(N_K - 1, i + N_K - N + right).  A row that sees no key gets
 * zeros and lse = +inf (:309-310).  With every mode off this is b200_attn_fwd; with any of
 * them on the CUDA-core kernel runs (at most 8192 keys).  The reference's own `ref` covers the
 * dense case only (:370-418): these modes are checked against a restatement of the kernel's
 * lines.  Paged K / V (:91-108): page_table int32 [Z, pages] or NULL; key j of batch z is
 * row j % block_size of physical page page_table[z][j / block_size], at page * page_stride +
 * (j % block_size) * k->stride[2] elements past the head's base k->data + head *
 * k->stride[1] -- for K and for V alike, as in the kernel; k->shape[2] = v->shape[2] is the
 * number of keys in use.  Dropout and the returned softmax are not taken. */
int b200_attn_fwd_modes(const b200_tensor *q, const b200_tensor *k, const b200_tensor *v,
                        b200_tensor *o, b200_tensor *lse, float scale, int causal,
                        float softcap, const b200_tensor *alibi_slopes, int window_left,
                        int window_right, const b200_tensor *page_table, int block_size,
                        int64_t page_stride, void *stream);

/* Causal sliding-window attention with a gate bias and an attention sink.  Replaces
 * parallel_attn_fwd_kernel (ops/suite/dev/parallel_attn_fwd_kernel.py; arithmetic :142-166):
 * logit[t,j] = scale * log2(e) * q[t].k[j] + g[t] - g[j] over max(0, t-window+1) <= j <= t,
 * softmax in base 2 with the sink's 2^(sink - max) added to the denominator, lse = max +
 * log2(denominator).  Token-major tensors: q [B,T,HQ,K], k [B,T,H,K], v [B,T,H,V],
 * o [B,T,HQ,V], g_cumsum [B,T,HQ] or NULL, sink_bias [HQ] or NULL, lse [B,T,HQ] (q's type or
 * f32) or NULL; window <= 0 means every earlier token.  K and V widths are free; this is a
 * CUDA-core kernel (at most 8192 keys per row). */
int b200_attn_window_fwd(const b200_tensor *q, const b200_tensor *k, const b200_tensor *v,
                         b200_tensor *o, const b200_tensor *g_cumsum,
                         const b200_tensor *sink_bias, b200_tensor *lse, float scale,
                         int window, void *stream);

/* Decode-side attention: one query row per (batch, head) against that head's K / V
 * cache.  Replaces flash_decode_kernel (ops/suite/perf/flash_decode.py:21-49):
 * out[b] = softmax(scale * K[b / group] q[b]) V[b / group].  q, out: [B, D]; k, v:
 * [B / group, N, D] with unit last stride (f16 / bf16 / f32, all the same type); group =
 * B / k->shape[0] query rows share one K / V head (1 for flash_decode; the grouped-query
 * layout of ops/suite/dev/gqa.py:29 otherwise).  Head sizes 16 / 32 / 64 / 128 with
 * 16-byte aligned rows take the streaming kernel (the keys of all rows dealt to one wave
 * of CTAs in equal ranges; rows cut between CTAs are merged by a second small kernel from
 * softmax states kept in a 650 KiB scratch buffer that the library allocates once per
 * (device, stream) on the first call and keeps); anything else takes a one-CTA-per-row kernel limited to
 * 49152 keys. */
int b200_attn_decode(const b200_tensor *q, const b200_tensor *k,
                     const b200_tensor *v, b200_tensor *out, float scale,
                     void *stream);

/* C = A @ B with the rows of C scattered to their owners: rows [k*rows_per_rank,
 * (k+1)*rows_per_rank) go to slot `slot` of c_rank[k], a buffer laid out
 * [world, rows_per_rank, N] in rank k's memory (a peer GPU's buffer mapped into this
 * process for k != slot).  The tensor-core GEMM's epilogue stores each finished tile
 * straight to its owner, so the reduce-scatter traffic of a row-sharded GEMM crosses
 * NVLink while the remaining tiles are still being computed.  c_like supplies dtype and
 * shape [M,N] (contiguous); its data pointer is ignored.  rows_per_rank must be a multiple
 * of 128.  The merge of per-worker partials in the reference is a100c/plan/stages.py:278-316;
 * it has no multi-device counterpart. */
int b200_gemm_scatter_rows(const b200_tensor *a, const b200_tensor *b,
                           const b200_tensor *c_like, void *const *c_rank, int world,
                           int slot, int64_t rows_per_rank, void *stream);

/* Sums the `world` slices of staging ([world, rows, cols], f16/bf16, fp32 accumulation,
 * one rounding to out_dtype, f16/bf16) and stores the result into rows [dst_row0, dst_row0 +
 * rows) of every y_rank[k] (contiguous [*, cols]; peer memory for k != this rank).  Together
 * with b200_gemm_scatter_rows this is the all-reduce of the tensor-parallel MLP; the caller
 * separates the two with a cross-rank barrier. */
int b200_reduce_slices_broadcast(const void *staging, uint32_t dtype, uint32_t out_dtype,
                                 int world, int64_t rows, int64_t cols, int64_t dst_row0,
                                 void *const *y_rank, void *stream);

/* All-reduce (sum) of partial results through NVSwitch.  in_multicast / out_multicast are
 * the multicast addresses of buffers that every rank allocated symmetrically and bound to a
 * multicast object (torch.distributed._symmetric_memory: handle.multicast_ptr); elements
 * [offset, offset + count) are reduced.  This rank loads the sum of all ranks' copies of its
 * share [offset + rank*count/world, offset + (rank+1)*count/world) of the partial (f16, bf16
 * or f32) with multimem.ld_reduce -- added in the switch in fp32 -- rounds it once to
 * out_dtype (f16 / bf16) and stores it to all ranks' copies of the result with multimem.st.
 * 16-bit partials may be reduced in place (out_multicast == in_multicast).  offset and
 * count/world must be multiples of 8 elements.  `ctas` > 0 limits the grid (for running
 * beside another kernel), 0 = default.
 * signal_pads == NULL: the caller puts a cross-rank barrier before the call (all partials
 * written) and after it (all shares published).  Otherwise signal_pads[k] is rank k's flag
 * array of b200_signal_pad_bytes() bytes (symmetric memory, zeroed once, mapped into this
 * process) and the kernel does both barriers itself: `epoch` must be the same on all ranks,
 * never 0, and grow by one per call on those pads; calls that share pads must be ordered on
 * one stream per rank, and every rank must launch the call (a rank that waits about two
 * seconds in vain records B200_TIMEOUT in the device status word and returns).  The merge of
 * per-worker partials in the reference is a100c/plan/stages.py:278-316 behind the stage
 * barrier of a100c/runtime/pool.c:187-190; it has no multi-device counterpart. */
int b200_multimem_allreduce(const void *in_multicast, uint32_t in_dtype, void *out_multicast,
                            uint32_t out_dtype, int64_t offset, int64_t count, int rank,
                            int world, void *const *signal_pads, uint32_t epoch, int ctas,
                            void *stream);
size_t b200_signal_pad_bytes(void);

/* The same all-reduce over plain peer memory (no multicast object needed): partial_rank[k] /
 * out_rank[k] are rank k's partial and result buffers (f16 / bf16; peer memory mapped into
 * this process for k != rank, e.g. handle.buffer_ptrs of symmetric memory).  This rank loads
 * its share of every rank's partial with 16-byte peer loads, adds them in fp32 in rank order
 * (every rank computes the same bits), rounds once and stores the result into every rank's
 * output.  In place (out_rank == partial_rank) is allowed.  offset / count / signal_pads /
 * epoch / ctas as for b200_multimem_allreduce. */
int b200_peer_allreduce(void *const *partial_rank, uint32_t in_dtype, void *const *out_rank,
                        uint32_t out_dtype, int64_t offset, int64_t count, int rank, int world,
                        void *const *signal_pads, uint32_t epoch, int ctas, void *stream);

/* The product C = A B (B as [K,N], 16-bit operands, the CTA-pair kernel: at least one wave
 * of 256 x 256 tiles) with PROGRESS COUNTERS, and the all-reduce that runs beside it: the
 * merge of the tensor-parallel MLP overlapped with the down-projection that produces the
 * partials, block of rows by block of rows.  No reference counterpart (the reference's
 * workers meet at a stage barrier, a100c/plan/stages.py:278-316).
 *
 * b200_gemm_progress: rows of C in blocks of rows_per_block (a multiple of 256; a block is a
 * raster group of the kernel, so the blocks finish in order).  counters: device memory of
 * b200_progress_words() 32-bit words, zero before the first launch (the all-reduce below puts
 * them back to zero): 16 counters, one count of the all-reduce CTAs that are done with them, one
 * word of padding, then 64-bit %globaltimer stamps written by the all-reduce kernel's first
 * CTA (its start; per block: counted complete, reduced).  Every epilogue warp adds one to its block's counter after its stores
 * of a tile, fenced at system scope.  targets[b] (host, max_blocks entries) receives the count
 * block b reaches; *blocks the number of blocks.  The kernel releases its programmatic
 * dependents as soon as its CTAs are set up.  REJECTED for shapes the CTA-pair kernel does not
 * take.
 *
 * b200_peer_allreduce_blocks: launched on the same stream directly behind it, as its
 * programmatic dependent (CTAs of 128 threads that fit beside the GEMM's).  total elements in
 * blocks of block_elems (= rows_per_block x row length; both multiples of 8 x world).  Per
 * block: wait for progress[b] >= targets[b], cross-rank barrier with epoch0 + b (signal_pads
 * as for b200_multimem_allreduce; the caller advances its epoch by the number of blocks), then
 * this rank's share of the block as in b200_peer_allreduce.  Only the last block's all-reduce
 * is left when the GEMM ends.  progress == NULL (then targets == NULL): no waiting on a
 * producer, an ordinary launch.  Every wait is bounded (B200_TIMEOUT, sites 40 - 42).  A
 * b200_gemm_progress launch is always followed by the all-reduce launch that reads its
 * counters and puts them back to zero: counters left standing would release the next
 * all-reduce before its GEMM has run. */
int b200_gemm_progress(const b200_tensor *a, const b200_tensor *b, b200_tensor *c,
                       int64_t rows_per_block, unsigned int *counters, unsigned int *targets,
                       int max_blocks, int *blocks, void *stream);
int b200_peer_allreduce_blocks(void *const *partial_rank, uint32_t in_dtype,
                               void *const *out_rank, uint32_t out_dtype, int64_t total,
                               int64_t block_elems, unsigned int *progress,
                               const unsigned int *targets, int rank, int world,
                               void *const *signal_pads, uint32_t epoch0, int ctas, void *stream);
/* The same through the switch (multicast pointers as for b200_multimem_allreduce). */
int b200_multimem_allreduce_blocks(const void *in_multicast, uint32_t in_dtype,
                                   void *out_multicast, uint32_t out_dtype, int64_t total,
                                   int64_t block_elems, unsigned int *progress,
                                   const unsigned int *targets, int rank, int world,
                                   void *const *signal_pads, uint32_t epoch0, int ctas,
                                   void *stream);
int b200_progress_words(void);

/* out = x * sigmoid(x) * y elementwise.  Replaces swiglu_fwd_kernel
 * (ops/suite/perf/swiglu_fwd.py:18-36).  [rows, cols], unit column stride. */
int b200_swiglu_fwd(const b200_tensor *x, const b200_tensor *y,
                    b200_tensor *out, void *stream);

/* On-device allclose of two same-shape contiguous f32 buffers.  Replaces
 * _allclose_kernel (ops/harness/opslib/devices/_cuda_compare.py:24-46).
 * result[0] = number of violating elements, max_abs_err = max |a-b| over
 * elements that are not exactly equal.  Synchronises `stream`. */
int b200_allclose_f32(const void *actual, const void *expected, int64_t count,
                      double rtol, double atol, int equal_nan,
                      int64_t *bad_count, double *max_abs_err, void *stream);

/* The same comparison as b200_allclose_f32 for callers that must not allocate device
 * memory: services whose memory pool owns the whole device (a cudaMalloc there fails or
 * fragments the pool), and latency-critical loops that cannot afford the device-wide
 * synchronisation an allocation and a free imply.  (No counterpart in the reference: its
 * device compare allocates three buffers per call, ops/harness/opslib/devices/cuda.py.)
 * It calls no cudaMalloc / cudaFree and no allocating library routine.  Its scratch is a
 * 128 KiB array built into the library image, present on every GPU that loads the
 * library until the process exits; it covers at most 134,201,344 elements per call
 * ((8192 - 1) blocks x 16384 elements) and a larger count is rejected with
 * B200_REJECTED.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and keeps it for the life of the
 * process (a cudaDeviceReset invalidates it); make that first call before starting any
 * stream capture.  All calls share the one array, which keeps the previous call's contents
 * (each call overwrites every slot it later reads, so nothing has to be cleared); two calls
 * that overlap on the GPU -- different streams, or several host threads -- race on it and
 * must be serialised by the caller.  Results match b200_allclose_f32.
 * The call BLOCKS the host: it copies the two result words back and synchronises `stream`
 * before it returns.  `stream` must therefore not be a stream that is being captured (nor
 * the legacy default stream while another thread holds a global-mode capture): pass a
 * stream of your own that is outside the capture. */
int b200_allclose_f32_static(const void *actual, const void *expected, int64_t count,
                             double rtol, double atol, int equal_nan,
                             int64_t *bad_count, double *max_abs_err, void *stream);

/* Runs `repeats` launches of an operator closure-free: restores `out` from
 * nothing, compares launch r>0 bitwise with launch 0 (the --repeats check of
 * a100c/runtime/main.c:117-152).  first/other: device buffers of `bytes`.
 * Returns B200_REPEAT_MISMATCH when they differ.  Synchronises `stream`. */
int b200_bitwise_equal(const void *first, const void *other, size_t bytes,
                       int *equal, void *stream);

#ifdef __cplusplus
}
#endif

/* Layout pins: the ctypes Structures in compiler_b200/runtime/abi.py mirror
 * these; a layout change must update both (a100rt.h:186-216 does the same for
 * the assembly stub). */
#ifdef __cplusplus
static_assert(sizeof(b200_tensor) == 80, "b200_tensor layout");
static_assert(offsetof(b200_tensor, shape) == 8, "b200_tensor.shape");
static_assert(offsetof(b200_tensor, stride) == 40, "b200_tensor.stride");
static_assert(offsetof(b200_tensor, dtype) == 72, "b200_tensor.dtype");
static_assert(sizeof(b200_device_props) == 96, "b200_device_props layout");
#endif

#endif /* B200OPS_H */
