/*
 * C ABI of libtlaloc_kernels.so: the B200 (sm_100a) kernels of Tlaloc's LLM
 * decode hot path.  Plain pointers and sizes only; every pointer named
 * "device" is a CUDA device pointer, `stream` is a cudaStream_t / CUstream
 * passed as void*, and every function only enqueues work on that stream (no
 * allocation, no synchronisation, no context switch), so it can be called
 * while the stream is being captured into a CUDA graph.
 *
 * Each function returns TLALOC_B200_OK or a negative status; the calling
 * thread's message is then available from tlaloc_b200_last_error().
 *
 * Reference interfaces these entry points stand in for (paths inside the
 * reference project) are cited at each declaration.  Bindings: the typed-FFI
 * handlers registered by TlalocRegisterKernels call these same functions; a
 * JVM binds them with java.lang.foreign downcalls exactly as
 * runtime-cuda/src/jvmMain/kotlin/io/tlaloc/runtime/cuda/CudaDriverFfm.kt:68-72
 * binds libcuda.
 */
#ifndef TLALOC_B200_H_
#define TLALOC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TLALOC_B200_ABI_VERSION 1

/* Status codes. */
#define TLALOC_B200_OK 0
#define TLALOC_B200_INVALID_ARGUMENT (-1) /* a shape/dtype the op's contract refuses; message names it */
#define TLALOC_B200_UNSUPPORTED (-2)      /* legal for the op, outside what these kernels cover */
#define TLALOC_B200_INTERNAL (-3)         /* a CUDA error; message carries cudaGetErrorString */

/* Element types, numbered as XLA_FFI_DataType (xla/ffi/api/c_api.h:239-260) so
 * the typed-FFI handlers pass a buffer's dtype through unchanged. */
#define TLALOC_B200_S8 2
#define TLALOC_B200_S32 4
#define TLALOC_B200_F32 11
#define TLALOC_B200_BF16 16
#define TLALOC_B200_F8E4M3FN 20 /* KV pools only: values stored clamped to +-448 and rounded to nearest even */

int tlaloc_b200_abi_version(void);

/* The calling thread's last error message ("" if none). Static storage per thread. */
const char* tlaloc_b200_last_error(void);

/*
 * Kernel set-up for the CURRENT device (opt-in dynamic shared memory; it is a
 * per-device attribute).  Call it once on every device the process uses, with
 * that device current, before the first launch that may run inside a CUDA graph
 * capture; launches outside a capture do it lazily.
 * Replaces: tlaloc_kernels::AllowMaxSharedMemory at XLA's INITIALIZE stage
 * (triton/kernels/kernel_setup.cuh:24-47, paged_attention.cu:1347-1350).
 */
int tlaloc_b200_init(void);

/*
 * Device-side health: 1 if a bounded wait inside a kernel (an mbarrier poll of a tensor-core projection or of the
 * paged-attention kernel's K/V tiles) has given up since the last call, 0 if none has, -1 on a CUDA error.
 * Synchronises with the device: a test and debugging aid, not for the per-step path.  A kernel whose wait gave up has freed its resources and returned;
 * its output is undefined.
 */
int tlaloc_b200_device_status(void);

/*
 * Parity mode, process-wide: while on, every operator below evaluates in the reference interpreter's own order
 * instead of the fast kernels' (the projections as with TLALOC_B200_GEMM_EXACT; paged attention with double
 * accumulators, positions in ascending order and one narrowing at the end, DxirInterpreter.kt:2049-2140; RMSNorm's
 * mean as a sequential f32 sum, :1450-1496,1791-1807; SiLU in double, :567-592), so that results equal the
 * interpreter's up to the last bit of the library exponential.  Slow, for parity runs only: the fast kernels reorder
 * f32 sums, which may flip a bf16 rounding of an activation and, on a near-tie, a greedy token.  Launches captured
 * into a CUDA graph keep the mode they were captured in.  Returns the previous setting.
 */
int tlaloc_b200_set_order_faithful(int on);

/* Kernels this library has launched (or captured into a graph) since it was loaded, over all threads. */
long long tlaloc_b200_launch_count(void);

/* ------------------------------------------------------------------ paged attention */

/*
 * Number of context splits the kernels would like for a decode call of this
 * shape, and the bytes of the f32 scratch [splits, R, H, D + 2] that goes with
 * a split count.  The record per (split, row, head) is {max, sum, acc[D]} as
 * in triton/kernels/paged_attention.cu:13-15.
 */
int tlaloc_b200_paged_attention_splits(int32_t num_rows, int32_t num_kv_heads, int32_t num_tables,
                                       int32_t max_blocks_per_seq, int32_t block_size);
size_t tlaloc_b200_paged_attention_scratch_bytes(int32_t num_rows, int32_t num_heads, int32_t head_dim,
                                                 int32_t splits);

/*
 * PAGED_ATTENTION (ir/.../PagedAttentionAttrs.kt:79-286, interpreter
 * ir/.../passes/DxirInterpreter.kt:2049-2140); replaces the launch pair
 * SliceKernel + CombineKernel behind the tlaloc_paged_attention custom call
 * (triton/kernels/paged_attention.cu:135-274,1174-1216,1300-1319) and the
 * three-stage PTX chain kptx_paged_scores/softmax/out (kptx/.../KptxKernels.kt:970-1356).
 *
 *   query        device [R, H, D]            q_dtype  F32 | BF16
 *   key_cache    device [P, bs, Hkv, D]      kv_dtype F32 | BF16 | F8E4M3FN (the reference's three pool dtypes,
 *                                            triton/kernels/paged_attention.cu:1429-1441; e4m3fn values widen exactly)
 *   value_cache  device, same shape/dtype
 *   block_tables device i32 [Tb, M]          row r reads table r / (R / Tb)
 *   seq_lens     device i32 [R]              row r attends positions [first, seq_lens[r])
 *   keep         device i32 [R, keep_chunks] or NULL: position t of row r takes part
 *                iff keep[r, t / (M*bs/keep_chunks)] != 0
 *   out          device [R, H, D]            out_dtype F32 | BF16
 *   lse          device f32 [R, H] or NULL   log-sum-exp of the scaled scores (return_lse)
 *   scratch      device f32 [splits, R, H, D + 2], caller-owned, contents undefined
 *                on entry and exit; at most `splits` context slices are used
 *   scale        softmax temperature (required attr); sliding_window 0 = none, else
 *                first = max(0, len - window)
 *
 * GQA: query head h reads kv head h / (H / Hkv).  A row with seq_len 0 gives
 * zeros (and lse -inf), as the interpreter does.  Positions >= seq_len are
 * never read; block ids are clamped into [0, P) and lengths into [0, M*bs]
 * rather than trusted.
 */
int tlaloc_b200_paged_attention(const void* query, int32_t q_dtype, const void* key_cache, const void* value_cache,
                                int32_t kv_dtype, const int32_t* block_tables, const int32_t* seq_lens,
                                const int32_t* keep, int32_t keep_chunks, void* out, int32_t out_dtype, float* lse,
                                float* scratch, int32_t splits, int32_t num_rows, int32_t num_heads, int32_t head_dim,
                                int32_t num_blocks, int32_t block_size, int32_t num_kv_heads,
                                int32_t max_blocks_per_seq, int32_t num_tables, float scale, int32_t sliding_window,
                                void* stream);

/*
 * The same operator for callers that cannot allocate device memory: a handler running inside a CUDA graph
 * capture, an XLA program whose emitter declared no scratch result for the call, or a host runtime (a JVM
 * binding, a plugin) that is handed device pointers but owns no allocator.  It takes no scratch: the split
 * records go to a 16 MiB array built into the library (tlaloc_b200_paged_attention_static_scratch_bytes()),
 * which every GPU that loads the library holds until the process exits.  This entry point has no counterpart
 * in the reference, whose kernel always receives an XLA-owned scratch result.
 *
 *  - It calls no cudaMalloc, cudaFree or other allocating routine.
 *  - Limit: the records of ceil(M*bs / 8192) slices, num_rows * num_heads * (head_dim + 2) floats each, must fit
 *    the array; a larger call is refused with TLALOC_B200_INVALID_ARGUMENT and a message giving both sizes.
 *    Within the limit it uses as many slices as fit (at most ceil(M*bs / 256)).
 *  - The first call on each device looks up the array's device address (with that device current); make that
 *    first call before any stream capture begins.
 *  - All calls on a device share the one array.  Nothing in it needs clearing between calls (every record that
 *    is read was written by the same call), but two calls whose kernels overlap on the GPU (different streams,
 *    or threads launching concurrently) race on it: serialise them, or give them their own scratch through
 *    tlaloc_b200_paged_attention.
 * All other arguments are those of tlaloc_b200_paged_attention.
 */
size_t tlaloc_b200_paged_attention_static_scratch_bytes(void);
int tlaloc_b200_paged_attention_static(const void* query, int32_t q_dtype, const void* key_cache,
                                       const void* value_cache, int32_t kv_dtype, const int32_t* block_tables,
                                       const int32_t* seq_lens, const int32_t* keep, int32_t keep_chunks, void* out,
                                       int32_t out_dtype, float* lse, int32_t num_rows, int32_t num_heads,
                                       int32_t head_dim, int32_t num_blocks, int32_t block_size, int32_t num_kv_heads,
                                       int32_t max_blocks_per_seq, int32_t num_tables, float scale,
                                       int32_t sliding_window, void* stream);

/*
 * KV_CACHE_WRITE (ir/.../KvCacheWriteAttrs.kt:62-159, interpreter
 * DxirInterpreter.kt:2233-2272; XLA scatter form stablehlo/.../StablehloEmitter.kt:4634):
 * row i of new_kv [T, Hkv*D] goes to pool slot slot_mapping[i]; a negative slot
 * is padding and is skipped; slots >= P*bs are skipped too (the interpreter
 * refuses them; the scatter drops them).  In place on the pool.  pool_dtype F32 | BF16 |
 * F8E4M3FN: a bf16 pool stores each value rounded to nearest even, an e4m3fn pool clamped
 * to +-448 and rounded (core/.../Fp8.kt:89-90 saturateToF8e4m3fn); new_dtype F32 | BF16.
 */
int tlaloc_b200_kv_cache_write(void* pool, int32_t pool_dtype, const void* new_kv, int32_t new_dtype,
                               const int32_t* slot_mapping, int32_t num_tokens, int32_t row_elems,
                               int32_t num_slots, void* stream);

/* ------------------------------------------------------------------ int8 weight-only projection */

/* Bytes of scratch the projection wants for this shape: room for the bf16 copy of an F32 x, or for the two int8 planes
 * of the activations (17 to 128 rows, see below) and their row steps. */
size_t tlaloc_b200_int8_gemm_scratch_bytes(int32_t m, int32_t k, int32_t n);

/*
 * y = (cast(x) @ cast(codes)) * scale: HfDecoderGraph.proj over a
 * WeightQuant.INT8 weight (ir/.../inference/HfDecoderGraph.kt:625-655,
 * WeightQuant.kt:8-22); replaces the XLA fusion of convert + dot_general +
 * multiply the reference emits for it (stablehlo Int8WeightEmitTest.kt:44-61,
 * docs/SERVING_ARCHITECTURE.md:562-564,786-789).
 *
 *   x       device [M, K]  x_dtype F32 | BF16 (F32 is rounded to bf16 RNE first, as
 *           the graph's CAST does when the weight dtype is bf16)
 *   codes   device int8 [K, N]  (in, out): the staged layout of HfStagedWeights.quantize
 *   scales  device f32 [N], or NULL for none
 *   residual device f32 [M, N] or NULL: added after the scale (the layer's residual add)
 *   y       device [M, N]  y_dtype F32 | BF16
 *   scratch device memory, 16-byte aligned, contents undefined on entry and exit, or NULL:
 *           tlaloc_b200_int8_gemm_scratch_bytes(m, k, n) bytes.  An F32 x needs it (its bf16 copy); with it, 17 to 128
 *           rows may take the int8 tensor-core kernel below (TLALOC_B200_GEMM_I8_MMA).
 *
 * Kernels by row count: up to 16 rows a row-vector kernel (HBM-bound); 17 rows and more a tcgen05 kernel, in one of two
 * forms.  BF16 form: the codes become exact bf16 on the way into shared memory, bf16 x bf16 -> f32 in tensor memory;
 * only the f32 summation order differs from the reference's.  INT8 form (opt-in: flag TLALOC_B200_GEMM_I8_MMA, 17 to 128
 * rows, K and N multiples of 16, scratch given, $TLALOC_B200_GEMM_I8 not 0; otherwise the BF16 form runs): the codes reach the tensor core as they
 * are (TMA, kind::i8) and each activation row becomes a 16-bit fixed-point number under a power-of-two row step s[m],
 * x ~ (256 hi + lo) s[m] with hi, lo int8, so y = (256 sum hi w + sum lo w) s[m] scale[n] with exact int32 sums.
 * Elements within 2^8 of their row's largest magnitude are exact (so are integer-valued rows); the rest round to a
 * multiple of s[m] <= max|x[m,:]| / 16256, which bounds the result's error by (s[m] / 2) scale[n] sum_k |codes[k, n]|
 * (measured: 5e-6 of the output's rms on normal rows, 3e-4 with 60x outlier channels).  A row holding an infinity or a
 * NaN comes out all NaN.  About 1.35x faster than the BF16 form at 128 rows.
 *
 * The fast kernels read x and codes in 16-byte pieces; when either pointer is not 16-byte aligned (a view into a
 * larger buffer at an odd offset), or N is not a multiple of 16 or K of 8, the call runs the order-faithful kernel
 * below instead: slower, same contract.
 *
 * flags: TLALOC_B200_GEMM_EXACT runs the order-faithful kernel (f32 accumulate
 * in increasing k with separate multiply and add, bit-identical to the
 * interpreter's MATMUL, DxirInterpreter.kt:739-765); it is slow and exists for
 * parity runs and odd shapes.
 */
#define TLALOC_B200_GEMM_EXACT 1
#define TLALOC_B200_GEMM_X_F32_EXACT 2 /* with GEMM_EXACT: do not round an F32 x to bf16 (weight dtype F32) */
/* codes and scales are constants of the program: no kernel placed just before this call in the stream writes them.
 * Lets the batched-row kernel request its first weights while that kernel is still finishing (results are the same). */
#define TLALOC_B200_GEMM_WEIGHTS_CONST 4
/* take the INT8 form of the tensor-core kernel where it applies (activations as 16-bit fixed point per row, exact
 * int32 sums); without it the BF16 form (f32 accumulation of exact products) runs */
#define TLALOC_B200_GEMM_I8_MMA 8
/* with GEMM_I8_MMA: the scratch already holds the activation planes of this x (written by tlaloc_b200_rmsnorm_planes or
 * tlaloc_b200_peer_sum_rows_f32 for exactly this [m, k]); ignored when the call does not take the INT8 form */
#define TLALOC_B200_GEMM_X_PLANES 16
int tlaloc_b200_int8_gemm(const void* x, int32_t x_dtype, const int8_t* codes, const float* scales,
                          const float* residual, void* y, int32_t y_dtype, float* scratch, size_t scratch_bytes,
                          int32_t m, int32_t k, int32_t n, int32_t flags, void* stream);

/*
 * The MLP's gate and up projections with SwiGLU folded into the epilogue (mlpOut, HfDecoderGraph.kt:953-988:
 * silu(proj(x, gate)) * proj(x, up)): one pass over both weights, and the [M, 2F] intermediate never reaches memory.
 *   codes   int8 [K, N], N = 2F a multiple of 256, the two weights interleaved in column blocks of 128: columns
 *           256t .. 256t+127 are gate columns 128t .. 128t+127, columns 256t+128 .. 256t+255 the same up columns
 *           (both in the staged [in, out] layout; tlaloc_b200.sharding.interleave_gate_up builds it at load time)
 *   scales  f32 [N] in the same column order, or NULL
 *   y       [M, F] F32 | BF16: silu(gate * scale) * (up * scale), SiLU in f32 as tlaloc_b200_swiglu computes it
 * 17 rows and more run on a tensor-core kernel; fewer rows, unaligned pointers, parity mode and GEMM_EXACT take an
 * order-faithful kernel (slow).  scratch and flags as tlaloc_b200_int8_gemm (an F32 x, or TLALOC_B200_GEMM_I8_MMA).
 */
int tlaloc_b200_int8_gemm_swiglu(const void* x, int32_t x_dtype, const int8_t* codes, const float* scales, void* y,
                                 int32_t y_dtype, float* scratch, size_t scratch_bytes, int32_t m, int32_t k, int32_t n,
                                 int32_t flags, void* stream);

/*
 * The same projection over an unquantized weight w [K, N] (F32 | BF16), order-faithful
 * (the embedding-free head of ReferenceDecodeGraph.kt:113-147 and a bf16 lm_head).
 */
int tlaloc_b200_dense_gemm_exact(const void* x, int32_t x_dtype, const void* w, int32_t w_dtype, float* y, int32_t m,
                                 int32_t k, int32_t n, int32_t flags, void* stream);

/* ------------------------------------------------------------------ the decode step's small ops */

/* EMBEDDING (DxirInterpreter.kt:1007-1040): out[p, :] = table[ids[p], :] widened to f32; ids clamped into the vocabulary. */
int tlaloc_b200_embedding(const void* table, int32_t table_dtype, const int32_t* ids, float* out, int32_t positions,
                          int32_t vocab, int32_t dim, void* stream);

/*
 * RMSNorm over the last axis (HfDecoderGraph.kt:663-699): x * rsqrt(mean(x^2) + eps) * gain.
 * x f32 [rows, n]; gain f32 [n] or NULL; out F32 | BF16.
 */
int tlaloc_b200_rmsnorm(const float* x, const float* gain, void* out, int32_t out_dtype, int32_t rows, int32_t n,
                        float eps, void* stream);

/*
 * The same with a BF16 out, and the normalised rows also written as the activation planes of the int8 tensor-core
 * projection (see tlaloc_b200_int8_gemm): `planes` is that projection's scratch for an [rows, n] activation
 * (planes_bytes >= tlaloc_b200_int8_gemm_scratch_bytes(rows, n, 0), 16-byte aligned; n a multiple of 16).  The projection that
 * consumes `out` is then called with the same scratch and TLALOC_B200_GEMM_X_PLANES and skips its own quantizer launch.
 * The planes are exactly what that launch would have written.
 */
int tlaloc_b200_rmsnorm_planes(const float* x, const float* gain, void* out, void* planes, size_t planes_bytes, int32_t rows,
                               int32_t n, float eps, void* stream);

/*
 * RoPE (HfDecoderGraph.kt:792-818, HF rotate_half with the duplicated cos/sin tables of
 * ropeTables :436-462) applied to q [T, H, hd] and k [T, Hkv, hd] (f32), followed by the two
 * KV_CACHE_WRITEs of attention() (:1230-1231): rotated k and v [T, Hkv, hd] go to the pools at
 * slot_mapping (kv_dtype F32 | BF16 | F8E4M3FN, narrowed as KV_CACHE_WRITE narrows).  q_out [T, H, hd] is F32 | BF16.
 * cos/sin are f32 [max_pos, hd].  ld_q/ld_k/ld_v are the row
 * strides of q, k and v in elements, so the three may be column blocks of one fused q|k|v projection result.
 */
int tlaloc_b200_rope_kv_write(const float* q, const float* k, const float* v, const int32_t* positions,
                              const float* cos_table, const float* sin_table, const int32_t* slot_mapping,
                              void* q_out, int32_t q_out_dtype, void* key_cache, void* value_cache, int32_t kv_dtype,
                              int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                              int32_t num_slots, int32_t max_pos, int32_t ld_q, int32_t ld_k, int32_t ld_v,
                              void* stream);

/* SwiGLU (HfDecoderGraph.kt:979-988): silu(gate) * up; gate/up f32 with row stride `ld`, out F32 | BF16 [rows, n]. */
int tlaloc_b200_swiglu(const float* gate, const float* up, int32_t ld, void* out, int32_t out_dtype, int32_t rows,
                       int32_t n, void* stream);

/* Greedy NEXT_TOKEN (DxirInterpreter.kt:2414-2426; triton/kernels/sample.cu greedy arm): first index of the maximum. */
int tlaloc_b200_argmax(const float* logits, int32_t* out, int32_t rows, int32_t n, void* stream);

/* ------------------------------------------------------------------ tensor parallelism: the sum over ranks */

#define TLALOC_B200_MAX_PEERS 8
#define TLALOC_B200_IPC_HANDLE_BYTES 64

/*
 * Peer-mapped device memory, one process per GPU.  tlaloc_b200_peer_alloc makes `bytes` of zeroed device memory on the
 * current device and an opaque 64-byte handle; the handle travels to the other ranks over any host channel, and
 * tlaloc_b200_peer_open maps that rank's buffer into this process (peer access over NVLink is enabled on first use).
 * _peer_close unmaps, _peer_free releases the owner's allocation once every peer has closed it.
 */
int tlaloc_b200_peer_alloc(size_t bytes, void** ptr, unsigned char handle[TLALOC_B200_IPC_HANDLE_BYTES]);
int tlaloc_b200_peer_open(const unsigned char handle[TLALOC_B200_IPC_HANDLE_BYTES], void** ptr);
int tlaloc_b200_peer_close(void* ptr);
int tlaloc_b200_peer_free(void* ptr);

/*
 * In-place sum over `world` ranks of `count` f32 values, the `stablehlo.all_reduce` with an add region that follows
 * the row-parallel o_proj and down_proj (stablehlo/.../StablehloEmitter.kt:3048-3072; semantics checked by
 * stablehlo/src/jvmTest/.../MultiDeviceCpuTest.kt:35-46).  One kernel per rank, all ranks launching the same call in
 * the same order: reduce-scatter by peer loads, all-gather by peer stores, flag words in the same peer-mapped buffer.
 *   bases[q]     device address, in THIS process, of rank q's peer buffer (bases[rank] is the local one); host array
 *   data_offset  byte offset of the values inside every buffer (multiple of 16)
 *   flag_offset  byte offset of 2 * world u32 flag words inside every buffer, zero before the first call
 *   state        4 u32 words of LOCAL device memory, zero before the first call: [0] all-reduces finished,
 *                [2] status (0, or 1 + 16 * phase + the rank that did not arrive within the time limit; once set,
 *                later calls do not wait), [3] the limit of each wait in microseconds (0 = 20 s; a caller may set
 *                it before the first call).  The sums are added in rank order: every rank gets identical bits.
 * count must be a multiple of 4.  world == 1 is a no-op.
 */
int tlaloc_b200_peer_allreduce_f32(void* const* bases, size_t data_offset, size_t flag_offset, uint32_t* state,
                                   int32_t rank, int32_t world, size_t count, void* stream);

/*
 * The same sum with the RMSNorm that follows it in the decode step (HfDecoderGraph.kt:663-699) folded in: the values
 * are an f32 [rows, cols] matrix at data_offset; the rank that reduces a row also normalises it and writes, into
 * EVERY rank's buffer, the summed row (in place) and x * rsqrt(mean(x^2) + eps) * gain as bf16 [rows, cols] at
 * norm_offset.  gain: f32 [cols] in local memory (the same values on every rank) or NULL.  rows must divide by
 * world, cols must be a multiple of 16 and at most 32768; world >= 2.  Otherwise as tlaloc_b200_peer_allreduce_f32,
 * with which it shares the flag words and the state (calls of the two may be mixed, in the same order on every rank).
 */
int tlaloc_b200_peer_allreduce_rmsnorm_f32(void* const* bases, size_t data_offset, size_t norm_offset, size_t flag_offset,
                                           uint32_t* state, const float* gain, float eps, int32_t rank, int32_t world,
                                           int32_t rows, int32_t cols, void* stream);

/*
 * The same exchange with the residual stream left DISTRIBUTED BY ROWS: rank r keeps rows [rows r / world, rows (r + 1) /
 * world) of the f32 residual stream in LOCAL memory (own_rows, [rows / world, cols]) and nobody else needs them.  The
 * values at data_offset are this sub-layer's PARTIAL results (no residual added by anyone); the rank adds its own rows
 * of the residual stream and every rank's partial (rank order), writes the sums back to own_rows, normalises them and
 * writes only the bf16 normalised rows into every rank's buffer at norm_offset.  Per rank 2 bytes per element leave
 * instead of 6: at 8 ranks the exchange moves 5.25 MB per rank instead of 8.75 MB for a 128 x 8192 matrix.
 * Arguments and limits as tlaloc_b200_peer_allreduce_rmsnorm_f32; own_rows 16-byte aligned.
 * planes != 0: the normalised rows travel as the activation planes of the int8 tensor-core projection that reads them
 * (tlaloc_b200_int8_gemm with TLALOC_B200_GEMM_I8_MMA | TLALOC_B200_GEMM_X_PLANES and the region as its scratch)
 * instead of bf16: every rank's region at norm_offset then holds [rows][cols] hi bytes, [rows][cols] lo bytes and
 * [rows] f32 steps, bit for bit what that projection's own quantizer makes of the bf16 rows, and must have
 * tlaloc_b200_int8_gemm_scratch_bytes(rows, cols, 0) bytes.  The same bytes per element leave; the projection's
 * quantizer launch is saved.
 */
int tlaloc_b200_peer_reduce_rmsnorm_rows_f32(void* const* bases, size_t data_offset, size_t norm_offset, size_t flag_offset,
                                             uint32_t* state, float* own_rows, const float* gain, float eps, int32_t rank,
                                             int32_t world, int32_t rows, int32_t cols, int32_t planes, void* stream);

/*
 * The one-barrier form of the same sum, for the decode step: out = residual + sum over ranks of an f32 [rows, cols]
 * PARTIAL matrix at partial_offset of every rank's buffer, added in rank order (identical bits on every rank), kept in
 * this rank's LOCAL memory, with the RMSNorm that follows it: norm_out (bf16 [rows, cols], local, or NULL) = out *
 * rsqrt(mean(out^2) + eps) * gain.  Each rank reads every rank's partial; nothing is stored to a peer, so there is one
 * rendezvous (before the reads) instead of two.  What the caller owes for that: a rank must not overwrite this partial
 * buffer until it has completed ONE MORE call of this function (on another partial buffer, e.g. alternating between
 * two): every peer passes that call's rendezvous only after its reads of this one are done.
 *   residual  local f32 [rows, cols] or NULL; may equal out (the residual stream updated in place)
 *   flag words (world of them at flag_offset) and state as tlaloc_b200_peer_allreduce_f32; calls of the three functions
 *   may be mixed on one state if every rank makes the same calls in the same order.
 *   planes    NULL, or (with norm_out) the scratch of the int8 tensor-core projection that consumes norm_out
 *             (planes_bytes >= tlaloc_b200_int8_gemm_scratch_bytes(rows, cols, 0), 16-byte aligned, cols a multiple of 16): the
 *             normalised rows are also written as that projection's activation planes (TLALOC_B200_GEMM_X_PLANES)
 * cols a multiple of 4 up to 8192.  world == 1 is legal (out = residual + partial).
 */
int tlaloc_b200_peer_sum_rows_f32(void* const* bases, size_t partial_offset, size_t flag_offset, uint32_t* state,
                                  const float* residual, float* out, void* norm_out, const float* gain, float eps,
                                  int32_t rank, int32_t world, int32_t rows, int32_t cols, void* planes, size_t planes_bytes,
                                  void* stream);

/* ------------------------------------------------------------------ XLA typed-FFI registration */

struct PJRT_Api;
/*
 * Registers this library's typed-FFI handlers (tlaloc_paged_attention,
 * tlaloc_int8_gemm, tlaloc_kv_cache_write) with a PJRT GPU plugin's custom-call
 * extension.  Returns NULL on success, else a message in static storage.
 * Same name, signature and protocol as triton/kernels/tlaloc_kernels.cu:479-526,
 * so triton/backend/pjrt_runtime.cc:139-164 (RegisterKernels) and
 * runtime-pjrt/.../ffm/PjrtFfiRegistry.kt:192-204 (registerNativeLibrary) load
 * this library unchanged.
 */
const char* TlalocRegisterKernels(const struct PJRT_Api* api);

/*
 * One handler by target name ("tlaloc_paged_attention", "tlaloc_int8_gemm",
 * "tlaloc_kv_cache_write"), as an XLA_FFI_Handler* (XLA_FFI_Error* (*)(XLA_FFI_CallFrame*)),
 * or NULL for an unknown name: for callers that register handlers one at a time
 * (runtime-pjrt/.../ffm/PjrtFfiRegistry.kt:168-182) and for tests that drive a
 * handler with a hand-built call frame (runtime-pjrt/.../ffm/XlaFfiCallFrameTest.kt:55-100).
 */
void* tlaloc_b200_ffi_handler(const char* target);

#ifdef __cplusplus
}
#endif

#endif /* TLALOC_B200_H_ */
