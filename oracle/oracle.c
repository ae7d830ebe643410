/*
 * TEST INFRASTRUCTURE — NOT PRODUCT CODE.
 *
 * A CPU restatement, in plain C, of the arithmetic the reference's host
 * interpreter (ir/src/commonMain/kotlin/io/tlaloc/ir/passes/DxirInterpreter.kt)
 * performs for the LLM decode hot path: paged attention, the int8 weight-only
 * projection, the KV-cache write and the small ops of a Llama decode step.
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may
 * load this file's library; the CUDA product path never calls it.
 *
 * Every function names the reference lines it follows.  The loops keep the
 * interpreter's visit order and accumulator widths (f32 storage, f64
 * accumulation in the paged walk, f32 accumulation in MATMUL with separate
 * multiply and add) so that results are bit-identical to the interpreter's.
 * Build with -ffp-contract=off (the JVM never fuses a*b+c).
 *
 * Pinned against the reference's own golden vectors:
 *   triton/examples/reference/reference_decode.json (5 decode steps, logits),
 *   ir/src/commonTest/.../passes/PagedAttentionTest.kt hand-exact cases.
 *
 * The *_mt variants split independent rows across OpenMP threads for the
 * timed CPU baseline; each row keeps the single-thread order, so they give
 * the same bits.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* core/.../Bf16.kt:57-71 floatToBf16Bits: round to nearest even by
 * bias-and-carry; NaN keeps sign and top payload bits and gets the quiet bit. */
static inline uint16_t bf16_bits(float v)
{
  uint32_t bits;
  memcpy(&bits, &v, 4);
  if (v != v) return (uint16_t)((bits >> 16) | 0x0040u);
  uint32_t lsb = (bits >> 16) & 1u;
  return (uint16_t)((bits + 0x7FFFu + lsb) >> 16);
}

/* core/.../Bf16.kt:74 bf16BitsToFloat: exact widening. */
static inline float bf16_widen(uint16_t b)
{
  uint32_t bits = ((uint32_t)b) << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* DxirInterpreter.kt:108-109 snapToBf16. */
ORC_API void orc_snap_bf16(const float* in, float* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_widen(bf16_bits(in[i]));
}

ORC_API void orc_f32_to_bf16_bits(const float* in, uint16_t* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_bits(in[i]);
}

ORC_API void orc_bf16_bits_to_f32(const uint16_t* in, float* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_widen(in[i]);
}

/*
 * core/.../Fp8.kt:8-16,30-59,89-90: an f8e4m3fn KV pool stores saturateToF8e4m3fn(v) = the value clamped to +-448 and
 * rounded to the nearest e4m3fn (ties to even; subnormals are multiples of 2^-9; NaN encodes as 0x7F and reads back NaN).
 */
static inline uint8_t e4m3_bits(float v)
{
  if (v != v) return 0x7F;
  if (v > 448.f) v = 448.f;
  if (v < -448.f) v = -448.f;
  uint32_t bits;
  memcpy(&bits, &v, 4);
  const uint32_t sign = (bits >> 24) & 0x80u;
  bits &= 0x7FFFFFFFu;
  float a;
  memcpy(&a, &bits, 4);
  uint32_t code;
  if (a < 0.015625f) {
    const double scaled = (double)a * 512.0;
    const double lower = floor(scaled);
    const double frac = scaled - lower;
    int lo = (int)lower;
    code = (uint32_t)(frac > 0.5 ? lo + 1 : frac < 0.5 ? lo : (lo % 2 == 0 ? lo : lo + 1));
  } else {
    int e = (int)(bits >> 23) - 127;
    uint32_t m = bits & 0x7FFFFFu;
    const uint32_t lsb = (m >> 20) & 1u;
    m += 0x7FFFFu + lsb;
    if (m >= 0x800000u) {
      m -= 0x800000u;
      e += 1;
    }
    code = ((uint32_t)(e + 7) << 3) | (m >> 20);
  }
  return (uint8_t)(sign | code);
}

static inline float e4m3_widen(uint8_t b)
{
  const float sign = (b & 0x80) ? -1.f : 1.f;
  const int e = (b >> 3) & 0xF, m = b & 7;
  if (e == 0xF && m == 7) return NAN;
  const float v = e == 0 ? (float)m / 8.f * 0.015625f : (1.f + (float)m / 8.f) * ldexpf(1.f, e - 7);
  return sign * v;
}

ORC_API void orc_f32_to_e4m3_bits(const float* in, uint8_t* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) out[i] = e4m3_bits(in[i]);
}

ORC_API void orc_e4m3_bits_to_f32(const uint8_t* in, float* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) out[i] = e4m3_widen(in[i]);
}

ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/*
 * DxirInterpreter.kt:2049-2140 evalPagedAttention (full tables; `window` <= 0
 * means none, PagedAttentionAttrs.kt:124-126 firstLive; `keep` may be null,
 * keep_chunks entries per row).
 *   q       [R, H, D]           f32 (bf16 inputs arrive widened)
 *   kc, vc  [P, bs, Hkv, D]     f32
 *   tables  [Tb, M] i32, lens [R] i32
 *   out     [R, H, D] f32;  lse [R, H] or null (return_lse: max + ln(denom))
 * Returns 0, or a negative code for the interpreter's refusals:
 *   -1 len outside [0, M*bs], -2 block id outside [0, P).
 * An empty row stays zero.  Positions >= len are never read.
 */
static int paged_row(const float* q, const float* kc, const float* vc, const int32_t* tables, const int32_t* lens,
                     const int32_t* keep, int keep_chunks, float* out, float* lse, int R, int H, int D, int P, int bs,
                     int Hkv, int M, int Tb, double scale, int window, int s, double* scores, double* acc)
{
  const int group = H / Hkv, rows_per_table = R / Tb, ctx = M * bs;
  const int keep_chunk = keep ? ctx / keep_chunks : 0;
  const int len = lens[s];
  if (len < 0 || len > ctx) return -1;
  if (len == 0) return 0;
  const int table = s / rows_per_table;
  const int pages = (len + bs - 1) / bs;
  for (int h = 0; h < H; ++h) {
    const int kv = h / group;
    const int64_t qoff = ((int64_t)s * H + h) * D;
    double mx = -INFINITY;
    for (int page = 0; page < pages; ++page) {
      const int blk = tables[(int64_t)table * M + page];
      if (blk < 0 || blk >= P) return -2;
      const int base = page * bs;
      const int slots = bs < len - base ? bs : len - base;
      for (int slot = 0; slot < slots; ++slot) {
        const int64_t koff = (((int64_t)blk * bs + slot) * Hkv + kv) * D;
        double dot = 0.0;
        for (int j = 0; j < D; ++j) dot += (double)q[qoff + j] * (double)kc[koff + j];
        const double sc = dot * scale;
        scores[base + slot] = sc;
        if (sc > mx) mx = sc;
      }
    }
    const int first = window > 0 ? (len - window > 0 ? len - window : 0) : 0;
#define KEPT(t) (keep == NULL || keep[(int64_t)s * keep_chunks + (t) / keep_chunk] != 0)
    if (first > 0 || keep != NULL) {
      mx = -INFINITY;
      for (int t = first; t < len; ++t)
        if (KEPT(t) && scores[t] > mx) mx = scores[t];
    }
    double denom = 0.0;
    for (int t = first; t < len; ++t) {
      if (!KEPT(t)) continue;
      const double e = exp(scores[t] - mx);
      scores[t] = e;
      denom += e;
    }
    if (lse) lse[(int64_t)s * H + h] = (float)(mx + log(denom));
    for (int j = 0; j < D; ++j) acc[j] = 0.0;
    for (int page = 0; page < pages; ++page) {
      const int blk = tables[(int64_t)table * M + page];
      const int base = page * bs;
      const int slots = bs < len - base ? bs : len - base;
      for (int slot = 0; slot < slots; ++slot) {
        if (base + slot < first || !KEPT(base + slot)) continue;
        const double w = scores[base + slot] / denom;
        const int64_t voff = (((int64_t)blk * bs + slot) * Hkv + kv) * D;
        for (int j = 0; j < D; ++j) acc[j] += w * (double)vc[voff + j];
      }
    }
#undef KEPT
    for (int j = 0; j < D; ++j) out[qoff + j] = (float)acc[j];
  }
  return 0;
}

ORC_API int orc_paged_attention(const float* q, const float* kc, const float* vc, const int32_t* tables,
                                const int32_t* lens, const int32_t* keep, int keep_chunks, float* out, float* lse,
                                int R, int H, int D, int P, int bs, int Hkv, int M, int Tb, double scale, int window,
                                int threads)
{
  memset(out, 0, sizeof(float) * (size_t)R * H * D);
  if (lse)
    for (int64_t i = 0; i < (int64_t)R * H; ++i) lse[i] = -INFINITY;
  int status = 0;
  const int ctx = M * bs;
#ifdef _OPENMP
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
#endif
  {
    double* scores = (double*)malloc(sizeof(double) * (size_t)(ctx > 0 ? ctx : 1));
    double* acc = (double*)malloc(sizeof(double) * (size_t)(D > 0 ? D : 1));
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 1)
#endif
    for (int s = 0; s < R; ++s) {
      const int e = paged_row(q, kc, vc, tables, lens, keep, keep_chunks, out, lse, R, H, D, P, bs, Hkv, M, Tb, scale,
                              window, s, scores, acc);
      if (e != 0) {
#ifdef _OPENMP
#pragma omp critical
#endif
        status = e;
      }
    }
    free(scores);
    free(acc);
  }
  return status;
}

/*
 * The same walk with bf16 storage for q and the pools (bit patterns), widened
 * on read (DxirInterpreter.kt:85-109: a bf16 node holds widened bf16 values),
 * so the benchmark's CPU leg reads the bytes the GPU kernel reads instead of
 * an f32 copy twice the size.  Arithmetic as orc_paged_attention.
 */
ORC_API int orc_paged_attention_bf16(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, const int32_t* tables,
                                     const int32_t* lens, float* out, int R, int H, int D, int P, int bs, int Hkv,
                                     int M, int Tb, double scale, int threads)
{
  memset(out, 0, sizeof(float) * (size_t)R * H * D);
  int status = 0;
  const int group = H / Hkv, rows_per_table = R / Tb, ctx = M * bs;
#ifdef _OPENMP
#pragma omp parallel num_threads(threads > 0 ? threads : 1)
#endif
  {
    double* scores = (double*)malloc(sizeof(double) * (size_t)(ctx > 0 ? ctx : 1));
    double* acc = (double*)malloc(sizeof(double) * (size_t)(D > 0 ? D : 1));
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 1) collapse(2)
#endif
    for (int s = 0; s < R; ++s) {
      for (int h = 0; h < H; ++h) {
        const int len = lens[s];
        if (len < 0 || len > ctx) {
#ifdef _OPENMP
#pragma omp atomic write
#endif
          status = -1;
          continue;
        }
        if (len == 0) continue;
        const int table = s / rows_per_table, kv = h / group;
        const int64_t qoff = ((int64_t)s * H + h) * D;
        double mx = -INFINITY;
        int bad = 0;
        for (int t = 0; t < len; ++t) {
          const int blk = tables[(int64_t)table * M + t / bs];
          if (blk < 0 || blk >= P) {
            bad = 1;
            break;
          }
          const int64_t koff = (((int64_t)blk * bs + t % bs) * Hkv + kv) * D;
          double dot = 0.0;
          for (int j = 0; j < D; ++j) dot += (double)bf16_widen(q[qoff + j]) * (double)bf16_widen(kc[koff + j]);
          const double sc = dot * scale;
          scores[t] = sc;
          if (sc > mx) mx = sc;
        }
        if (bad) {
#ifdef _OPENMP
#pragma omp atomic write
#endif
          status = -2;
          continue;
        }
        double denom = 0.0;
        for (int t = 0; t < len; ++t) {
          const double e = exp(scores[t] - mx);
          scores[t] = e;
          denom += e;
        }
        for (int j = 0; j < D; ++j) acc[j] = 0.0;
        for (int t = 0; t < len; ++t) {
          const int blk = tables[(int64_t)table * M + t / bs];
          const double w = scores[t] / denom;
          const int64_t voff = (((int64_t)blk * bs + t % bs) * Hkv + kv) * D;
          for (int j = 0; j < D; ++j) acc[j] += w * (double)bf16_widen(vc[voff + j]);
        }
        for (int j = 0; j < D; ++j) out[qoff + j] = (float)acc[j];
      }
    }
    free(scores);
    free(acc);
  }
  return status;
}

/*
 * DxirInterpreter.kt:739-765 MATMUL, rank 2: out[i,j] += a[i,p] * b[p,j] in
 * f32, p outermost per output row, terms with a[i,p] == 0 skipped, product and
 * sum rounded separately.  out must be zeroed by the caller or is zeroed here.
 */
ORC_API void orc_matmul_f32(const float* a, const float* b, float* out, int m, int k, int n, int threads)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
#endif
  for (int i = 0; i < m; ++i) {
    float* row = out + (int64_t)i * n;
    for (int j = 0; j < n; ++j) row[j] = 0.f;
    for (int p = 0; p < k; ++p) {
      const float aip = a[(int64_t)i * k + p];
      if (aip == 0.f) continue;
      const float* brow = b + (int64_t)p * n;
      for (int j = 0; j < n; ++j) {
        const float prod = aip * brow[j];
        row[j] = row[j] + prod;
      }
    }
  }
}

/*
 * ir/.../inference/HfDecoderGraph.kt:625-655 proj() with an int8 weight:
 *   rhs = CAST(codes -> weight dtype)   exact (DxirInterpreter.kt:1206-1247)
 *   lhs = x, or CAST(x -> bf16) (RNE snap) when round_x_bf16 != 0
 *   y   = MATMUL(lhs, rhs) in f32 (orc_matmul_f32's order), then y * scale[j].
 * codes are [K, N] (in, out), scales [N], x [M, K] f32, y [M, N] f32.
 * Columns are split across threads when M is small; each output keeps its
 * own p-ascending order, so threading does not change a bit.
 */
ORC_API void orc_proj_int8(const float* x, const int8_t* codes, const float* scales, float* y, int m, int k, int n,
                           int round_x_bf16, int threads)
{
  float* xs = (float*)malloc(sizeof(float) * (size_t)m * k);
  for (int64_t i = 0; i < (int64_t)m * k; ++i) xs[i] = round_x_bf16 ? bf16_widen(bf16_bits(x[i])) : x[i];
  const int nt = threads > 0 ? threads : 1;
  const int chunk = 1024;
  const int nchunks = (n + chunk - 1) / chunk;
  (void)nt;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 1) collapse(2) num_threads(nt)
#endif
  for (int i = 0; i < m; ++i) {
    for (int c = 0; c < nchunks; ++c) {
      const int j0 = c * chunk, j1 = j0 + chunk < n ? j0 + chunk : n;
      float* row = y + (int64_t)i * n;
      for (int j = j0; j < j1; ++j) row[j] = 0.f;
      for (int p = 0; p < k; ++p) {
        const float aip = xs[(int64_t)i * k + p];
        if (aip == 0.f) continue;
        const int8_t* brow = codes + (int64_t)p * n;
        for (int j = j0; j < j1; ++j) {
          const float prod = aip * (float)brow[j];
          row[j] = row[j] + prod;
        }
      }
      for (int j = j0; j < j1; ++j) row[j] = row[j] * scales[j];
    }
  }
  free(xs);
}

/*
 * ir/src/jvmMain/.../HfStagedWeights.kt:433-444 quantize, INT8 arm
 * (WeightQuant.kt:8-22): per output row o of w [out, in]:
 *   scale = max|row| / 127 (1 for a zero row), in f32
 *   code  = clamp(rint((double)(row[c] / scale)), -127, 127)   rint = half-even
 * written transposed: codes[c * out + o], i.e. [in, out].
 */
ORC_API void orc_quantize_int8(const float* w, int rows_out, int cols_in, int8_t* codes, float* scales)
{
  for (int o = 0; o < rows_out; ++o) {
    const float* row = w + (int64_t)o * cols_in;
    float mx = 0.f;
    for (int c = 0; c < cols_in; ++c) {
      const float a = fabsf(row[c]);
      if (a > mx) mx = a;
    }
    const float scale = mx == 0.f ? 1.f : mx / 127.f;
    scales[o] = scale;
    for (int c = 0; c < cols_in; ++c) {
      double r = rint((double)(row[c] / scale));
      if (r < -127.0) r = -127.0;
      if (r > 127.0) r = 127.0;
      codes[(int64_t)c * rows_out + o] = (int8_t)(int)r;
    }
  }
}

/*
 * DxirInterpreter.kt:2233-2272 evalKvCacheWrite: row i of new_kv [T, stride]
 * is copied to pool + slot[i]*stride; a negative slot is padding and skipped.
 * Returns -1 for a slot past the pool, -2 for a repeated live slot.
 * The pool is updated in place (the interpreter copies it first; callers that
 * need the old pool keep their own copy).
 */
ORC_API int orc_kv_cache_write(float* pool, const float* new_kv, const int32_t* slots, int tokens, int stride,
                               int num_slots)
{
  for (int i = 0; i < tokens; ++i) {
    const int s = slots[i];
    if (s < 0) continue;
    if (s >= num_slots) return -1;
    for (int j = 0; j < i; ++j)
      if (slots[j] == s) return -2;
    memcpy(pool + (int64_t)s * stride, new_kv + (int64_t)i * stride, sizeof(float) * (size_t)stride);
  }
  return 0;
}

/*
 * HfDecoderGraph.kt:663-699 rmsNorm over the last axis, as the interpreter
 * evaluates it: sq = x*x (f32); SUM sequential in index order in f32
 * (DxirInterpreter.kt:1450-1496); MEAN = sum / n (:1791-1807); + eps (f32);
 * RSQRT in double then narrowed (:567-572); (x * rsq) * gain.  gain may be
 * null (no gain).
 */
ORC_API void orc_rmsnorm(const float* x, const float* gain, float* out, int rows, int n, float eps)
{
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (int64_t)r * n;
    float acc = 0.f;
    for (int j = 0; j < n; ++j) {
      const float sq = xr[j] * xr[j];
      acc = acc + sq;
    }
    const float mean = acc / (float)n;
    const float shifted = mean + eps;
    const float rsq = (float)(1.0 / sqrt((double)shifted));
    for (int j = 0; j < n; ++j) {
      const float scaled = xr[j] * rsq;
      out[(int64_t)r * n + j] = gain ? scaled * gain[j] : scaled;
    }
  }
}

/*
 * HfDecoderGraph.kt:436-462 ropeTables: cos/sin [positions, hd] computed in
 * double and narrowed; both halves of a row carry the same value.
 */
ORC_API void orc_rope_tables(double theta, int hd, int positions, float* cos_t, float* sin_t)
{
  const int half = hd / 2;
  for (int p = 0; p < positions; ++p) {
    for (int i = 0; i < half; ++i) {
      const double inv_freq = pow(theta, -2.0 * (double)i / (double)hd);
      const double angle = (double)p * inv_freq;
      const float c = (float)cos(angle), s = (float)sin(angle);
      cos_t[(int64_t)p * hd + i] = c;
      cos_t[(int64_t)p * hd + half + i] = c;
      sin_t[(int64_t)p * hd + i] = s;
      sin_t[(int64_t)p * hd + half + i] = s;
    }
  }
}

/*
 * HfDecoderGraph.kt:792-818 rope(): x*cos + rotate_half(x)*sin with
 * rotate_half = cat(-x[hd/2:], x[:hd/2]); each product and the sum rounded to
 * f32.  x [rows, heads, hd]; pos[rows] selects the table row.
 */
ORC_API void orc_rope(const float* x, const int32_t* pos, const float* cos_t, const float* sin_t, float* out, int rows,
                      int heads, int hd)
{
  const int half = hd / 2;
  for (int r = 0; r < rows; ++r) {
    const float* c = cos_t + (int64_t)pos[r] * hd;
    const float* s = sin_t + (int64_t)pos[r] * hd;
    for (int h = 0; h < heads; ++h) {
      const float* xr = x + ((int64_t)r * heads + h) * hd;
      float* o = out + ((int64_t)r * heads + h) * hd;
      for (int j = 0; j < hd; ++j) {
        const float rot = j < half ? -xr[j + half] : xr[j - half];
        const float a = xr[j] * c[j];
        const float b = rot * s[j];
        o[j] = a + b;
      }
    }
  }
}

/*
 * HfDecoderGraph.kt:979-988 SwiGLU: SILU(gate) * up, SILU evaluated in double
 * and narrowed (DxirInterpreter.kt:573-583: x / (1 + exp(-x))).
 */
ORC_API void orc_swiglu(const float* gate, const float* up, float* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) {
    const double g = (double)gate[i];
    const float silu = (float)(g / (1.0 + exp(-g)));
    out[i] = silu * up[i];
  }
}

/* DxirInterpreter.kt:2414-2426 evalArgmax over the last axis: first maximum wins. */
ORC_API void orc_argmax(const float* x, int32_t* out, int rows, int n)
{
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (int64_t)r * n;
    int best = 0;
    for (int i = 1; i < n; ++i)
      if (xr[i] > xr[best]) best = i;
    out[r] = best;
  }
}

/* DxirInterpreter.kt:1007-1040 EMBEDDING: out[p,:] = table[idx[p],:]; -1 for an index outside the vocabulary. */
ORC_API int orc_embedding(const float* table, const int32_t* idx, float* out, int positions, int vocab, int dim)
{
  for (int p = 0; p < positions; ++p) {
    const int v = idx[p];
    if (v < 0 || v >= vocab) return -1;
    memcpy(out + (int64_t)p * dim, table + (int64_t)v * dim, sizeof(float) * (size_t)dim);
  }
  return 0;
}

/* The element-wise f32 add of the residual connections (HfDecoderGraph.kt:1009, 1273). */
ORC_API void orc_add(const float* a, const float* b, float* out, int64_t n)
{
  for (int64_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}
