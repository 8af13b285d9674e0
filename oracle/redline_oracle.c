/*
 * redline_oracle.c - CPU restatement of the non-GEMM decode path of
 * Kasamix/redline-llm, used ONLY as a checker.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. Nothing in the shipped library may link,
 * load or call it: only the test-suite, the smoke check and the benchmark's
 * CPU-baseline / reference legs do. The shipped path is the CUDA library and
 * it has no CPU fallback.
 *
 * Parity status: PINNED. Every function below is compared bit for bit with
 * the reference's own header-only CPU implementation (tests/reference/...,
 * compiled where it lies by oracle/Makefile into oracle/_ref/) on seeded
 * inputs, and with the reference's committed RoPE capture
 * (tests/data/rope_fixture.json) and its RMSNorm rounding landmarks
 * (tests/reference/rmsnorm_ref.hpp:192-201).
 *
 * Two families:
 *   rlo_*      FP64 math on FP16-quantised inputs, the rounding points of the
 *              reference's CPU references (the arbiter).
 *   rlo_*_f32  the same operations in the FP32 operation order of the
 *              reference's CUDA kernels (what "FP32 compute" means for the
 *              1-ulp gates). libm's expf/sincosf stand in for the device
 *              routines, so a last-place FP32 difference is possible.
 *
 * FP16 values travel as uint16_t bit patterns everywhere.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define RLO_BLOCK 16 /* tokens per KV page: src/core/types.hpp:21-43 (kKvBlockSize) */

/* ------------------------------------------------------------------ FP16 */

/* binary16 -> binary64, exact. Follows tests/reference/fp16_ref.hpp:49-64. */
double rlo_half_to_double(uint16_t h) {
  const int sign = h >> 15;
  const int e = (h >> 10) & 31;
  const int m = h & 1023;
  double v;
  if (e == 31) {
    v = m ? NAN : INFINITY;
  } else if (e == 0) {
    v = ldexp((double)m, -24);
  } else {
    v = ldexp((double)(m | 1024), e - 25);
  }
  return sign ? -v : v;
}

/*
 * binary64 -> binary16, one round-to-nearest-even step, subnormals kept,
 * |x| >= 65520 -> inf, NaN -> 0x7E00. Same function as
 * tests/reference/fp16_ref.hpp:71-118, computed on the integer significand
 * instead of with floor().
 */
uint16_t rlo_quantize(double x) {
  uint64_t bits;
  memcpy(&bits, &x, sizeof bits);
  const uint16_t sign = (uint16_t)((bits >> 48) & 0x8000u);
  const int be = (int)((bits >> 52) & 0x7FF);
  uint64_t frac = bits & 0xFFFFFFFFFFFFFull;
  if (be == 0x7FF) {
    return frac ? 0x7E00u : (uint16_t)(sign | 0x7C00u);
  }
  if (be == 0) {
    return sign; /* zero or a binary64 subnormal: far below half the smallest FP16 step */
  }
  const int e = be - 1023;            /* value = 1.frac * 2^e */
  uint64_t sig = frac | (1ull << 52); /* 53-bit significand, value = sig * 2^(e-52) */
  /* Target step is 2^(e-10) for normal results, 2^-24 in the subnormal band. */
  int drop = (e >= -14) ? 42 : 42 + (-14 - e); /* low bits of sig to discard */
  if (drop > 63) {
    return sign; /* below 2^-35: rounds to zero */
  }
  const uint64_t keep = sig >> drop;
  const uint64_t rem = sig & ((1ull << drop) - 1);
  const uint64_t halfway = 1ull << (drop - 1);
  uint64_t r = keep;
  if (rem > halfway || (rem == halfway && (keep & 1))) {
    r += 1;
  }
  if (e >= -14) {
    /* r in [1024, 2048]; 2048 carries into the next binade by itself below. */
    const uint32_t out = (uint32_t)((e + 14) << 10) + (uint32_t)r; /* (e+15)<<10 | (r-1024) */
    if (out >= 0x7C00u) {
      return (uint16_t)(sign | 0x7C00u);
    }
    return (uint16_t)(sign | out);
  }
  return (uint16_t)(sign | (uint16_t)r); /* r in [0, 1024]; 1024 is the smallest normal */
}

static inline double rt(double x) { return rlo_half_to_double(rlo_quantize(x)); }
static inline float h2f(uint16_t h) { return (float)rlo_half_to_double(h); }
static inline uint16_t f2h(float f) { return rlo_quantize((double)f); }

/* fp16(a+b) with one rounding: tests/reference/fp16_ref.hpp:129-132. */
uint16_t rlo_half_add(uint16_t a, uint16_t b) {
  return rlo_quantize(rlo_half_to_double(a) + rlo_half_to_double(b));
}

/*
 * Relative distance from v to the nearest FP16 rounding midpoint; 0 for
 * zero / non-finite / overflowing v. tests/reference/fp16_ref.hpp:142-164.
 */
double rlo_rel_distance_to_boundary(double v) {
  const double a = fabs(v);
  if (!isfinite(a) || a == 0.0) return 0.0;
  const uint16_t q = rlo_quantize(a);
  if ((q & 0x7C00u) == 0x7C00u) return 0.0;
  const double qv = rlo_half_to_double(q);
  const double below = (q == 0) ? -ldexp(1.0, -25) : 0.5 * (qv + rlo_half_to_double((uint16_t)(q - 1)));
  const double above = (q == 0x7BFFu) ? 65520.0 : 0.5 * (qv + rlo_half_to_double((uint16_t)(q + 1)));
  const double d1 = fabs(a - below), d2 = fabs(a - above);
  return (d1 < d2 ? d1 : d2) / a;
}

/* ------------------------------------------------------------------- RNG */

/* splitmix64 stream of tests/reference/fp16_ref.hpp:170-192. */
static inline uint64_t sm64_next(uint64_t* s) {
  *s += 0x9E3779B97F4A7C15ull;
  uint64_t z = *s;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static inline double sm64_uniform(uint64_t* s) { return (double)(sm64_next(s) >> 11) * 0x1.0p-53; }

/* n FP16 values uniform in [lo, hi); returns the advanced state. */
uint64_t rlo_fill_uniform_half(uint64_t state, uint16_t* out, int64_t n, double lo, double hi) {
  for (int64_t i = 0; i < n; ++i) out[i] = rlo_quantize(lo + sm64_uniform(&state) * (hi - lo));
  return state;
}

/* n FP16 values ~ N(mean, sigma): Box-Muller over the same uniform stream. */
uint64_t rlo_fill_normal_half(uint64_t state, uint16_t* out, int64_t n, double mean, double sigma) {
  for (int64_t i = 0; i < n; i += 2) {
    double u1 = sm64_uniform(&state);
    const double u2 = sm64_uniform(&state);
    if (u1 < 0x1.0p-53) u1 = 0x1.0p-53;
    const double r = sqrt(-2.0 * log(u1));
    const double a = 6.283185307179586476925286766559 * u2;
    out[i] = rlo_quantize(mean + sigma * r * cos(a));
    if (i + 1 < n) out[i + 1] = rlo_quantize(mean + sigma * r * sin(a));
  }
  return state;
}

/* n raw 64-bit draws. */
uint64_t rlo_fill_u64(uint64_t state, uint64_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = sm64_next(&state);
  return state;
}

/* --------------------------------------------------------------- RMSNorm */

/* Plain RMSNorm, FP64: tests/reference/rmsnorm_ref.hpp:36-56. */
void rlo_rmsnorm(uint16_t* out, const uint16_t* in, const uint16_t* w, int32_t rows, int32_t hidden,
                 float eps) {
#pragma omp parallel for schedule(static)
  for (int32_t r = 0; r < rows; ++r) {
    const uint16_t* x = in + (size_t)r * hidden;
    uint16_t* y = out + (size_t)r * hidden;
    double ss = 0.0;
    for (int32_t c = 0; c < hidden; ++c) {
      const double v = rlo_half_to_double(x[c]);
      ss += v * v;
    }
    const double inv = 1.0 / sqrt(ss / (double)hidden + (double)eps);
    for (int32_t c = 0; c < hidden; ++c) {
      const double n = rt(rlo_half_to_double(x[c]) * inv);
      y[c] = rlo_quantize(n * rlo_half_to_double(w[c]));
    }
  }
}

/*
 * Fused residual-add + RMSNorm, FP64: tests/reference/rmsnorm_ref.hpp:72-110.
 *   h = fp16(res + in) (rounding point 1), res <- h, ms over the ROUNDED h,
 *   out = fp16(fp16(h * inv) * w) (rounding point 2 before the weight).
 * residual is updated in place. inv_rms (per row) and excluded (per element,
 * set when |h*inv| lies within rel_floor of an FP16 midpoint) may be NULL.
 */
void rlo_rmsnorm_residual(uint16_t* out, uint16_t* residual, const uint16_t* in, const uint16_t* w,
                          int32_t rows, int32_t hidden, float eps, double* inv_rms,
                          uint8_t* excluded, double rel_floor) {
#pragma omp parallel for schedule(static)
  for (int32_t r = 0; r < rows; ++r) {
    uint16_t* res = residual + (size_t)r * hidden;
    const uint16_t* x = in + (size_t)r * hidden;
    uint16_t* y = out + (size_t)r * hidden;
    double ss = 0.0;
    for (int32_t c = 0; c < hidden; ++c) {
      res[c] = rlo_half_add(res[c], x[c]);
      const double h = rlo_half_to_double(res[c]);
      ss += h * h;
    }
    const double inv = 1.0 / sqrt(ss / (double)hidden + (double)eps);
    if (inv_rms) inv_rms[r] = inv;
    for (int32_t c = 0; c < hidden; ++c) {
      const double v = rlo_half_to_double(res[c]) * inv;
      y[c] = rlo_quantize(rt(v) * rlo_half_to_double(w[c]));
      if (excluded) {
        excluded[(size_t)r * hidden + c] =
            (rel_floor > 0.0 && rlo_rel_distance_to_boundary(v) < rel_floor) ? 1 : 0;
      }
    }
  }
}

/* Wrong order 1: normalises the UNROUNDED sum (rmsnorm_ref.hpp:126-147). */
void rlo_rmsnorm_residual_mutant_unrounded(uint16_t* out, const uint16_t* residual,
                                           const uint16_t* in, const uint16_t* w, int32_t rows,
                                           int32_t hidden, float eps) {
  for (int32_t r = 0; r < rows; ++r) {
    const size_t b = (size_t)r * hidden;
    double ss = 0.0;
    for (int32_t c = 0; c < hidden; ++c) {
      const double s = rlo_half_to_double(residual[b + c]) + rlo_half_to_double(in[b + c]);
      ss += s * s;
    }
    const double inv = 1.0 / sqrt(ss / (double)hidden + (double)eps);
    for (int32_t c = 0; c < hidden; ++c) {
      const double s = rlo_half_to_double(residual[b + c]) + rlo_half_to_double(in[b + c]);
      out[b + c] = rlo_quantize(rt(s * inv) * rlo_half_to_double(w[c]));
    }
  }
}

/* Wrong order 2: one rounding of h*inv*w (rmsnorm_ref.hpp:152-173). */
void rlo_rmsnorm_residual_mutant_single_round(uint16_t* out, const uint16_t* residual,
                                              const uint16_t* in, const uint16_t* w, int32_t rows,
                                              int32_t hidden, float eps) {
  for (int32_t r = 0; r < rows; ++r) {
    const size_t b = (size_t)r * hidden;
    double ss = 0.0;
    for (int32_t c = 0; c < hidden; ++c) {
      const double h = rlo_half_to_double(rlo_half_add(residual[b + c], in[b + c]));
      ss += h * h;
    }
    const double inv = 1.0 / sqrt(ss / (double)hidden + (double)eps);
    for (int32_t c = 0; c < hidden; ++c) {
      const double h = rlo_half_to_double(rlo_half_add(residual[b + c], in[b + c]));
      out[b + c] = rlo_quantize(h * inv * rlo_half_to_double(w[c]));
    }
  }
}

/*
 * Half-ULP boundary fixture of tests/reference/rmsnorm_ref.hpp:175-250:
 * 8 rows x 1536, 256 boundary columns per row at c = 6i + (r mod 6) holding
 * (residual 0x3C00 | 0x3C01 by row parity, input 0x1000); filler residual
 * ~U(0.25,4) from stream seed+r, filler input +0; weight ~U(0.5,2) from stream
 * seed+1000003. is_boundary may be NULL.
 */
void rlo_build_rmsnorm_boundary_fixture(uint64_t seed, uint16_t* residual, uint16_t* input,
                                        uint16_t* weight, uint8_t* is_boundary) {
  enum { ROWS = 8, HID = 1536, NB = 256 };
  for (int r = 0; r < ROWS; ++r) {
    uint64_t st = seed + (uint64_t)r;
    for (int c = 0; c < HID; ++c) {
      const int on = (c % 6 == r % 6) && (c / 6 < NB);
      const size_t i = (size_t)r * HID + c;
      if (is_boundary) is_boundary[i] = (uint8_t)on;
      if (on) {
        residual[i] = (r & 1) ? 0x3C01u : 0x3C00u;
        input[i] = 0x1000u;
      } else {
        residual[i] = rlo_quantize(0.25 + sm64_uniform(&st) * 3.75);
        input[i] = 0;
      }
    }
  }
  uint64_t ws = seed + 1000003ull;
  for (int c = 0; c < HID; ++c) weight[c] = rlo_quantize(0.5 + sm64_uniform(&ws) * 1.5);
}

/*
 * FP32 operation order of the CUDA kernels (src/kernels/rmsnorm.cu:125-141,
 * 204-254): h = fp16(f32(r)+f32(x)); sum of squares in FP32; inv =
 * 1/sqrtf(ss/H + eps); out = fp16(f32(fp16(f32(h)*inv)) * f32(w)). The FP32
 * summation order is left-to-right here (the kernels use a tree); residual
 * may be NULL for the plain variant (then `in` is normalised directly).
 */
void rlo_rmsnorm_f32(uint16_t* out, uint16_t* residual, const uint16_t* in, const uint16_t* w,
                     int32_t rows, int32_t hidden, float eps) {
#pragma omp parallel for schedule(static)
  for (int32_t r = 0; r < rows; ++r) {
    const uint16_t* x = in + (size_t)r * hidden;
    uint16_t* res = residual ? residual + (size_t)r * hidden : NULL;
    uint16_t* y = out + (size_t)r * hidden;
    double ss = 0.0; /* exact-ish sum, rounded once: within the kernels' couple-of-ulp spread */
    for (int32_t c = 0; c < hidden; ++c) {
      uint16_t hb = x[c];
      if (res) {
        hb = f2h(h2f(res[c]) + h2f(x[c]));
        res[c] = hb;
      }
      const float h = h2f(hb);
      ss += (double)h * (double)h;
    }
    const float inv = 1.0f / sqrtf((float)ss / (float)hidden + eps);
    for (int32_t c = 0; c < hidden; ++c) {
      const float h = h2f(res ? res[c] : x[c]);
      const uint16_t n = f2h(h * inv);
      y[c] = f2h(h2f(n) * h2f(w[c]));
    }
  }
}

/* ------------------------------------------------------------------ RoPE */

/*
 * NeoX half-rotation in place, FP64 trig, three FP16 rounding points
 * (cos/sin, each product, each sum): tests/reference/rope_ref.hpp:40-72.
 * heads: [num_tokens, num_heads*head_dim] with rows row_stride apart.
 */
void rlo_rope(uint16_t* heads, int64_t row_stride, const int32_t* positions, int32_t num_tokens,
              int32_t num_heads, int32_t head_dim, double theta) {
  const int32_t hd2 = head_dim / 2;
#pragma omp parallel for schedule(static)
  for (int32_t t = 0; t < num_tokens; ++t) {
    const double pos = (double)positions[t];
    for (int32_t d = 0; d < hd2; ++d) {
      const double f = pow(theta, -2.0 * (double)d / (double)head_dim);
      const double c = rt(cos(pos * f));
      const double s = rt(sin(pos * f));
      for (int32_t h = 0; h < num_heads; ++h) {
        uint16_t* p = heads + (size_t)t * row_stride + (size_t)h * head_dim;
        const double a = rlo_half_to_double(p[d]);
        const double b = rlo_half_to_double(p[d + hd2]);
        p[d] = rlo_quantize(rt(a * c) - rt(b * s));
        p[d + hd2] = rlo_quantize(rt(b * c) + rt(a * s));
      }
    }
  }
}

/*
 * FP32 order of src/kernels/rope.cu:150-210,231-257: inv_freq[d] =
 * 1.0f / powf(theta, (float)(2d)/(float)head_dim); angle = (float)pos *
 * inv_freq[d]; sincosf; then the same three FP16 rounding points with FP32
 * products and sums.
 */
void rlo_rope_f32(uint16_t* heads, int64_t row_stride, const int32_t* positions, int32_t num_tokens,
                  int32_t num_heads, int32_t head_dim, float theta) {
  const int32_t hd2 = head_dim / 2;
#pragma omp parallel for schedule(static)
  for (int32_t t = 0; t < num_tokens; ++t) {
    const float pos = (float)positions[t];
    for (int32_t d = 0; d < hd2; ++d) {
      const float f = 1.0f / powf(theta, (float)(2 * d) / (float)head_dim);
      const float ang = pos * f;
      const float c = h2f(f2h(cosf(ang)));
      const float s = h2f(f2h(sinf(ang)));
      for (int32_t h = 0; h < num_heads; ++h) {
        uint16_t* p = heads + (size_t)t * row_stride + (size_t)h * head_dim;
        const float a = h2f(p[d]);
        const float b = h2f(p[d + hd2]);
        const float ac = h2f(f2h(a * c)), bs = h2f(f2h((-b) * s));
        const float bc = h2f(f2h(b * c)), as = h2f(f2h(a * s));
        p[d] = f2h(ac + bs);
        p[d + hd2] = f2h(bc + as);
      }
    }
  }
}

/* The FP32 inverse-frequency table exactly as the launcher computes it. */
void rlo_rope_inv_freq_f32(float* table, int32_t head_dim, float theta) {
  for (int32_t d = 0; d < head_dim / 2; ++d)
    table[d] = 1.0f / powf(theta, (float)(2 * d) / (float)head_dim);
}

/* ------------------------------------------------------------ paged pool */

/*
 * Element index in one layer's pool slice [num_blocks, 2, kv_heads, 16,
 * head_dim]: tests/reference/pool_ref.hpp:21-34, src/kernels/kv_scatter.cu:82-88.
 */
static inline int64_t pool_index(int32_t block, int32_t kv, int32_t head, int32_t slot, int32_t d,
                                 int32_t kv_heads, int32_t head_dim) {
  return ((((int64_t)block * 2 + kv) * kv_heads + head) * RLO_BLOCK + slot) * head_dim + d;
}

/*
 * KV scatter, a pure bit move: tests/reference/pool_ref.hpp:41-63,
 * src/kernels/kv_scatter.cu:98-137. p = positions[t]; block =
 * tables[t*table_row_stride + p/16]; slot = p%16. table_row_stride 0 = all
 * tokens share one row (prefill).
 */
void rlo_kv_scatter(uint16_t* pool, const uint16_t* k, const uint16_t* v, int64_t k_row_stride,
                    int64_t v_row_stride, const int32_t* tables, int64_t table_row_stride,
                    const int32_t* positions, int32_t num_tokens, int32_t kv_heads,
                    int32_t head_dim) {
  for (int32_t t = 0; t < num_tokens; ++t) {
    const int32_t p = positions[t];
    const int32_t block = tables[(int64_t)t * table_row_stride + p / RLO_BLOCK];
    const int32_t slot = p % RLO_BLOCK;
    for (int32_t h = 0; h < kv_heads; ++h) {
      memcpy(pool + pool_index(block, 0, h, slot, 0, kv_heads, head_dim),
             k + (int64_t)t * k_row_stride + (int64_t)h * head_dim, (size_t)head_dim * 2);
      memcpy(pool + pool_index(block, 1, h, slot, 0, kv_heads, head_dim),
             v + (int64_t)t * v_row_stride + (int64_t)h * head_dim, (size_t)head_dim * 2);
    }
  }
}

/*
 * Paged GQA decode attention, FP64 two-pass softmax per (sequence, q head),
 * one FP16 rounding at the end; rows with seq_len <= 0 are left untouched
 * (the reference's CPU function zero-fills them, its kernels do not write
 * them: tests/reference/attention_ref.hpp:32-81,
 * src/kernels/paged_attention.cu:153-156). Only positions < seq_len are read.
 * q and out are dense [num_seqs, q_heads*head_dim].
 */
void rlo_paged_attention(uint16_t* out, const uint16_t* q, const uint16_t* pool,
                         const int32_t* tables, const int32_t* seq_lens, int32_t num_seqs,
                         int32_t max_blocks_per_seq, int32_t q_heads, int32_t kv_heads,
                         int32_t head_dim, double scale) {
  const int32_t group = q_heads / kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int32_t s = 0; s < num_seqs; ++s) {
    for (int32_t h = 0; h < q_heads; ++h) {
      const int32_t len = seq_lens[s];
      if (len <= 0) continue;
      const int32_t* row = tables + (size_t)s * max_blocks_per_seq;
      const int32_t kvh = h / group;
      const size_t qb = ((size_t)s * q_heads + h) * head_dim;
      double* w = (double*)malloc(sizeof(double) * (size_t)len);
      double* qd = (double*)malloc(sizeof(double) * (size_t)head_dim);
      double* acc = (double*)calloc((size_t)head_dim, sizeof(double));
      for (int32_t d = 0; d < head_dim; ++d) qd[d] = rlo_half_to_double(q[qb + d]);
      double mx = -INFINITY;
      for (int32_t t = 0; t < len; ++t) {
        const uint16_t* kr = pool + pool_index(row[t / RLO_BLOCK], 0, kvh, t % RLO_BLOCK, 0, kv_heads, head_dim);
        double dot = 0.0;
        for (int32_t d = 0; d < head_dim; ++d) dot += qd[d] * rlo_half_to_double(kr[d]);
        w[t] = dot * scale;
        if (w[t] > mx) mx = w[t];
      }
      double den = 0.0;
      for (int32_t t = 0; t < len; ++t) {
        w[t] = exp(w[t] - mx);
        den += w[t];
      }
      /* token-outer accumulation; FP64 reassociation noise is ~1e-16, far below the FP16 step */
      for (int32_t t = 0; t < len; ++t) {
        const uint16_t* vr = pool + pool_index(row[t / RLO_BLOCK], 1, kvh, t % RLO_BLOCK, 0, kv_heads, head_dim);
        for (int32_t d = 0; d < head_dim; ++d) acc[d] += w[t] * rlo_half_to_double(vr[d]);
      }
      for (int32_t d = 0; d < head_dim; ++d) out[qb + d] = rlo_quantize(acc[d] / den);
      free(w);
      free(qd);
      free(acc);
    }
  }
}

/* Same, returning the unrounded FP64 result (for max-abs gates free of output rounding). */
void rlo_paged_attention_f64out(double* out, const uint16_t* q, const uint16_t* pool,
                                const int32_t* tables, const int32_t* seq_lens, int32_t num_seqs,
                                int32_t max_blocks_per_seq, int32_t q_heads, int32_t kv_heads,
                                int32_t head_dim, double scale) {
  const int32_t group = q_heads / kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int32_t s = 0; s < num_seqs; ++s) {
    for (int32_t h = 0; h < q_heads; ++h) {
      const int32_t len = seq_lens[s];
      if (len <= 0) continue;
      const int32_t* row = tables + (size_t)s * max_blocks_per_seq;
      const int32_t kvh = h / group;
      const size_t qb = ((size_t)s * q_heads + h) * head_dim;
      double* w = (double*)malloc(sizeof(double) * (size_t)len);
      double* acc = (double*)calloc((size_t)head_dim, sizeof(double));
      double mx = -INFINITY;
      for (int32_t t = 0; t < len; ++t) {
        const uint16_t* kr = pool + pool_index(row[t / RLO_BLOCK], 0, kvh, t % RLO_BLOCK, 0, kv_heads, head_dim);
        double dot = 0.0;
        for (int32_t d = 0; d < head_dim; ++d) dot += rlo_half_to_double(q[qb + d]) * rlo_half_to_double(kr[d]);
        w[t] = dot * scale;
        if (w[t] > mx) mx = w[t];
      }
      double den = 0.0;
      for (int32_t t = 0; t < len; ++t) {
        w[t] = exp(w[t] - mx);
        den += w[t];
      }
      for (int32_t t = 0; t < len; ++t) {
        const uint16_t* vr = pool + pool_index(row[t / RLO_BLOCK], 1, kvh, t % RLO_BLOCK, 0, kv_heads, head_dim);
        for (int32_t d = 0; d < head_dim; ++d) acc[d] += w[t] * rlo_half_to_double(vr[d]);
      }
      for (int32_t d = 0; d < head_dim; ++d) out[qb + d] = acc[d] / den;
      free(w);
      free(acc);
    }
  }
}

/* -------------------------------------------------------------- SiLU*mul */

/*
 * out[r,c] = fp16(silu(g) * u), silu(x) = x/(1+exp(-x)), FP64, one rounding:
 * tests/reference/elementwise_ref.hpp:23-37. gate_up rows are 2*inter wide
 * (gate | up); out rows are out_row_stride apart (inter when dense, 2*inter
 * when written in place over the gate half).
 */
void rlo_silu_mul(uint16_t* out, int64_t out_row_stride, const uint16_t* gate_up, int32_t rows,
                  int32_t inter) {
#pragma omp parallel for schedule(static)
  for (int32_t r = 0; r < rows; ++r) {
    const uint16_t* g = gate_up + (size_t)r * 2 * inter;
    const uint16_t* u = g + inter;
    uint16_t* y = out + (size_t)r * out_row_stride;
    for (int32_t c = 0; c < inter; ++c) {
      const double x = rlo_half_to_double(g[c]);
      const double up = rlo_half_to_double(u[c]); /* read before the (possibly aliased) store */
      y[c] = rlo_quantize(x / (1.0 + exp(-x)) * up);
    }
  }
}

/* FP32 order of src/kernels/silu_mul.cu:67-83: x/(1.0f+expf(-x)) * u, one rounding. */
void rlo_silu_mul_f32(uint16_t* out, int64_t out_row_stride, const uint16_t* gate_up, int32_t rows,
                      int32_t inter) {
#pragma omp parallel for schedule(static)
  for (int32_t r = 0; r < rows; ++r) {
    const uint16_t* g = gate_up + (size_t)r * 2 * inter;
    const uint16_t* u = g + inter;
    uint16_t* y = out + (size_t)r * out_row_stride;
    for (int32_t c = 0; c < inter; ++c) {
      const float x = h2f(g[c]);
      const float up = h2f(u[c]);
      const float s = x / (1.0f + expf(-x));
      y[c] = f2h(s * up);
    }
  }
}

/* ---------------------------------------------------- embed / argmax (next) */

/* Greedy argmax, lowest index wins ties, NaN never wins, all-NaN -> 0:
 * tests/reference/elementwise_ref.hpp:46-64. */
void rlo_argmax(int32_t* out, const uint16_t* logits, int32_t rows, int32_t vocab) {
#pragma omp parallel for schedule(static)
  for (int32_t r = 0; r < rows; ++r) {
    const uint16_t* x = logits + (size_t)r * vocab;
    double best = -INFINITY;
    int32_t bi = -1;
    for (int32_t i = 0; i < vocab; ++i) {
      const double v = rlo_half_to_double(x[i]);
      if (v > best || (bi < 0 && v == best)) {
        best = v;
        bi = i;
      }
    }
    out[r] = bi < 0 ? 0 : bi;
  }
}

/* Worker threads the parallel loops above will use. */
int rlo_omp_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void rlo_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------ prefill-side launchers */

/*
 * KV gather, the inverse bit move of the scatter: position t of ONE sequence comes from
 * block_table_row[t/16], slot t%16 (tests/reference/pool_ref.hpp:68-87,
 * src/kernels/kv_gather.cu:136-168). khat/vhat are [kv_heads, ctx_len, head_dim] views with a
 * head stride and a row stride in elements.
 */
void rlo_kv_gather(uint16_t* khat, uint16_t* vhat, int64_t khat_head_stride, int64_t khat_row_stride,
                   int64_t vhat_head_stride, int64_t vhat_row_stride, const uint16_t* pool,
                   const int32_t* table_row, int32_t ctx_len, int32_t kv_heads, int32_t head_dim) {
  for (int32_t t = 0; t < ctx_len; ++t) {
    const int32_t block = table_row[t / RLO_BLOCK], slot = t % RLO_BLOCK;
    for (int32_t h = 0; h < kv_heads; ++h) {
      memcpy(khat + h * khat_head_stride + (int64_t)t * khat_row_stride,
             pool + pool_index(block, 0, h, slot, 0, kv_heads, head_dim), (size_t)head_dim * 2);
      memcpy(vhat + h * vhat_head_stride + (int64_t)t * vhat_row_stride,
             pool + pool_index(block, 1, h, slot, 0, kv_heads, head_dim), (size_t)head_dim * 2);
    }
  }
}

/*
 * Prefill causal softmax over FP32 scores [heads, chunk_len, kv_len]: query row i sits at global
 * position chunk_start + i and sees keys j <= that position; live entries get
 * fp16(exp(s - max) / sum) with FP64 max/sum, masked entries exact +0 and are never read
 * (tests/reference/attention_ref.hpp:88-114, src/kernels/prefill_attention.cu:103-162).
 */
void rlo_prefill_softmax(uint16_t* probs, const float* scores, int32_t heads, int32_t chunk_len,
                         int32_t kv_len, int32_t chunk_start) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int32_t h = 0; h < heads; ++h) {
    for (int32_t i = 0; i < chunk_len; ++i) {
      const size_t base = ((size_t)h * chunk_len + i) * (size_t)kv_len;
      int32_t live = chunk_start + i + 1;
      if (live > kv_len) live = kv_len;
      double mx = -INFINITY, den = 0.0;
      for (int32_t j = 0; j < live; ++j) if ((double)scores[base + j] > mx) mx = (double)scores[base + j];
      for (int32_t j = 0; j < live; ++j) den += exp((double)scores[base + j] - mx);
      for (int32_t j = 0; j < live; ++j) probs[base + j] = rlo_quantize(exp((double)scores[base + j] - mx) / den);
      for (int32_t j = live > 0 ? live : 0; j < kv_len; ++j) probs[base + j] = 0;
    }
  }
}
