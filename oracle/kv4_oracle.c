/*
 * CPU oracle for the KV4 attention path -- TEST INFRASTRUCTURE, NOT PRODUCT.
 * See kv4_oracle.h for scope and pinning.  Build: oracle/Makefile
 * (gcc -O2 -ffp-contract=off -fopenmp): no FMA contraction, plain IEEE float,
 * default rounding mode (nearest-even), so the codec arithmetic reproduces the
 * reference's `--fmad=false` kernels bit for bit.
 */
#include "kv4_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ scalars */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> fp16, round to nearest even; what __float2half_rn does
 * (src/a8_prologue.cuh:37 `f2h`). */
uint16_t ysko_f32_to_f16(float f) {
  const uint32_t x = f2u(f), sign = (x >> 16) & 0x8000u, ax = x & 0x7fffffffu;
  if (ax >= 0x7f800000u) return (uint16_t)(sign | (ax > 0x7f800000u ? 0x7e00u : 0x7c00u));
  if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);             /* rounds to >= 65520 -> inf */
  if (ax < 0x33000001u) return (uint16_t)sign;                          /* <= 2^-25 -> 0 (tie to even) */
  int e = (int)(ax >> 23) - 127;
  uint32_t man = (ax & 0x7fffffu) | 0x800000u;                          /* 24-bit significand */
  int shift;                                                            /* bits to drop */
  uint32_t base;
  if (e >= -14) { shift = 13; base = (uint32_t)(e + 15) << 10; man &= 0x7fffffu; }
  else { shift = 13 + (-14 - e); base = 0; }                            /* subnormal half */
  uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;                     /* carry may bump the exponent: intended */
  return (uint16_t)(sign | (base + q));
}
/* fp16 -> fp32 (exact) (src/a8_prologue.cuh:36 `h2f`). */
float ysko_f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 0x3ffu;
  if (e == 31u) return u2f(sign | 0x7f800000u | (m << 13));
  if (e == 0u) { return (h & 0x8000u ? -1.f : 1.f) * (float)m * 5.9604644775390625e-8f; }  /* m * 2^-24 */
  return u2f(sign | ((e + 112u) << 23) | (m << 13));
}
uint16_t ysko_f32_to_bf16(float f) {
  uint32_t x = f2u(f);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
  x += 0x7fffu + ((x >> 16) & 1u);
  return (uint16_t)(x >> 16);
}
float ysko_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }
void ysko_bf16_to_f16_array(const uint16_t* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = ysko_f32_to_f16(ysko_bf16_to_f32(in[i]));
}
static inline float h2f(uint16_t h) { return ysko_f16_to_f32(h); }
static inline float round_f16(float f) { return ysko_f16_to_f32(ysko_f32_to_f16(f)); }

int ysko_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* --------------------------------------------------------------- rope table */

/* src/attention_gqa.cu:158-162: out[t][i] = (cos, sin)(float(t) * theta^(-2i/rd)).
 * The reference evaluates powf/sincosf with the CUDA math library, whose last-bit
 * results a CPU cannot reproduce; this restatement takes the exponent and the
 * trigonometric functions in double and rounds once, keeping the fp32 product
 * float(t) * freq_i that defines the angle. */
void ysko_rope_table(float* out, int max_ctx, float theta, int rd) {
  const int half = rd / 2;
  for (int i = 0; i < half; ++i) {
    const float freq = (float)pow((double)theta, -(double)(2 * i) / (double)rd);
    for (int t = 0; t < max_ctx; ++t) {
      const float ang = (float)t * freq;
      out[((size_t)t * half + i) * 2 + 0] = (float)cos((double)ang);
      out[((size_t)t * half + i) * 2 + 1] = (float)sin((double)ang);
    }
  }
}

/* -------------------------------------------------------------------- codec */

/* One int4 code, the formula shared by K groups and V tokens
 * (src/attention_gqa.cu:152, src/post_kernels.cu:77): q = rne((v-lo)*inv) in [0,15]. */
static inline int quant4(float v, float lo, float inv) {
  int q = (int)lrintf((v - lo) * inv);
  return q < 0 ? 0 : (q > 15 ? 15 : q);
}

/* src/attention_gqa.cu:143-154 (= src/post_kernels.cu:86-96 for HD 128). */
/* min / max with the zero signs of CUDA's fminf / fmaxf, which the reference's kernels call (src/post_kernels.cu:71,
 * src/attention_gqa.cu:147): -0.0 orders below +0.0, so a row of signed zeros gets lo = -0.0.  C's fminf leaves that
 * case to the implementation. */
static float min_dev(float a, float b) { if (a == b) return signbit(a) ? a : b; return a < b ? a : b; }
static float max_dev(float a, float b) { if (a == b) return signbit(a) ? b : a; return a > b ? a : b; }

void ysko_group_quant(const ysko_kv_layer* kv, int hkv, int hd, int max_ctx, int pos0, int M) {
  const int last = pos0 + M - 1;
  for (int gi = pos0 / 32; gi * 32 + 31 <= last; ++gi) {
    if (gi * 32 + 31 < pos0) continue;
    for (int head = 0; head < hkv; ++head) {
      const size_t gb = (size_t)head * (max_ctx / 32) + gi;
      for (int ch = 0; ch < hd; ++ch) {
        float v[32], lo = 1e30f, hi = -1e30f;
        for (int t = 0; t < 32; ++t) {
          v[t] = h2f(kv->kshadow[((size_t)head * max_ctx + gi * 32 + t) * hd + ch]);
          lo = min_dev(lo, v[t]); hi = max_dev(hi, v[t]);
        }
        const float sc = (hi - lo) / 15.f, inv = hi > lo ? 15.f / (hi - lo) : 0.f;
        kv->kscale[gb * hd + ch] = ysko_f32_to_f16(sc);
        kv->kzero[gb * hd + ch] = ysko_f32_to_f16(lo);
        for (int t = 0; t < 32; ++t) {
          const int q = quant4(v[t], lo, inv);
          uint8_t* b = &kv->kq[(gb * 32 + t) * (hd / 2) + (ch >> 1)];
          *b = (ch & 1) ? (uint8_t)((*b & 0x0f) | (q << 4)) : (uint8_t)((*b & 0xf0) | q);
        }
      }
    }
  }
}

void ysko_append(const ysko_kv_layer* kv, int hkv, int hd, int max_ctx, int pos0, int M,
                 const uint16_t* k16, const uint16_t* v16) {
  for (int r = 0; r < M; ++r) {
    const int pos = pos0 + r;
    for (int head = 0; head < hkv; ++head) {
      const uint16_t* kr = k16 + ((size_t)r * hkv + head) * hd;
      const uint16_t* vr = v16 + ((size_t)r * hkv + head) * hd;
      /* K: fp16 shadow row, un-rotated (src/post_kernels.cu:52-54) */
      memcpy(kv->kshadow + ((size_t)head * max_ctx + pos) * hd, kr, (size_t)hd * 2);
      /* V: per-(token, kv-head) min/max int4 (src/post_kernels.cu:64-82) */
      float lo = h2f(vr[0]), hi = lo;
      for (int d = 1; d < hd; ++d) { const float y = h2f(vr[d]); lo = min_dev(lo, y); hi = max_dev(hi, y); }
      const float sc = (hi - lo) / 15.f, inv = hi > lo ? 15.f / (hi - lo) : 0.f;
      const size_t slot = (size_t)head * max_ctx + pos;
      for (int d = 0; d < hd; d += 2) {
        const int q0 = quant4(h2f(vr[d]), lo, inv), q1 = quant4(h2f(vr[d + 1]), lo, inv);
        kv->vq[slot * (hd / 2) + (d >> 1)] = (uint8_t)(q0 | (q1 << 4));
      }
      kv->vscale[slot] = ysko_f32_to_f16(sc);
      kv->vzero[slot] = ysko_f32_to_f16(lo);
    }
  }
  ysko_group_quant(kv, hkv, hd, max_ctx, pos0, M);
}

/* ---------------------------------------------------------------- attention */

/* Dequantised, rotated key and value of token t as query row at `pos` sees them
 * (src/attention_gqa.cu:38-70).  kd, vd: float[hd]. */
/* Key and value of the token at position t.  `slot` is where its rows are stored: t itself, except for the own key of a
 * row of a tree-shaped pass (src/q35_atx.cu:111-119: position base + depth, cache slot base + row), which is read from
 * the shadow like every key of the row's own group. */
static void load_token_at(const ysko_kv_layer* kv, int max_ctx, int kvh, int hd, int rd, const float* rope,
                          int t, int slot_t, int cur_group, float* kd, float* vd);
static void load_token(const ysko_kv_layer* kv, int max_ctx, int kvh, int hd, int rd, const float* rope,
                       int t, int cur_group, float* kd, float* vd) {
  load_token_at(kv, max_ctx, kvh, hd, rd, rope, t, t, cur_group, kd, vd);
}
static void load_token_at(const ysko_kv_layer* kv, int max_ctx, int kvh, int hd, int rd, const float* rope,
                          int t, int slot_t, int cur_group, float* kd, float* vd) {
  if (t / 32 < cur_group) {                         /* 4-bit group: nib*scale + zero, separate mul and add */
    const size_t gb = (size_t)kvh * (max_ctx / 32) + t / 32; const int tt = t & 31;
    for (int ch = 0; ch < hd; ++ch) {
      const uint8_t b = kv->kq[(gb * 32 + tt) * (hd / 2) + (ch >> 1)];
      const int nib = (ch & 1) ? (b >> 4) : (b & 15);
      const float m = (float)nib * h2f(kv->kscale[gb * hd + ch]);
      kd[ch] = m + h2f(kv->kzero[gb * hd + ch]);
    }
  } else {                                          /* the query's own group stays fp16 */
    for (int ch = 0; ch < hd; ++ch) kd[ch] = h2f(kv->kshadow[((size_t)kvh * max_ctx + slot_t) * hd + ch]);
  }
  for (int i = 0; i < rd / 2; ++i) {                /* rotate-half on the first rd dims */
    const float c = rope[((size_t)t * (rd / 2) + i) * 2], s = rope[((size_t)t * (rd / 2) + i) * 2 + 1];
    const float a = kd[i], b = kd[i + rd / 2];
    kd[i] = a * c - b * s; kd[i + rd / 2] = a * s + b * c;
  }
  const size_t slot = (size_t)kvh * max_ctx + slot_t;
  const float vs = h2f(kv->vscale[slot]), vz = h2f(kv->vzero[slot]);
  for (int ch = 0; ch < hd; ++ch) {
    const uint8_t b = kv->vq[slot * (hd / 2) + (ch >> 1)];
    const int nib = (ch & 1) ? (b >> 4) : (b & 15);
    vd[ch] = (float)nib * vs + vz;
  }
}

void ysko_attention_partials(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                             int S, float* pm, float* pl, float* pacc, const float* rope,
                             int hkv, int hq, int hd, int rd, float qscale, int threads) {
  ysko_attention_partials_shard(q16, kv, max_ctx, M, pos0, S, pm, pl, pacc, rope, hkv, hq, hd, rd, qscale, threads, 0, max_ctx);
}

/* The same over a cache that holds only global tokens [shard_start, shard_start+shard_len): local token t is
 * global token t + shard_start; pos0 stays global; rope is the full table.  No reference counterpart (the
 * reference is single-GPU); with shard_start 0 and shard_len max_ctx it is the function above. */
void ysko_attention_partials_shard(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                                   int S, float* pm, float* pl, float* pacc, const float* rope,
                                   int hkv, int hq, int hd, int rd, float qscale, int threads,
                                   int shard_start, int shard_len) {
  const int g = hq / hkv, jobs = M * hkv * S;
  if (rope) rope += (size_t)shard_start * (rd / 2) * 2;
  if (threads < 1) threads = 1;
  #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
  for (int job = 0; job < jobs; ++job) {
    const int r = job / (hkv * S), kvh = (job / S) % hkv, split = job % S;
    const int pos = pos0 + r - shard_start;
    int len = pos + 1; if (len > shard_len) len = shard_len; if (len < 0) len = 0;
    const int per = (len + S - 1) / S;
    const int t0 = split * per, t1 = (t0 + per < len) ? t0 + per : len;
    const int cur_group = pos / 32;
    float* kd = (float*)malloc(sizeof(float) * hd * 2); float* vd = kd + hd;
    float* q = (float*)malloc(sizeof(float) * (size_t)g * hd);
    float* acc = (float*)calloc((size_t)g * hd, sizeof(float));
    float m[8], l[8];
    for (int i = 0; i < g; ++i) { m[i] = -1e30f; l[i] = 0.f;
      for (int d = 0; d < hd; ++d) q[i * hd + d] = h2f(q16[((size_t)r * hq + kvh * g + i) * hd + d]) * qscale; }
    for (int t = t0; t < t1; ++t) {
      load_token(kv, max_ctx, kvh, hd, rd, rope, t, cur_group, kd, vd);
      for (int i = 0; i < g; ++i) {
        float s = 0.f;
        for (int d = 0; d < hd; ++d) s += q[i * hd + d] * kd[d];
        const float mn = fmaxf(m[i], s), a = expf(m[i] - mn), b = expf(s - mn);
        l[i] = l[i] * a + b;
        for (int d = 0; d < hd; ++d) acc[i * hd + d] = acc[i * hd + d] * a + b * vd[d];
        m[i] = mn;
      }
    }
    for (int i = 0; i < g; ++i) {
      const size_t p = ((size_t)r * S + split) * hq + kvh * g + i;
      pm[p] = m[i]; pl[p] = l[i];
      memcpy(pacc + p * hd, acc + (size_t)i * hd, sizeof(float) * hd);
    }
    free(kd); free(q); free(acc);
  }
}

void ysko_combine(const float* pm, const float* pl, const float* pacc, int S, int M, int hq, int g, int hd,
                  const uint16_t* bv, const uint16_t* gate, uint16_t* o16) {
  for (int r = 0; r < M; ++r)
    for (int head = 0; head < hq; ++head) {
      const int kvh = head / g;
      float M2 = -1e30f;
      for (int s = 0; s < S; ++s) M2 = fmaxf(M2, pm[((size_t)r * S + s) * hq + head]);
      for (int d = 0; d < hd; ++d) {
        float L2 = 0.f, o = 0.f;
        for (int s = 0; s < S; ++s) {
          const size_t p = ((size_t)r * S + s) * hq + head;
          const float sc = (pm[p] > -1e29f) ? expf(pm[p] - M2) : 0.f;
          L2 += sc * pl[p]; o += sc * pacc[p * hd + d];
        }
        float y = round_f16(o / L2);
        if (bv) y = y + h2f(bv[kvh * hd + d]);
        if (gate) { const float gt = h2f(gate[((size_t)r * hq + head) * hd + d]); y = y * (1.f / (1.f + expf(-gt))); }
        o16[((size_t)r * hq + head) * hd + d] = ysko_f32_to_f16(y);
      }
    }
}

void ysko_attention_exact(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                          const float* rope, int hkv, int hq, int hd, int rd, float qscale,
                          float* out, int row_begin, int row_end, int threads) {
  ysko_attention_exact_wk(q16, kv, max_ctx, M, pos0, rope, hkv, hq, hd, rd, qscale, out, row_begin, row_end, threads, NULL);
}

/* wk: row -> depth table of a tree-shaped verify pass or NULL (depth = row index): row r sits at position pos0 + wk[r], sees
 * the cached keys 0 .. pos0 + wk[r] - 1 and its own key, stored in slot pos0 + r (src/q35_atx.cu:111-119). */
void ysko_attention_exact_wk(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                             const float* rope, int hkv, int hq, int hd, int rd, float qscale,
                             float* out, int row_begin, int row_end, int threads, const uint8_t* wk) {
  const int g = hq / hkv;
  if (row_begin < 0) row_begin = 0;
  if (row_end > M) row_end = M;
  const int jobs = (row_end - row_begin) * hkv;
  if (threads < 1) threads = 1;
  #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
  for (int job = 0; job < jobs; ++job) {
    const int r = row_begin + job / hkv, kvh = job % hkv;
    const int pos = pos0 + (wk ? (int)wk[r] : r), own = pos0 + r, len = pos + 1, cur_group = pos / 32;
    float* kd = (float*)malloc(sizeof(float) * hd * 2); float* vd = kd + hd;
    float* q = (float*)malloc(sizeof(float) * (size_t)g * hd);
    double* sc = (double*)malloc(sizeof(double) * (size_t)g * len);
    double* acc = (double*)calloc((size_t)g * hd, sizeof(double));
    for (int i = 0; i < g; ++i)
      for (int d = 0; d < hd; ++d) q[i * hd + d] = h2f(q16[((size_t)r * hq + kvh * g + i) * hd + d]) * qscale;
    double mx[8];
    for (int i = 0; i < g; ++i) mx[i] = -1e300;
    for (int t = 0; t < len; ++t) {                                   /* pass 1: scores */
      load_token_at(kv, max_ctx, kvh, hd, rd, rope, t, t == pos ? own : t, cur_group, kd, vd);
      for (int i = 0; i < g; ++i) {
        double s = 0.0;
        for (int d = 0; d < hd; ++d) s += (double)q[i * hd + d] * (double)kd[d];
        sc[(size_t)i * len + t] = s; if (s > mx[i]) mx[i] = s;
      }
    }
    double l[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int t = 0; t < len; ++t) {                                   /* pass 2: weights and values */
      load_token_at(kv, max_ctx, kvh, hd, rd, rope, t, t == pos ? own : t, cur_group, kd, vd);
      for (int i = 0; i < g; ++i) {
        const double p = exp(sc[(size_t)i * len + t] - mx[i]);
        l[i] += p;
        for (int d = 0; d < hd; ++d) acc[i * hd + d] += p * (double)vd[d];
      }
    }
    for (int i = 0; i < g; ++i)
      for (int d = 0; d < hd; ++d) out[((size_t)r * hq + kvh * g + i) * hd + d] = (float)(acc[i * hd + d] / l[i]);
    free(kd); free(q); free(sc); free(acc);
  }
}

/* The int8 input of the next projection: attn_combine_gqa_xform_kernel's tail (src/attention_gqa.cu:135-139) through
 * a8_group512_tail and fwht512_v (src/a8_prologue.cuh:86-98,122-133).  o16 [M][n] fp16 bits, signs [n], qx [M][n], alpha [M][n/512]. */
void ysko_xform_a8(const uint16_t* o16, const int8_t* signs, int8_t* qx, float* alpha, int M, int n) {
  const int ng = n / 512;
  for (int tok = 0; tok < M; ++tok)
    for (int blk = 0; blk < ng; ++blk) {
      float v[512], w[512];
      for (int p = 0; p < 512; ++p) v[p] = h2f(o16[(size_t)tok * n + blk * 512 + p]) * (float)signs[blk * 512 + p];
      for (int h = 1; h < 512; h <<= 1) {                     /* the upper element of a pair gets lower - upper */
        for (int p = 0; p < 512; ++p) { const float q = v[p ^ h]; w[p] = (p & h) ? (q - v[p]) : (v[p] + q); }
        memcpy(v, w, sizeof(v));
      }
      float amax = 0.f;
      for (int p = 0; p < 512; ++p) { v[p] = round_f16(v[p] * 0.044194173824159216f); if (fabsf(v[p]) > amax) amax = fabsf(v[p]); }
      const float al = amax / 127.f;
      alpha[(size_t)tok * ng + blk] = al;
      for (int p = 0; p < 512; ++p) {
        const float r = al > 0.f ? v[p] / al : 0.f;
        /* __float2int_rn: NaN gives 0 and infinities saturate (a group whose transform overflows fp16 has alpha = inf) */
        int q = r != r ? 0 : (r >= 127.f ? 127 : (r <= -127.f ? -127 : (int)nearbyintf(r)));
        qx[(size_t)tok * n + blk * 512 + p] = (int8_t)q;
      }
    }
}

void ysko_merge_triples(const float* parts, int R, int hq, int hd, float* out) {
  const int w = hd + 2;
  for (int head = 0; head < hq; ++head) {
    double M2 = -1e300;
    for (int r = 0; r < R; ++r) { const double m = parts[((size_t)r * hq + head) * w]; if (m > M2) M2 = m; }
    double L = 0.0;
    for (int r = 0; r < R; ++r) { const float* p = parts + ((size_t)r * hq + head) * w;
      if (p[0] > -1e29f) L += exp((double)p[0] - M2) * (double)p[1]; }
    for (int d = 0; d < hd; ++d) {
      double o = 0.0;
      for (int r = 0; r < R; ++r) { const float* p = parts + ((size_t)r * hq + head) * w;
        if (p[0] > -1e29f) o += exp((double)p[0] - M2) * (double)p[2 + d]; }
      out[(size_t)head * hd + d] = (float)(o / L);
    }
  }
}
