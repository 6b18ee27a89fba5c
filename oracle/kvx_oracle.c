/*
 * CPU oracle for the Family-B row codec, step 1 (sign-Hadamard-256 rotation + INT8 rows)
 * -- TEST INFRASTRUCTURE, NOT PRODUCT (same rules as kv4_oracle.c).
 *
 * A scalar C restatement of the reference's src/kvx_codec.cuh as the shipping engine builds it
 * (YSKN_KVX_MODE 3, CMakeLists.txt:56: rotation on, INT8 payload) and of the round trip its probe
 * runs (src/kvx_probe.cu:7-20).  Every operation is a single IEEE fp32 operation, as the reference's
 * explicit __fmul_rn/__fadd_rn/__fsub_rn/__fdiv_rn are; compile with -ffp-contract=off.
 *
 * Pinning: the reference holds no golden vectors for this codec; the restatement is pinned against the
 * reference's own probe (yskn_kvx_probe, compiled from its source into oracle/_ref and run on a GPU)
 * and against tests/golden/kvx_kat.npz, which this oracle produced.
 */
#include "kv4_oracle.h"
#include <math.h>
#include <string.h>

/* src/kvx_codec.cuh:28-32: +-1 from bit 0 of a 32-bit multiply-xorshift hash of d + 1 */
float ysko_kvx_sign(int d) {
  uint32_t x = (uint32_t)d + 1u;
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return (x & 1u) ? -1.f : 1.f;
}

/* src/kvx_codec.cuh:35-49: forward = sign, then butterflies h = 1, 2, ... 128 (the lower index of a pair gets a + b,
 * the upper one gets lower - upper), then x 1/16; inverse = butterflies, x 1/16, then sign. */
static void rotate_row(const float* x, float* y, int inverse) {
  float buf[256], nxt[256];
  for (int d = 0; d < 256; ++d) buf[d] = inverse ? x[d] : x[d] * ysko_kvx_sign(d);
  for (int h = 1; h < 256; h *= 2) {
    for (int d = 0; d < 256; ++d) {
      const float a = buf[d], b = buf[d ^ h];
      nxt[d] = (d & h) ? b - a : a + b;
    }
    memcpy(buf, nxt, sizeof buf);
  }
  for (int d = 0; d < 256; ++d) {
    float v = buf[d] * 0.0625f;
    if (inverse) v = v * ysko_kvx_sign(d);
    y[d] = v;
  }
}

void ysko_kvx_rotate(const float* x, float* y, long rows, int inverse) {
  for (long r = 0; r < rows; ++r) rotate_row(x + r * 256, y + r * 256, inverse);
}

/* src/kvx_codec.cuh:50-70 (INT8 branch): scale = max|x| / 127, q = rne(x / scale) clamped to +-127, 0 for an all-zero row */
void ysko_kvx_encode(const float* x, int8_t* q8, float* scales, long rows) {
  for (long r = 0; r < rows; ++r) {
    float rot[256];
    rotate_row(x + r * 256, rot, 0);
    float amax = 0.f;
    for (int d = 0; d < 256; ++d) { const float a = fabsf(rot[d]); if (a > amax) amax = a; }
    const float sc = amax / 127.f;
    for (int d = 0; d < 256; ++d) {
      int q = sc > 0.f ? (int)nearbyintf(rot[d] / sc) : 0;
      q = q > 127 ? 127 : (q < -127 ? -127 : q);
      q8[r * 256 + d] = (int8_t)q;
    }
    scales[r] = sc;
  }
}

/* src/kvx_probe.cu:15-19: value = (float)q * scale, then the inverse rotation */
void ysko_kvx_decode(const int8_t* q8, const float* scales, float* y, long rows) {
  for (long r = 0; r < rows; ++r) {
    float v[256];
    for (int d = 0; d < 256; ++d) v[d] = (float)q8[r * 256 + d] * scales[r];
    rotate_row(v, y + r * 256, 1);
  }
}

/* Family-B decode attention over INT8 rows, restated from q35_attention_kernel<KV8> (src/q35_kernels.cu:1176-1281):
 * row r at pos0 + r sees keys 0 .. pos0 + r; s_t = (sum_c (q_c * qscale) * k8_tc) * ks_t; softmax; O = sum_t p_t * vs_t * v8_t.
 * q is the rotated query as fp32 values [M][nh][256]; out [M][nh][256] in the rotated basis.  Double accumulation:
 * this is the exact answer the tolerance is measured against, not a bit-level model of the kernel. */
void ysko_kv8_attention_exact(const float* q, const int8_t* k8, const int8_t* v8, const float* ks, const float* vs, int max_ctx,
                              int M, int pos0, int kvh, int nh, float qscale, float* out) {
  const int G = nh / kvh;
  #pragma omp parallel for collapse(2) schedule(dynamic)
  for (int r = 0; r < M; ++r)
    for (int h = 0; h < nh; ++h) {
      const int kv = h / G, len = pos0 + r + 1;
      const float* qr = q + ((size_t)r * nh + h) * 256;
      double mx = -1e300, l = 0.0, o[256];
      for (int d = 0; d < 256; ++d) o[d] = 0.0;
      for (int t = 0; t < len; ++t) {
        const int8_t* kr = k8 + ((size_t)kv * max_ctx + t) * 256;
        double s = 0.0;
        for (int d = 0; d < 256; ++d) s += (double)(qr[d] * qscale) * (double)kr[d];
        s *= (double)ks[(size_t)kv * max_ctx + t];
        if (s > mx) { const double a = exp(mx - s); l *= a; for (int d = 0; d < 256; ++d) o[d] *= a; mx = s; }
        const double p = exp(s - mx);
        l += p;
        const double pv = p * (double)vs[(size_t)kv * max_ctx + t];
        const int8_t* vr = v8 + ((size_t)kv * max_ctx + t) * 256;
        for (int d = 0; d < 256; ++d) o[d] += pv * (double)vr[d];
      }
      for (int d = 0; d < 256; ++d) out[((size_t)r * nh + h) * 256 + d] = (float)(o[d] / l);
    }
}

/* ---- The attention block's row epilogue for INT8 rows, restated from q35_attn_post_kernel (src/q35_kernels.cu:1013-1065)
 * from the point where a thread holds its bf16-rounded projection value y (:1029): the weight path's combine and inverse
 * Hadamard-512 in front of it (:1025-1028) are not part of this path.
 *   V head:  rotate (sign-Hadamard-256) -> INT8 row at position pos                                            (:1030-1038)
 *   Q, K:    ss = y*y summed per warp of 32 channels by an xor-shuffle tree (strides 16, 8, 4, 2, 1), the 8 warp sums
 *            added in order; r = 1/sqrt(tot/256 + eps) with IEEE sqrt and division (the reference's portable-math mode,
 *            src/pm_math.cuh:16; its default rsqrtf is an approximation with no CPU restatement);
 *            xn = bf16(y*r*(1 + w[d])); rotate-half over the first rd channels with the table row of pos, every product
 *            and the sum rounded to bf16; rotate; Q -> bf16, K -> INT8 row                                      (:1043-1064)
 *   gate:    the second 256 outputs of a query head, copied as bf16                                            (:1042)
 * Rows are bf16 bit patterns.  q_rows [M][nh][512], k_rows / v_rows [M][kvh][256]; rope float2 [max_ctx][rd/2]. */
static float bf_bits_to_f(uint16_t b) { union { uint32_t u; float f; } v; v.u = (uint32_t)b << 16; return v.f; }
static uint16_t f_to_bf_bits(float f) {                       /* __float2bfloat16_rn: round to nearest even, NaN kept quiet */
  union { uint32_t u; float f; } v; v.f = f;
  if ((v.u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
  return (uint16_t)((v.u + 0x7fffu + ((v.u >> 16) & 1u)) >> 16);
}
static float rbf(float f) { return bf_bits_to_f(f_to_bf_bits(f)); }

static void post_norm_rope(const uint16_t* y16, const uint16_t* w16, float eps, const float* rope_row, int rd, float* out) {
  float y[256], xn[256], s[8];
  for (int d = 0; d < 256; ++d) y[d] = bf_bits_to_f(y16[d]);
  for (int w = 0; w < 8; ++w) {
    float t[32];
    for (int j = 0; j < 32; ++j) t[j] = y[32 * w + j] * y[32 * w + j];
    for (int o = 16; o; o >>= 1) { float n[32]; for (int j = 0; j < 32; ++j) n[j] = t[j] + t[j ^ o]; memcpy(t, n, sizeof t); }
    s[w] = t[0];
  }
  float tot = 0.f;
  for (int w = 0; w < 8; ++w) tot = tot + s[w];
  const float r = 1.f / sqrtf(tot / 256.f + eps);
  for (int d = 0; d < 256; ++d) xn[d] = rbf((y[d] * r) * (1.f + bf_bits_to_f(w16[d])));
  for (int d = 0; d < 256; ++d) {
    float o = xn[d];
    if (d < rd / 2) { const float c = rope_row[2 * d], sn = rope_row[2 * d + 1]; o = rbf(rbf(xn[d] * c) + rbf(-xn[d + rd / 2] * sn)); }
    else if (d < rd) { const float c = rope_row[2 * (d - rd / 2)], sn = rope_row[2 * (d - rd / 2) + 1]; o = rbf(rbf(xn[d] * c) + rbf(xn[d - rd / 2] * sn)); }
    out[d] = o;
  }
}

void ysko_kvx_attn_post(const uint16_t* q_rows, const uint16_t* k_rows, const uint16_t* v_rows, const uint16_t* qn_w, const uint16_t* kn_w,
                        float eps, int M, int pos0, const float* rope, int rd, int nh, int kvh, int max_ctx,
                        uint16_t* q16, uint16_t* gate16, int8_t* k8, float* ks, int8_t* v8, float* vs) {
  float x[256], rot[256];
  for (int t = 0; t < M; ++t) {
    const int pos = pos0 + t;
    const float* rr = rope + (size_t)pos * (rd / 2) * 2;
    for (int h = 0; h < nh; ++h) {
      const uint16_t* row = q_rows + ((size_t)t * nh + h) * 512;
      post_norm_rope(row, qn_w, eps, rr, rd, x);
      rotate_row(x, rot, 0);
      for (int d = 0; d < 256; ++d) {
        q16[((size_t)t * nh + h) * 256 + d] = f_to_bf_bits(rot[d]);
        gate16[((size_t)t * nh + h) * 256 + d] = row[256 + d];
      }
    }
    for (int h = 0; h < kvh; ++h) {
      const size_t dst = (size_t)h * max_ctx + pos;
      post_norm_rope(k_rows + ((size_t)t * kvh + h) * 256, kn_w, eps, rr, rd, x);
      ysko_kvx_encode(x, k8 + dst * 256, ks + dst, 1);
      for (int d = 0; d < 256; ++d) x[d] = bf_bits_to_f(v_rows[((size_t)t * kvh + h) * 256 + d]);
      ysko_kvx_encode(x, v8 + dst * 256, vs + dst, 1);
    }
  }
}

/* Exact attention over fp32 rows: what the attention over packed trellis rows must equal once every row is unpacked
 * (ysko_tb_unpack).  Same row semantics as q35_attention_kernel (src/q35_kernels.cu:1176-1281): row r at pos0 + r sees keys
 * 0 .. pos0 + r; s_t = sum_c (q_c * qscale) * k_tc; softmax; O = sum_t p_t * v_t.  q [M][nh][256], k / v [kvh][max_ctx][256];
 * out [M][nh][256].  Double accumulation: the oracle for tolerance parity, not a restatement of a summation order. */
void ysko_rows_attention_exact(const float* q, const float* k, const float* v, int max_ctx, int M, int pos0, int kvh, int nh,
                               float qscale, float* out) {
  const int G = nh / kvh;
  #pragma omp parallel for collapse(2) schedule(dynamic)
  for (int r = 0; r < M; ++r)
    for (int h = 0; h < nh; ++h) {
      const int kv = h / G, len = pos0 + r + 1;
      const float* qr = q + ((size_t)r * nh + h) * 256;
      double mx = -1e300, l = 0.0, o[256];
      for (int d = 0; d < 256; ++d) o[d] = 0.0;
      for (int t = 0; t < len; ++t) {
        const float* kr = k + ((size_t)kv * max_ctx + t) * 256;
        double s = 0.0;
        for (int d = 0; d < 256; ++d) s += (double)(qr[d] * qscale) * (double)kr[d];
        if (s > mx) { const double a = exp(mx - s); l *= a; for (int d = 0; d < 256; ++d) o[d] *= a; mx = s; }
        const double p = exp(s - mx);
        l += p;
        const float* vr = v + ((size_t)kv * max_ctx + t) * 256;
        for (int d = 0; d < 256; ++d) o[d] += p * (double)vr[d];
      }
      for (int d = 0; d < 256; ++d) out[((size_t)r * nh + h) * 256 + d] = (float)(o[d] / l);
    }
}
