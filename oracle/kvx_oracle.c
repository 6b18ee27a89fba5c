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
