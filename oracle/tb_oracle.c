/* TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * CPU restatement of the reference's trellis ("CDQ") re-quantisation of a 256-value KV row and of its packed
 * payload, the second step of the Family-B cache codec:
 *   - blob fields ("KVQP v1"):            src/kvq_gpu.cuh:57-68, checks src/engine35.cpp:50-53, src/kvq_fast.hpp:52-76
 *   - residual, low-rank part, rms:       src/kvq_gpu.cuh:70-81      (= tbf_pre, src/kvq_fast.cuh:96-110)
 *   - flat 4-bit mode:                    src/kvq_gpu.cuh:84-87
 *   - Viterbi over 4 chains of 64 steps, 256 states, kk new bits per step, best of nm scale multipliers:
 *                                         src/kvq_gpu.cuh:89-139     (= tbf_chain + tbf_sel, src/kvq_fast.cuh:113-214)
 *   - fields, MSB-first bit packing, side words: src/kvq_fast.cuh:207-232
 * Block reductions follow the reference's order (tb_sum, src/kvq_gpu.cuh:32-42): a xor-butterfly over each run of 32
 * values, then the eight run sums added in order; every operation that the reference writes as an _rn intrinsic is a
 * plain IEEE float operation here (compile with -ffp-contract=off).
 * Pinned against the reference's own probe yskn_tb_probe (src/kvx_probe.cu:40-62) on a GPU by tests/test_ref_pin.py. */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "kv4_oracle.h"

static unsigned u16(const uint8_t* p) { return (unsigned)p[0] | ((unsigned)p[1] << 8); }
static unsigned u32(const uint8_t* p) { return u16(p) | (u16(p + 2) << 16); }
static float f32(const uint8_t* p) { const unsigned u = u32(p); float f; memcpy(&f, &u, 4); return f; }
static float h2f(unsigned h) { return ysko_f16_to_f32((uint16_t)h); }
static float f16r(float v) { return ysko_f16_to_f32(ysko_f32_to_f16(v)); }

static float warp_sum(const float* v) {                 /* v[32]: the butterfly every lane of a warp ends with */
  float a[32], b[32];
  memcpy(a, v, sizeof(a));
  for (int o = 16; o; o >>= 1) { for (int i = 0; i < 32; ++i) b[i] = a[i] + a[i ^ o]; memcpy(a, b, sizeof(a)); }
  return a[0];
}
static float block_sum(const float* v) {                /* v[256] */
  float t = 0.f;
  for (int w = 0; w < 8; ++w) t = t + warp_sum(v + 32 * w);
  return t;
}

/* Header check of src/engine35.cpp:50-53 and the table check of :53 / src/kvq_fast.hpp:66-69.  0 = a blob the reference accepts. */
int ysko_tb_check_blob(const uint8_t* b, size_t n) {
  if (n < 100 || memcmp(b, "KVQP", 4) != 0 || u16(b + 4) != 1 || u16(b + 6) != 96 || u32(b + 8) != n) return 1;
  if (u16(b + 16) != 256 || u16(b + 18) != 16 || u16(b + 20) != 4 || u32(b + 28) != 128u) return 2;
  const unsigned nt = u16(b + 22), off_t = u32(b + 36);
  for (unsigned t = 0; t < nt; ++t) {
    const size_t o = u32(b + off_t + 4 * t);
    if (o + 12 + 512 > n || b[o] != 8 || b[o + 2] != 64 || b[o + 3] != 8) return 3;
    for (int s = 0; s < 256; ++s) { const int c = (int)(int16_t)u16(b + o + 12 + 2 * s); if (c > 1100 || c < -1100) return 4; }
  }
  const unsigned nm = u16(b + 24);
  if (nm < 1 || nm > 16) return 5;
  return 0;
}

/* One row.  y_fq[256]: the re-quantised row (what tb_fakequant returns).  If the row is packed (not a guard row):
 * fields[256] (kb-bit values), pay[8*kb] 32-bit words (MSB-first bit stream), side[0] = scale bits, side[1] = the two fp16
 * low-rank coefficients, *kb_out = bits per field; otherwise *kb_out = 0. */
static void tb_row(const uint8_t* b, const float* y, int g, int pos, float* y_fq, uint8_t* fields, uint32_t* pay, uint32_t* side, int* kb_out) {
  const int nm = (int)u16(b + 24);
  const unsigned off_m = u32(b + 32), off_t = u32(b + 36), off_g = u32(b + 40), ngrp = u32(b + 28);
  const int okg = (unsigned)g < ngrp;
  const unsigned go = okg ? u32(b + off_g + 4u * (unsigned)g) : 0u;
  const int mode = okg ? b[go] : 0, kk = okg ? b[go + 1] : 4, tix = okg ? b[go + 2] : 0, guard = okg ? b[go + 3] : 0, m = okg ? b[go + 4] : 0,
            has_mu = okg ? b[go + 5] : 0;
  *kb_out = 0;
  if (!okg || pos < guard) { memcpy(y_fq, y, 256 * sizeof(float)); return; }
  const uint8_t* mup = b + go + 8;
  const uint8_t* Up = mup + (has_mu ? 512 : 0);
  float r[256], mud[256], uj[2][256], cj[2] = {0.f, 0.f}, tmp[256];
  for (int d = 0; d < 256; ++d) { mud[d] = has_mu ? h2f(u16(mup + 2 * d)) : 0.f; r[d] = has_mu ? y[d] - mud[d] : y[d]; }
  for (int j = 0; j < 2 && j < m; ++j) {
    for (int d = 0; d < 256; ++d) { uj[j][d] = h2f(u16(Up + 2 * (j * 256 + d))); tmp[d] = r[d] * uj[j][d]; }
    cj[j] = f16r(block_sum(tmp));
    for (int d = 0; d < 256; ++d) r[d] = r[d] - cj[j] * uj[j][d];
  }
  for (int d = 0; d < 256; ++d) tmp[d] = r[d] * r[d];
  float rms = sqrtf(block_sum(tmp) / 256.f); if (rms == 0.f) rms = 1.f;
  float xq[256], psc = 1.f; int kb = 4;
  if (mode == 1) {                                      /* flat: symmetric 4-bit codes, one scale */
    float am = 0.f;
    for (int d = 0; d < 256; ++d) am = fmaxf(am, fabsf(r[d]));
    float s7 = am / 7.f; if (s7 == 0.f) s7 = 1.f;
    for (int d = 0; d < 256; ++d) { float q = rintf(r[d] / s7); q = fminf(fmaxf(q, -7.f), 7.f); xq[d] = q * s7; fields[d] = (uint8_t)((int)q + 8); }
    psc = s7; kb = 4;
  } else {                                              /* trellis-coded */
    const unsigned to = u32(b + off_t + 4u * (unsigned)tix);
    const float gain = f32(b + to + 4);
    const int Kq = 1 << kk, UU = 256 >> kk;
    int ci[256]; float cdec[256];
    for (int d = 0; d < 256; ++d) { ci[d] = (int)(int16_t)u16(b + to + 12 + 2 * d); cdec[d] = ((float)ci[d] * 0.00390625f) * gain; }
    float best_e = 0.f; int have = 0; uint8_t best_st[256]; float best_s = 1.f;
    static const int INF = 0x40000000;
    for (int mi = 0; mi < nm; ++mi) {
      float s = f16r(rms * f32(b + off_m + 4u * (unsigned)mi)); if (s == 0.f) s = 1.f;
      int xi[256]; uint8_t st_of[256]; float rec[256];
      for (int d = 0; d < 256; ++d) { const float t = rintf((r[d] / s) * 256.f); xi[d] = (int)fminf(fmaxf(t, -2048.f), 2048.f); }
      for (int c = 0; c < 4; ++c) {
        int cost[2][256]; uint8_t bp[64][256];
        for (int d = 0; d < 256; ++d) cost[0][d] = d == 0 ? 0 : INF;
        for (int t = 0; t < 64; ++t) {
          const int* cp = cost[t & 1]; int* cn = cost[(t + 1) & 1];
          for (int d = 0; d < 256; ++d) {
            const int uidx = d >> kk;
            int mn = cp[uidx], jb = 0;
            for (int j = 1; j < Kq; ++j) { const int cc = cp[j * UU + uidx]; if (cc < mn) { mn = cc; jb = j; } }
            const int dx = xi[c * 64 + t] - ci[d];
            cn[d] = dx * dx + mn; bp[t][d] = (uint8_t)jb;
          }
        }
        int st = 0; unsigned long long mk = ~0ull;
        for (int d = 0; d < 256; ++d) { const unsigned long long key = ((unsigned long long)(unsigned)cost[0][d] << 8) | (unsigned long long)d; if (key < mk) { mk = key; st = d; } }
        for (int t = 63; t >= 0; --t) {
          rec[c * 64 + t] = cdec[st] * s; st_of[c * 64 + t] = (uint8_t)st;
          const int j = bp[t][st];
          st = (j << (8 - kk)) | (st >> kk);
        }
      }
      for (int d = 0; d < 256; ++d) { const float dd = r[d] - rec[d]; tmp[d] = dd * dd; }
      const float e = block_sum(tmp);
      if (!have || e < best_e) { have = 1; best_e = e; best_s = s; memcpy(best_st, st_of, 256); memcpy(xq, rec, sizeof(rec)); }
    }
    for (int d = 0; d < 256; ++d) fields[d] = (uint8_t)(best_st[d] & (Kq - 1));
    psc = best_s; kb = kk;
  }
  for (int d = 0; d < 256; ++d) {
    float x = xq[d];
    for (int j = 0; j < 2 && j < m; ++j) x = x + cj[j] * uj[j][d];
    if (has_mu) x = x + mud[d];
    y_fq[d] = x;
  }
  for (int w = 0; w < 8 * kb; ++w) {                    /* src/kvq_fast.cuh:228-232: field bits MSB first, 32 per word */
    uint32_t v = 0u;
    for (int i = 0; i < 32; ++i) { const int gbit = 32 * w + i, e = gbit / kb, jb = gbit - e * kb; v |= (((uint32_t)fields[e] >> (kb - 1 - jb)) & 1u) << (31 - i); }
    pay[w] = v;
  }
  memcpy(&side[0], &psc, 4);
  side[1] = (uint32_t)ysko_f32_to_f16(cj[0]) | ((uint32_t)ysko_f32_to_f16(cj[1]) << 16);
  *kb_out = kb;
}

/* rows of 256 floats; grp[r] = group record of the row ((layer*4 + kv_head)*2 + kind), pos[r] = its position.
 * pay: [rows][40] words (8*kb used), side: [rows][2], kb: [rows] (0 = guard row, stored unpacked). */
void ysko_tb_encode(const uint8_t* blob, const float* x, const int* grp, const int* pos, int rows,
                    float* y_fq, uint8_t* fields, uint32_t* pay, uint32_t* side, int* kb) {
  #pragma omp parallel for schedule(dynamic, 1)
  for (int r = 0; r < rows; ++r) {
    memset(pay + (size_t)r * 40, 0, 40 * sizeof(uint32_t)); side[2 * r] = side[2 * r + 1] = 0u; memset(fields + (size_t)r * 256, 0, 256);
    tb_row(blob, x + (size_t)r * 256, grp[r], pos[r], y_fq + (size_t)r * 256, fields + (size_t)r * 256, pay + (size_t)r * 40, side + 2 * r, kb + r);
  }
}

/* Inverse of the packing and of the code: payload words + scale -> the trellis part of the row (before the low-rank part and
 * the mean are added back), by re-running the shift register from state 0 at the start of each chain of 64
 * (the decode records of src/kvq_atxpk.hpp:25-58 tabulate exactly this product). */
void ysko_tb_decode_fields(const uint8_t* blob, int g, const uint32_t* pay, float scale, float* xq) {
  const unsigned off_t = u32(blob + 36), off_g = u32(blob + 40);
  const unsigned go = u32(blob + off_g + 4u * (unsigned)g);
  const int mode = blob[go], kk = blob[go + 1], tix = blob[go + 2], kb = mode == 1 ? 4 : kk;
  const unsigned to = u32(blob + off_t + 4u * (unsigned)tix);
  const float gain = mode == 0 ? f32(blob + to + 4) : 1.f;
  int st = 0;
  for (int e = 0; e < 256; ++e) {
    int f = 0;
    for (int jb = 0; jb < kb; ++jb) { const int gbit = e * kb + jb; f = (f << 1) | (int)((pay[gbit >> 5] >> (31 - (gbit & 31))) & 1u); }
    if (mode == 1) { xq[e] = (float)(f - 8) * scale; continue; }
    if ((e & 63) == 0) st = 0;
    st = ((st << kk) | f) & 255;
    const int ci = (int)(int16_t)u16(blob + to + 12 + 2 * st);
    xq[e] = (((float)ci * 0.00390625f) * gain) * scale;
  }
}

/* Packed rows back to values (tba_unpack_kernel, src/kvq_attn.cuh:39-72): a value's state is the 8-bit window of the row's
 * bit stream that ends with its field (shorter at the start of a chain of 64), the code of that state times gain/256 times
 * the row's scale, then the low-rank part (fp16 coefficients from the side word) and the mean are added back.  Rows that
 * were not packed (below the group's guard position, or a group the blob does not have) keep yin. */
void ysko_tb_unpack(const uint8_t* blob, const int* grp, const int* pos, const uint32_t* pay, int stride_words, const uint32_t* side,
                    const float* yin, float* y, int rows) {
  const unsigned ngrp = u32(blob + 28), off_t = u32(blob + 36), off_g = u32(blob + 40);
  for (int r = 0; r < rows; ++r) {
    memcpy(y + (size_t)r * 256, yin + (size_t)r * 256, 256 * sizeof(float));
    const int g = grp[r];
    if ((unsigned)g >= ngrp) continue;
    const unsigned go = u32(blob + off_g + 4u * (unsigned)g);
    const int mode = blob[go], kk = blob[go + 1], tix = blob[go + 2], guard = blob[go + 3], m = blob[go + 4], has_mu = blob[go + 5];
    if (pos[r] < guard || mode > 1) continue;
    const uint32_t* wp = pay + (size_t)r * stride_words;
    float s; memcpy(&s, &side[2 * r], 4);
    const unsigned pc = side[2 * r + 1];
    const int kb = mode == 1 ? 4 : kk;
    const unsigned to = u32(blob + off_t + 4u * (unsigned)tix);
    const uint8_t* mup = blob + go + 8; const uint8_t* Up = mup + (has_mu ? 512 : 0);
    for (int d = 0; d < 256; ++d) {
      const int endb = kb * (d + 1), first = kb * (d & ~63), lo = mode == 1 ? endb - 4 : (endb - 8 > first ? endb - 8 : first);
      unsigned v = 0;
      for (int bit = lo; bit < endb; ++bit) v = (v << 1) | ((wp[bit >> 5] >> (31 - (bit & 31))) & 1u);
      float xq;
      if (mode == 1) xq = (float)((int)v - 8) * s;
      else { const int ci = (int)(int16_t)u16(blob + to + 12 + 2 * v); xq = (((float)ci * 0.00390625f) * f32(blob + to + 4)) * s; }
      float x = xq;
      if (m > 0) x = x + h2f(pc & 0xffffu) * h2f(u16(Up + 2 * d));
      if (m > 1) x = x + h2f(pc >> 16) * h2f(u16(Up + 2 * (256 + d)));
      if (has_mu) x = x + h2f(u16(mup + 2 * d));
      y[(size_t)r * 256 + d] = x;
    }
  }
}
