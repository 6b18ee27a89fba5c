// Family-B cache codec, step 2 (sm_100a): trellis ("CDQ") re-quantisation of 256-value KV rows and their packed payload.
//
// Arithmetic and formats are the reference's, bit for bit: tb_fakequant (src/kvq_gpu.cuh:54-148) = tbf_pre / tbf_chain /
// tbf_sel (src/kvq_fast.cuh:96-232), blob fields "KVQP v1" (src/kvq_gpu.cuh:57-68, src/engine35.cpp:50-53).
//   row -> (- mean) -> up to two low-rank projections (fp16 coefficients) -> rms
//   for each of nm scale multipliers: s = fp16(rms * mult); x_i = clamp(rint(r / s * 256), +-2048); for each of the 4 chains
//   of 64 values a Viterbi search over 256 states (an 8-bit shift register that takes kk = 3 / 4 / 5 new bits per step;
//   cost (x_i - code[state])^2); the multiplier with the smallest squared error wins (first on ties)
//   payload: the kk new bits of every step, MSB first, 8*kk 32-bit words per row; side words: scale, two fp16 coefficients.
// Sums over a row follow the reference's order (a xor-butterfly over each run of 32 values, then the eight run sums in
// order), and every product that feeds a rounding decision is an explicit _rn operation, so no FMA contraction moves a bit.
//
// Work split (not the reference's): the reference runs one 256-thread block per (row, multiplier, chain) with a block
// barrier per trellis step.  Here ONE WARP owns a (row, multiplier, chain) search: a lane owns eight consecutive states,
// which all share one predecessor set, so a step is one vector read of that set (the costs are kept transposed in the
// warp's own shared memory so that the set is contiguous), one minimum, eight squared differences and eight stores, with
// a warp-level barrier only.  A second kernel, one block per row, picks the multiplier, rebuilds the row and packs it.
#include "kv4_common.cuh"
#include <cstring>

namespace kv4 {
namespace {

__device__ __forceinline__ unsigned tb_u16(const uint8_t* p) { return (unsigned)p[0] | ((unsigned)p[1] << 8); }
__device__ __forceinline__ unsigned tb_u32(const uint8_t* p) { return tb_u16(p) | (tb_u16(p + 2) << 16); }
__device__ __forceinline__ float tb_f32(const uint8_t* p) { return __uint_as_float(tb_u32(p)); }
__device__ __forceinline__ float tb_f16r(float v) { return __half2float(__float2half_rn(v)); }

struct TbGroup { int ok, mode, kk, tix, guard, m, has_mu; unsigned go, off_m, off_t; };
__device__ __forceinline__ TbGroup tb_group(const uint8_t* b, int g) {
  TbGroup P;
  P.off_m = tb_u32(b + 32); P.off_t = tb_u32(b + 36);
  const unsigned off_g = tb_u32(b + 40), ngrp = tb_u32(b + 28);
  P.ok = (unsigned)g < ngrp;
  P.go = P.ok ? tb_u32(b + off_g + 4u * (unsigned)g) : 0u;
  P.mode = P.ok ? b[P.go] : 0; P.kk = P.ok ? b[P.go + 1] : 4; P.tix = P.ok ? b[P.go + 2] : 0; P.guard = P.ok ? b[P.go + 3] : 0;
  P.m = P.ok ? b[P.go + 4] : 0; P.has_mu = P.ok ? b[P.go + 5] : 0;
  return P;
}

// ---- a warp's view of a row: lane holds elements 32*w + lane, w = 0..7 (one per run of the reference's reduction)
__device__ __forceinline__ float warp_rowsum(const float (&v)[8]) {
  float t = 0.f;
  #pragma unroll
  for (int w = 0; w < 8; ++w) {
    float a = v[w];
    #pragma unroll
    for (int o = 16; o; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    t = __fadd_rn(t, a);
  }
  return t;
}
struct RowPre { float r[8], mud[8], u0[8], u1[8], c0, c1, rms; };
__device__ __forceinline__ void warp_pre(const uint8_t* b, const TbGroup& P, const float* y, int lane, RowPre& Q) {
  const uint8_t* mup = b + P.go + 8;
  const uint8_t* Up = mup + (P.has_mu ? 512 : 0);
  float tmp[8];
  Q.c0 = Q.c1 = 0.f;
  #pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int d = 32 * w + lane;
    Q.mud[w] = P.has_mu ? __half2float(__ushort_as_half((unsigned short)tb_u16(mup + 2 * d))) : 0.f;
    Q.r[w] = P.has_mu ? __fsub_rn(y[d], Q.mud[w]) : y[d];
    Q.u0[w] = P.m > 0 ? __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * d))) : 0.f;
    Q.u1[w] = P.m > 1 ? __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * (256 + d)))) : 0.f;
  }
  if (P.m > 0) {
    #pragma unroll
    for (int w = 0; w < 8; ++w) tmp[w] = __fmul_rn(Q.r[w], Q.u0[w]);
    Q.c0 = tb_f16r(warp_rowsum(tmp));
    #pragma unroll
    for (int w = 0; w < 8; ++w) Q.r[w] = __fsub_rn(Q.r[w], __fmul_rn(Q.c0, Q.u0[w]));
  }
  if (P.m > 1) {
    #pragma unroll
    for (int w = 0; w < 8; ++w) tmp[w] = __fmul_rn(Q.r[w], Q.u1[w]);
    Q.c1 = tb_f16r(warp_rowsum(tmp));
    #pragma unroll
    for (int w = 0; w < 8; ++w) Q.r[w] = __fsub_rn(Q.r[w], __fmul_rn(Q.c1, Q.u1[w]));
  }
  #pragma unroll
  for (int w = 0; w < 8; ++w) tmp[w] = __fmul_rn(Q.r[w], Q.r[w]);
  Q.rms = __fsqrt_rn(__fdiv_rn(warp_rowsum(tmp), 256.f));
  if (Q.rms == 0.f) Q.rms = 1.f;
}

constexpr int TB_WARPS = 8;                              // searches per block
struct alignas(16) TbWarpSmem { int cost[2][256]; uint8_t bp[64][32]; uint8_t st[64]; };

struct TbP {
  const uint8_t* blob; int nm; const float* x; const int* grp; const int* pos; int rows;
  float* y; uint8_t* pay; int pay_stride; uint32_t* side; uint8_t* scr_states; float* scr_err;
};

// One warp per (row, multiplier, chain).  States of the best path -> scr_states[row][mi][64*c ..], the two half-chain error
// sums -> scr_err[row][mi][2c], [2c+1] (the runs of the reference's error sum, src/kvq_fast.cuh:140-147).
template <int KK>
__device__ __forceinline__ void tb_search(TbWarpSmem& S, const uint8_t* b, const TbGroup& P, const RowPre& Q, float s, int c, int lane,
                                          uint8_t* so, float* wo) {
  constexpr int KQ = 1 << KK, UU = 256 >> KK, SH = 8 - KK;
  const unsigned to = tb_u32(b + P.off_t + 4u * (unsigned)P.tix);
  const float gain = tb_f32(b + to + 4);
  int ci[8];                                             // codes of this lane's states d = 8*lane + e
  #pragma unroll
  for (int e = 0; e < 8; ++e) ci[e] = (int)(short)tb_u16(b + to + 12 + 2 * (8 * lane + e));
  // this chain's 64 scaled values: lane holds steps lane and lane + 32
  const float ra = Q.r[2 * c], rb = Q.r[2 * c + 1];
  const int xa = (int)fminf(fmaxf(rintf(__fmul_rn(__fdiv_rn(ra, s), 256.f)), -2048.f), 2048.f);
  const int xb = (int)fminf(fmaxf(rintf(__fmul_rn(__fdiv_rn(rb, s), 256.f)), -2048.f), 2048.f);
  // transposed cost layout: state p sits at (p % UU) * KQ + p / UU, so the predecessors {j*UU + u} of group u are contiguous
  const int u = (8 * lane) >> KK;                        // the predecessor group of all eight states of this lane
  int widx[8];
  #pragma unroll
  for (int e = 0; e < 8; ++e) { const int d = 8 * lane + e; widx[e] = (d & (UU - 1)) * KQ + (d >> SH); }
  #pragma unroll
  for (int e = 0; e < 8; ++e) S.cost[0][widx[e]] = (8 * lane + e == 0) ? 0 : 0x40000000;
  __syncwarp();
  #pragma unroll 1
  for (int t = 0; t < 64; ++t) {
    const int4* cp = reinterpret_cast<const int4*>(&S.cost[t & 1][u * KQ]);
    int mn = 0x7fffffff, jb = 0;
    #pragma unroll
    for (int q = 0; q < KQ / 4; ++q) {                   // first minimum in predecessor order (src/kvq_gpu.cuh:101-102)
      const int4 v = cp[q];
      if (v.x < mn) { mn = v.x; jb = 4 * q; }
      if (v.y < mn) { mn = v.y; jb = 4 * q + 1; }
      if (v.z < mn) { mn = v.z; jb = 4 * q + 2; }
      if (v.w < mn) { mn = v.w; jb = 4 * q + 3; }
    }
    const int xt = __shfl_sync(0xffffffffu, t < 32 ? xa : xb, t & 31);
    int* cn = S.cost[(t + 1) & 1];
    #pragma unroll
    for (int e = 0; e < 8; ++e) { const int dx = xt - ci[e]; cn[widx[e]] = dx * dx + mn; }
    if (((8 * lane) & (KQ - 1)) == 0) S.bp[t][u] = (uint8_t)jb;
    __syncwarp();
  }
  // best final state: smallest (cost, state)
  unsigned long long key = ~0ull;
  #pragma unroll
  for (int e = 0; e < 8; ++e) { const unsigned long long k = ((unsigned long long)(unsigned)S.cost[0][widx[e]] << 8) | (unsigned long long)(8 * lane + e); key = k < key ? k : key; }
  #pragma unroll
  for (int o = 16; o; o >>= 1) { const unsigned long long k2 = __shfl_xor_sync(0xffffffffu, key, o); key = k2 < key ? k2 : key; }
  if (lane == 0) {
    int st = (int)(key & 255ull);
    for (int t = 63; t >= 0; --t) { S.st[t] = (uint8_t)st; const int j = S.bp[t][st >> KK]; st = (j << SH) | (st >> KK); }
  }
  __syncwarp();
  #pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int stt = S.st[lane + 32 * h];
    const int cs = (int)(short)tb_u16(b + to + 12 + 2 * stt);
    const float rec = __fmul_rn(__fmul_rn(__fmul_rn((float)cs, 0.00390625f), gain), s);
    const float dd = __fsub_rn(h ? rb : ra, rec);
    float v = __fmul_rn(dd, dd);
    #pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) wo[h] = v;
    so[lane + 32 * h] = (uint8_t)stt;
  }
  __syncwarp();
}

__global__ void __launch_bounds__(TB_WARPS * 32) tb_search_kernel(TbP A) {
  __shared__ TbWarpSmem S[TB_WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long job = (long long)blockIdx.x * TB_WARPS + warp;
  if (job >= (long long)A.rows * A.nm * 4) return;
  const int row = (int)(job / (A.nm * 4)), rem = (int)(job - (long long)row * (A.nm * 4)), mi = rem >> 2, c = rem & 3;
  const TbGroup P = tb_group(A.blob, A.grp[row]);
  if (!P.ok || A.pos[row] < P.guard || P.mode != 0) return;           // stored as is, or flat codes: no search
  RowPre Q;
  warp_pre(A.blob, P, A.x + (size_t)row * 256, lane, Q);
  float s = tb_f16r(__fmul_rn(Q.rms, tb_f32(A.blob + P.off_m + 4u * (unsigned)mi)));
  if (s == 0.f) s = 1.f;
  uint8_t* so = A.scr_states + ((size_t)row * A.nm + mi) * 256 + 64 * c;
  float* wo = A.scr_err + ((size_t)row * A.nm + mi) * 8 + 2 * c;
  if (P.kk == 3) tb_search<3>(S[warp], A.blob, P, Q, s, c, lane, so, wo);
  else if (P.kk == 4) tb_search<4>(S[warp], A.blob, P, Q, s, c, lane, so, wo);
  else if (P.kk == 5) tb_search<5>(S[warp], A.blob, P, Q, s, c, lane, so, wo);
  else { so[lane] = 0; so[lane + 32] = 0; if (lane == 0) { wo[0] = 3.0e38f; wo[1] = 3.0e38f; } }   // a step width the code does not have: never the best
}

// One block per row: pick the multiplier, rebuild the row, pack fields and side words.
__global__ void __launch_bounds__(256) tb_select_kernel(TbP A) {
  __shared__ uint8_t fld[256];
  __shared__ float red[8];
  const int row = blockIdx.x, d = threadIdx.x, warp = d >> 5, lane = d & 31;
  const uint8_t* b = A.blob;
  const TbGroup P = tb_group(b, A.grp[row]);
  const float yv = A.x[(size_t)row * 256 + d];
  if (!P.ok || A.pos[row] < P.guard) { if (A.y) A.y[(size_t)row * 256 + d] = yv; return; }
  auto bsum = [&](float v) -> float {                    // the reference's block sum (src/kvq_fast.cuh:33-43)
    #pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    #pragma unroll
    for (int w = 0; w < 8; ++w) t = __fadd_rn(t, red[w]);
    __syncthreads();
    return t;
  };
  const uint8_t* mup = b + P.go + 8;
  const uint8_t* Up = mup + (P.has_mu ? 512 : 0);
  float r = yv, mud = 0.f, u0 = 0.f, u1 = 0.f, c0 = 0.f, c1 = 0.f;
  if (P.has_mu) { mud = __half2float(__ushort_as_half((unsigned short)tb_u16(mup + 2 * d))); r = __fsub_rn(yv, mud); }
  if (P.m > 0) { u0 = __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * d))); c0 = tb_f16r(bsum(__fmul_rn(r, u0))); r = __fsub_rn(r, __fmul_rn(c0, u0)); }
  if (P.m > 1) { u1 = __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * (256 + d)))); c1 = tb_f16r(bsum(__fmul_rn(r, u1))); r = __fsub_rn(r, __fmul_rn(c1, u1)); }
  float rms = __fsqrt_rn(__fdiv_rn(bsum(__fmul_rn(r, r)), 256.f)); if (rms == 0.f) rms = 1.f;
  float xq, psc; int field, kb;
  if (P.mode == 1) {                                     // flat 4-bit codes (src/kvq_fast.cuh:193-198)
    float am = fabsf(r);
    #pragma unroll
    for (int o = 16; o; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if (lane == 0) red[warp] = am;
    __syncthreads();
    am = 0.f;
    #pragma unroll
    for (int w = 0; w < 8; ++w) am = fmaxf(am, red[w]);
    __syncthreads();
    float s7 = __fdiv_rn(am, 7.f); if (s7 == 0.f) s7 = 1.f;
    float q = rintf(__fdiv_rn(r, s7)); q = fminf(fmaxf(q, -7.f), 7.f);
    xq = __fmul_rn(q, s7); field = (int)q + 8; psc = s7; kb = 4;
  } else {
    const float* W = A.scr_err + (size_t)row * A.nm * 8;
    float best_e = 0.f; int best = 0; bool have = false;
    for (int mi = 0; mi < A.nm; ++mi) {
      float e = 0.f;
      #pragma unroll
      for (int w = 0; w < 8; ++w) e = __fadd_rn(e, W[mi * 8 + w]);
      if (!have || e < best_e) { have = true; best_e = e; best = mi; }
    }
    float s = tb_f16r(__fmul_rn(rms, tb_f32(b + P.off_m + 4u * (unsigned)best))); if (s == 0.f) s = 1.f;
    const unsigned to = tb_u32(b + P.off_t + 4u * (unsigned)P.tix);
    const float gain = tb_f32(b + to + 4);
    const int st = A.scr_states[((size_t)row * A.nm + best) * 256 + d];
    const int cs = (int)(short)tb_u16(b + to + 12 + 2 * st);
    xq = __fmul_rn(__fmul_rn(__fmul_rn((float)cs, 0.00390625f), gain), s);
    field = st & ((1 << P.kk) - 1); psc = s; kb = P.kk;
  }
  float x = xq;
  if (P.m > 0) x = __fadd_rn(x, __fmul_rn(c0, u0));
  if (P.m > 1) x = __fadd_rn(x, __fmul_rn(c1, u1));
  if (P.has_mu) x = __fadd_rn(x, mud);
  if (A.y) A.y[(size_t)row * 256 + d] = x;
  if (A.pay) {
    fld[d] = (uint8_t)field;
    __syncthreads();
    if (d < 8 * kb) {                                    // MSB-first bit stream, 32 bits per word (src/kvq_fast.cuh:228-232)
      unsigned w = 0u;
      for (int i = 0; i < 32; ++i) { const int gbit = 32 * d + i, e = gbit / kb, jb = gbit - e * kb; w |= (((unsigned)fld[e] >> (kb - 1 - jb)) & 1u) << (31 - i); }
      reinterpret_cast<unsigned*>(A.pay + (size_t)row * A.pay_stride)[d] = w;
    }
    if (d == 0 && A.side) {
      A.side[2 * row] = __float_as_uint(psc);
      A.side[2 * row + 1] = (unsigned)__half_as_ushort(__float2half_rn(c0)) | ((unsigned)__half_as_ushort(__float2half_rn(c1)) << 16);
    }
  }
}

// Packed rows back to values (the reference's tba_unpack_kernel, src/kvq_attn.cuh:39-72): one warp per row.  The state of a
// value is the 8-bit window of the row's bit stream that ends with its field (shorter at the start of a chain of 64), so
// every value decodes on its own: two payload words from the warp's shared-memory copy of the row, one funnel shift, one
// code lookup.  Lane owns values 32*w + lane, so the stores of a warp are contiguous.
struct TbDecP { const uint8_t* blob; const int* grp; const int* pos; const uint8_t* pay; int pay_stride; const uint32_t* side; const float* yin; float* y; int rows; };
__global__ void __launch_bounds__(256) tb_unpack_kernel(TbDecP A) {
  __shared__ unsigned s_w[8][44];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, row = blockIdx.x * 8 + warp;
  if (row >= A.rows) return;
  const uint8_t* b = A.blob;
  const TbGroup P = tb_group(b, A.grp[row]);
  const bool packed = P.ok && A.pos[row] >= P.guard && P.mode <= 1;
  if (!packed) {
    #pragma unroll
    for (int w = 0; w < 8; ++w) A.y[(size_t)row * 256 + 32 * w + lane] = A.yin ? A.yin[(size_t)row * 256 + 32 * w + lane] : 0.f;
    return;
  }
  const int kb = P.mode == 1 ? 4 : P.kk, nw = 8 * kb;
  const unsigned* wp = reinterpret_cast<const unsigned*>(A.pay + (size_t)row * A.pay_stride);
  for (int i = lane; i < 44; i += 32) s_w[warp][i] = i < nw ? wp[i] : 0u;
  __syncwarp();
  const float s = __uint_as_float(A.side[2 * (size_t)row]);
  const unsigned pc = A.side[2 * (size_t)row + 1];
  const unsigned to = tb_u32(b + P.off_t + 4u * (unsigned)P.tix);
  const float gain = P.mode == 0 ? tb_f32(b + to + 4) : 1.f;
  const uint8_t* mup = b + P.go + 8;
  const uint8_t* Up = mup + (P.has_mu ? 512 : 0);
  const float c0 = __half2float(__ushort_as_half((unsigned short)(pc & 0xffffu))), c1 = __half2float(__ushort_as_half((unsigned short)(pc >> 16)));
  #pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int d = 32 * w + lane, endb = kb * (d + 1), first = kb * (d & ~63);
    const int lo = P.mode == 1 ? endb - 4 : max(endb - 8, first), len = endb - lo;
    const unsigned hiw = s_w[warp][lo >> 5], low = s_w[warp][(lo >> 5) + 1];
    const unsigned v = __funnelshift_l(low, hiw, lo & 31) >> (32 - len);     // bits [lo, lo + len) of the MSB-first stream
    float xq;
    if (P.mode == 1) xq = __fmul_rn((float)((int)v - 8), s);
    else xq = __fmul_rn(__fmul_rn(__fmul_rn((float)(int)(short)tb_u16(b + to + 12 + 2 * v), 0.00390625f), gain), s);
    float x = xq;
    if (P.m > 0) x = __fadd_rn(x, __fmul_rn(c0, __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * d)))));
    if (P.m > 1) x = __fadd_rn(x, __fmul_rn(c1, __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * (256 + d))))));
    if (P.has_mu) x = __fadd_rn(x, __half2float(__ushort_as_half((unsigned short)tb_u16(mup + 2 * d))));
    A.y[(size_t)row * 256 + d] = x;
  }
}


// ---------------------------------------------------------------------------------------------------------------------
// Decode attention straight over packed rows: every key and value row is unpacked inside the kernel by tb_unpack_kernel's
// rule and consumed at once; nothing unpacked is written to memory.  The counterpart of the reference's attention over packed
// rows (launch_q35_atxpk, src/q35_atxpk3.cuh / q35_atxpk4.cuh) for passes of a few rows, on CUDA cores.  Row r at *d_pos + r
// sees keys 0 .. *d_pos + r; grid (splits, kvh, M); a warp takes every eighth run of 32 keys of the split.  Online softmax in
// the exp2 domain, one rescale per 32 keys.  Partials in the layout of yskn_kv8_attention.
constexpr int TBA_WARPS = 8;
struct TbAttnP { yskn_tb_attn_args a; int G; };
struct TbTab { float cg[256], mu[256], u0[256], u1[256]; };          // one group's code table (x gain / 256) and row terms

// per-group constants of the unpack rule
struct TbRule { int packed_ok, mode, kb, guard, m, has_mu; };
__device__ __forceinline__ TbRule tb_stage_group(const uint8_t* b, int g, TbTab& T) {   // all threads of the CTA
  const TbGroup P = tb_group(b, g);
  TbRule R{P.ok && P.mode <= 1, P.mode, P.mode == 1 ? 4 : P.kk, P.guard, P.m, P.has_mu};
  const unsigned to = tb_u32(b + P.off_t + 4u * (unsigned)P.tix);
  const float gain = P.mode == 0 ? tb_f32(b + to + 4) : 1.f;
  const uint8_t* mup = b + P.go + 8;
  const uint8_t* Up = mup + (P.has_mu ? 512 : 0);
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {
    T.cg[i] = !R.packed_ok ? 0.f : (P.mode == 1 ? (float)(i - 8) : __fmul_rn(__fmul_rn((float)(int)(short)tb_u16(b + to + 12 + 2 * i), 0.00390625f), gain));
    T.mu[i] = R.packed_ok && P.has_mu ? __half2float(__ushort_as_half((unsigned short)tb_u16(mup + 2 * i))) : 0.f;
    T.u0[i] = R.packed_ok && P.m > 0 ? __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * i))) : 0.f;
    T.u1[i] = R.packed_ok && P.m > 1 ? __half2float(__ushort_as_half((unsigned short)tb_u16(Up + 2 * (256 + i)))) : 0.f;
  }
  return R;
}
// ---- 32 keys per warp step.  Scores: a lane takes one key and walks its 256 fields (the window offsets
// are then the same in every lane and known at compile time per code width); the row terms of the unpack rule leave the inner
// loop: q.x = s * sum_d q_d cg[v_d] + c0 (q.U0) + c1 (q.U1) + q.mu, with the three dot products formed once per CTA.  Values: a
// lane takes eight channels of every key, O = sum_t p_t s_t cg[v_td] + (sum p_t c0_t) U0 + (sum p_t c1_t) U1 + (sum p_t) mu.
// The unpacked values themselves are those of tb_unpack_kernel; only the order of the fp32 sums differs (tolerance parity).
constexpr int TBA_PW = 41;                                           // staged payload row: 40 words + 1 (conflict-free lane stride)
struct TbWarpSm { unsigned kp[2][32 * TBA_PW]; unsigned vp[2][32 * TBA_PW]; float pw[32][8]; int vplain[32]; };   // two staging buffers: the next 32 keys arrive while these are used
__device__ __forceinline__ void tb_cp4(unsigned* dst, const unsigned* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int KB, bool FLAT>
__device__ __forceinline__ void tb_scores32(const unsigned* row, const float* cg, const float (*q)[8], float (&dot)[8]) {
  #pragma unroll 1
  for (int c = 0; c < 4; ++c) {                                      // chains of 64 fields: same bit offsets, 2*KB words further
    const unsigned* wr = row + 2 * KB * c;
    #pragma unroll
    for (int i = 0; i < 64; ++i) {
      constexpr int dummy = 0; (void)dummy;
      const int endb = KB * (i + 1), lo = FLAT ? endb - 4 : (endb - 8 > 0 ? endb - 8 : 0), len = endb - lo;
      const unsigned v = __funnelshift_l(wr[(lo >> 5) + 1], wr[lo >> 5], lo & 31) >> (32 - len);
      const float cv = cg[v];
      const float4 qa = *reinterpret_cast<const float4*>(&q[64 * c + i][0]), qb = *reinterpret_cast<const float4*>(&q[64 * c + i][4]);
      dot[0] = fmaf(cv, qa.x, dot[0]); dot[1] = fmaf(cv, qa.y, dot[1]); dot[2] = fmaf(cv, qa.z, dot[2]); dot[3] = fmaf(cv, qa.w, dot[3]);
      dot[4] = fmaf(cv, qb.x, dot[4]); dot[5] = fmaf(cv, qb.y, dot[5]); dot[6] = fmaf(cv, qb.z, dot[6]); dot[7] = fmaf(cv, qb.w, dot[7]);
    }
  }
}

template <int KB, bool FLAT>
__device__ __forceinline__ void tb_values32(const TbWarpSm& W, const unsigned* vp, const float* cg, const float* plain, int lane, int nk, float (&acc)[8][8]) {
  int wi[8], sh[8], ln[8];
  #pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int d = 32 * w + lane, endb = KB * (d + 1), first = KB * (d & ~63), lo = FLAT ? endb - 4 : max(endb - 8, first);
    wi[w] = lo >> 5; sh[w] = lo & 31; ln[w] = 32 - (endb - lo);
  }
  #pragma unroll 2
  for (int j = 0; j < nk; ++j) {
    const float4 pa = *reinterpret_cast<const float4*>(&W.pw[j][0]), pb = *reinterpret_cast<const float4*>(&W.pw[j][4]);
    const float pg[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
    const unsigned* row = vp + j * TBA_PW;
    const bool pl = W.vplain[j] != 0;                                // warp-uniform: a row the profile leaves unpacked
    #pragma unroll
    for (int w = 0; w < 8; ++w) {
      float x;
      if (pl) x = plain ? __ldg(plain + (size_t)j * 256 + 32 * w + lane) : 0.f;
      else x = cg[__funnelshift_l(row[wi[w] + 1], row[wi[w]], sh[w]) >> ln[w]];
      #pragma unroll
      for (int g = 0; g < 8; ++g) acc[g][w] = fmaf(pg[g], x, acc[g][w]);
    }
  }
}

template <int DT>
__global__ void __launch_bounds__(TBA_WARPS * 32) tb_attn32_kernel(TbAttnP P) {
  extern __shared__ __align__(16) unsigned char tba_smem[];
  const yskn_tb_attn_args& A = P.a;
  const int G = P.G, split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TbTab* tk = reinterpret_cast<TbTab*>(tba_smem); TbTab* tv = tk + 1;
  float (*q)[8] = reinterpret_cast<float (*)[8]>(tv + 1);            // [256][8]: q * qscale * log2(e), heads past G are zero
  float (*kq)[8] = q + 256;                                           // [3][8]: q.U0, q.U1, q.mu of the key group
  TbWarpSm* Wall = reinterpret_cast<TbWarpSm*>(kq + 4);
  TbWarpSm& W = Wall[warp];
  float* mbuf = reinterpret_cast<float*>(Wall);                       // [warp][8][258], takes the staging area's place after the loop
  const TbRule rk = tb_stage_group(A.blob, __ldg(A.grp_k + kvh), *tk), rv = tb_stage_group(A.blob, __ldg(A.grp_v + kvh), *tv);
  const float qs = A.qscale * 1.4426950408889634f;
  for (int e = threadIdx.x; e < 256 * 8; e += TBA_WARPS * 32) {
    const int d = e >> 3, g = e & 7;
    q[d][g] = g < G ? act_load<DT>(A.q16, ((size_t)r * A.nh + kvh * G + g) * 256 + d) * qs : 0.f;
  }
  __syncthreads();
  if (threadIdx.x < 24) {
    const int which = threadIdx.x >> 3, g = threadIdx.x & 7;
    const float* vec = which == 0 ? tk->u0 : (which == 1 ? tk->u1 : tk->mu);
    float a = 0.f;
    for (int d = 0; d < 256; ++d) a = fmaf(q[d][g], vec[d], a);
    kq[which][g] = a;
  }
  __syncthreads();
  const int pos = __ldg(A.d_pos) + r, len = max(0, min(pos + 1, A.max_ctx));
  const int per = (len + (int)gridDim.x - 1) / (int)gridDim.x, t0 = min(len, split * per), t1 = min(len, t0 + per);
  const size_t row0 = (size_t)kvh * A.max_ctx;
  const int psw = A.pay_stride / 4, nwk = 8 * rk.kb, nwv = 8 * rv.kb;
  float acc[8][8], m[8], l[8], a0[8], a1[8], am[8];
  #pragma unroll
  for (int g = 0; g < 8; ++g) {
    m[g] = -1e30f; l[g] = a0[g] = a1[g] = am[g] = 0.f;
    #pragma unroll
    for (int w = 0; w < 8; ++w) acc[g][w] = 0.f;
  }
  // payload rows of 32 keys into staging buffer `b`, asynchronously (4-byte copies: the padded row stride is not a multiple of 16)
  auto stage = [&](int tc, int b) {
    const int nk = min(32, t1 - tc);
    const unsigned* kw = reinterpret_cast<const unsigned*>(A.k_pay) + (row0 + tc) * psw;
    const unsigned* vw = reinterpret_cast<const unsigned*>(A.v_pay) + (row0 + tc) * psw;
    for (int idx = lane; idx < nk * 40; idx += 32) {
      const int rr = idx / 40, i = idx - 40 * rr;
      if (i < nwk) tb_cp4(&W.kp[b][rr * TBA_PW + i], kw + (size_t)rr * psw + i); else W.kp[b][rr * TBA_PW + i] = 0u;
      if (i < nwv) tb_cp4(&W.vp[b][rr * TBA_PW + i], vw + (size_t)rr * psw + i); else W.vp[b][rr * TBA_PW + i] = 0u;
    }
    if (lane < nk) { W.kp[b][lane * TBA_PW + 40] = 0u; W.vp[b][lane * TBA_PW + 40] = 0u; }
  };
  int buf = 0;
  if (t0 + 32 * warp < t1) stage(t0 + 32 * warp, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int tc = t0 + 32 * warp; tc < t1; tc += 32 * TBA_WARPS, buf ^= 1) {
    const int nk = min(32, t1 - tc);
    __syncwarp();                                                    // every lane is done with the other buffer
    if (tc + 32 * TBA_WARPS < t1) stage(tc + 32 * TBA_WARPS, buf ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");           // this step's rows have landed (this lane's copies)
    __syncwarp();                                                    // ... and every other lane's
    const int t = tc + lane;
    const bool live = lane < nk, kpk = rk.packed_ok && t >= rk.guard, vpk = rv.packed_ok && t >= rv.guard;
    float sk = 0.f, c0k = 0.f, c1k = 0.f, sv = 1.f, c0v = 0.f, c1v = 0.f;
    if (live && kpk) {
      sk = __uint_as_float(__ldg(A.k_side + 2 * (row0 + t))); const unsigned pc = __ldg(A.k_side + 2 * (row0 + t) + 1);
      c0k = rk.m > 0 ? __half2float(__ushort_as_half((unsigned short)(pc & 0xffffu))) : 0.f;
      c1k = rk.m > 1 ? __half2float(__ushort_as_half((unsigned short)(pc >> 16))) : 0.f;
    }
    if (live && vpk) {
      sv = __uint_as_float(__ldg(A.v_side + 2 * (row0 + t))); const unsigned pc = __ldg(A.v_side + 2 * (row0 + t) + 1);
      c0v = rv.m > 0 ? __half2float(__ushort_as_half((unsigned short)(pc & 0xffffu))) : 0.f;
      c1v = rv.m > 1 ? __half2float(__ushort_as_half((unsigned short)(pc >> 16))) : 0.f;
    }
    float dot[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const unsigned* myrow = W.kp[buf] + lane * TBA_PW;
    if (rk.mode == 1) tb_scores32<4, true>(myrow, tk->cg, q, dot);
    else if (rk.kb == 3) tb_scores32<3, false>(myrow, tk->cg, q, dot);
    else if (rk.kb == 4) tb_scores32<4, false>(myrow, tk->cg, q, dot);
    else tb_scores32<5, false>(myrow, tk->cg, q, dot);
    float sc[8];
    #pragma unroll
    for (int g = 0; g < 8; ++g) sc[g] = fmaf(sk, dot[g], fmaf(c0k, kq[0][g], fmaf(c1k, kq[1][g], kq[2][g])));
    if (live && !kpk) {                                              // a key row the profile leaves unpacked: the plain row
      #pragma unroll
      for (int g = 0; g < 8; ++g) sc[g] = 0.f;
      if (A.k_plain) {
        const float* pr = A.k_plain + (row0 + t) * 256;
        for (int d = 0; d < 256; ++d) {
          const float x = __ldg(pr + d);
          #pragma unroll
          for (int g = 0; g < 8; ++g) sc[g] = fmaf(q[d][g], x, sc[g]);
        }
      }
    }
    W.vplain[lane] = vpk ? 0 : 1;
    #pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (g >= G) { W.pw[lane][g] = 0.f; continue; }
      float mx = live ? sc[g] : -1e30f;
      #pragma unroll
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float mn = fmaxf(m[g], mx), al = exp2f(m[g] - mn), p = live ? exp2f(sc[g] - mn) : 0.f;
      float s0 = p, s1 = p * c0v, s2 = p * c1v, s3 = vpk ? p : 0.f;
      #pragma unroll
      for (int o = 16; o; o >>= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o); s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o); s3 += __shfl_xor_sync(0xffffffffu, s3, o);
      }
      l[g] = fmaf(l[g], al, s0); a0[g] = fmaf(a0[g], al, s1); a1[g] = fmaf(a1[g], al, s2); am[g] = fmaf(am[g], al, s3); m[g] = mn;
      #pragma unroll
      for (int w = 0; w < 8; ++w) acc[g][w] *= al;
      W.pw[lane][g] = p * sv;
    }
    __syncwarp();
    const float* vpl = A.v_plain ? A.v_plain + (row0 + tc) * 256 : nullptr;
    if (rv.mode == 1) tb_values32<4, true>(W, W.vp[buf], tv->cg, vpl, lane, nk, acc);
    else if (rv.kb == 3) tb_values32<3, false>(W, W.vp[buf], tv->cg, vpl, lane, nk, acc);
    else if (rv.kb == 4) tb_values32<4, false>(W, W.vp[buf], tv->cg, vpl, lane, nk, acc);
    else tb_values32<5, false>(W, W.vp[buf], tv->cg, vpl, lane, nk, acc);
  }
  // ---- the row terms of the value group, then the merge of the warps (natural-log m, as the merge kernel expects)
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();                                                   // the staging area becomes the merge buffer
  #pragma unroll
  for (int g = 0; g < 8; ++g) {
    if (g >= G) continue;
    float* wb = mbuf + ((size_t)warp * 8 + g) * 258;
    if (lane == 0) { wb[0] = m[g]; wb[1] = l[g]; }
    #pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int d = 32 * w + lane;
      wb[2 + d] = fmaf(a0[g], tv->u0[d], fmaf(a1[g], tv->u1[d], fmaf(am[g], tv->mu[d], acc[g][w])));
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * 256; e += TBA_WARPS * 32) {
    const int g = e >> 8, d = e & 255;
    float M2 = -1e30f;
    #pragma unroll
    for (int w = 0; w < TBA_WARPS; ++w) M2 = fmaxf(M2, mbuf[((size_t)w * 8 + g) * 258]);
    float L2 = 0.f, o = 0.f;
    #pragma unroll
    for (int w = 0; w < TBA_WARPS; ++w) {
      const float* wb = mbuf + ((size_t)w * 8 + g) * 258;
      const float f = wb[0] > -1e29f ? exp2f(wb[0] - M2) : 0.f;
      L2 += f * wb[1]; o += f * wb[2 + d];
    }
    const size_t pidx = ((size_t)r * A.splits + split) * A.nh + kvh * G + g;
    if (d == 0) { A.pm[pidx] = M2 > -1e29f ? M2 * 0.6931471805599453f : -1e30f; A.pl[pidx] = L2; }
    A.pacc[pidx * 256 + d] = o;
  }
}

}  // namespace

int launch_tb_decode(const uint8_t* blob, const int* grp, const int* pos, const uint8_t* pay, int pay_stride, const uint32_t* side, const float* yin,
                     float* y, int rows, cudaStream_t st) {
  if (!blob || !grp || !pos || !pay || !side || !y) KV4_REJECT("yskn_tb_decode: null buffer");
  if (rows <= 0 || pay_stride < 160 || pay_stride % 4 || ((uintptr_t)pay & 3)) KV4_REJECT("yskn_tb_decode: bad shape (rows %d, payload stride %d)", rows, pay_stride);
  TbDecP A{blob, grp, pos, pay, pay_stride, side, yin, y, rows};
  tb_unpack_kernel<<<(rows + 7) / 8, 256, 0, st>>>(A);
  return launch_status("tb_unpack_kernel");
}

size_t tb_scratch_bytes(int rows, int nm) { return rows > 0 && nm > 0 ? (size_t)rows * nm * (256 + 8 * sizeof(float)) : 0; }

// Host-side check of a "KVQP v1" blob, the reference loader's (src/engine35.cpp:50-53) plus its table checks
// (src/kvq_fast.hpp:66-69); *nm = number of scale multipliers.
int tb_blob_info(const uint8_t* b, size_t n, int* nm) {
  auto u16 = [&](size_t o) { return (unsigned)b[o] | ((unsigned)b[o + 1] << 8); };
  auto u32 = [&](size_t o) { return u16(o) | (u16(o + 2) << 16); };
  if (!b || n < 100 || memcmp(b, "KVQP", 4) != 0 || u16(4) != 1 || u16(6) != 96 || u32(8) != n) KV4_REJECT("yskn_tb_blob_info: not a KVQP v1 blob");
  if (u16(16) != 256 || u16(18) != 16 || u16(20) != 4 || u32(28) != 128u) KV4_REJECT("yskn_tb_blob_info: needs D 256, 16 layers, 4 kv heads");
  const unsigned nt = u16(22), off_t = u32(36), off_g = u32(40), ngrp = u32(28);
  if ((size_t)off_t + 4 * (size_t)nt > n || (size_t)off_g + 4 * (size_t)ngrp > n || (size_t)u32(32) + 4 * (size_t)u16(24) > n) KV4_REJECT("yskn_tb_blob_info: offsets beyond the blob");
  for (unsigned t = 0; t < nt; ++t) {
    const size_t o = u32(off_t + 4 * t);
    if (o + 12 + 512 > n || b[o] != 8 || b[o + 2] != 64 || b[o + 3] != 8) KV4_REJECT("yskn_tb_blob_info: code tables must have L 8, chain 64, F 8");
  }
  for (unsigned g = 0; g < ngrp; ++g) {
    const size_t go = u32(off_g + 4 * g);
    if (go + 8 > n) KV4_REJECT("yskn_tb_blob_info: group record %u beyond the blob", g);
    const int mode = b[go], kk = b[go + 1], tix = b[go + 2], m = b[go + 4], mu = b[go + 5];
    if (mode > 1 || (mode == 0 && (kk < 3 || kk > 5 || (unsigned)tix >= nt)) || m > 2 || go + 8 + (mu ? 512 : 0) + 512 * (size_t)m > n)
      KV4_REJECT("yskn_tb_blob_info: group record %u has fields this codec does not have", g);
  }
  const int k = (int)u16(24);
  if (k < 1 || k > 16) KV4_REJECT("yskn_tb_blob_info: %d scale multipliers (1..16)", k);
  if (nm) *nm = k;
  return 0;
}

int launch_tb_encode(const uint8_t* blob, int nm, const float* x, const int* grp, const int* pos, int rows, float* y, uint8_t* pay, int pay_stride,
                     uint32_t* side, void* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (!blob || !x || !grp || !pos || !scratch) KV4_REJECT("yskn_tb_encode: null buffer");
  if (rows <= 0 || nm < 1 || nm > 16) KV4_REJECT("yskn_tb_encode: bad shape (rows %d, multipliers %d)", rows, nm);
  if (pay && (pay_stride < 160 || pay_stride % 4 || ((uintptr_t)pay & 3))) KV4_REJECT("yskn_tb_encode: payload rows need a stride of at least 160 bytes, a multiple of 4");
  if (scratch_bytes < tb_scratch_bytes(rows, nm) || ((uintptr_t)scratch & 3)) KV4_REJECT("yskn_tb_encode: scratch of %zu bytes needed", tb_scratch_bytes(rows, nm));
  TbP A{blob, nm, x, grp, pos, rows, y, pay, pay_stride, side, nullptr, nullptr};
  A.scr_err = static_cast<float*>(scratch);
  A.scr_states = static_cast<uint8_t*>(scratch) + (size_t)rows * nm * 8 * sizeof(float);
  const long long jobs = (long long)rows * nm * 4;
  tb_search_kernel<<<(unsigned)((jobs + TB_WARPS - 1) / TB_WARPS), TB_WARPS * 32, 0, st>>>(A);
  if (int rc = launch_status("tb_search_kernel")) return rc;
  tb_select_kernel<<<rows, 256, 0, st>>>(A);
  return launch_status("tb_select_kernel");
}

int launch_tb_attention(const yskn_tb_attn_args& a, int act_dtype, cudaStream_t st) {
  if (!a.q16 || !a.blob || !a.k_pay || !a.v_pay || !a.k_side || !a.v_side || !a.grp_k || !a.grp_v || !a.d_pos || !a.pm || !a.pl || !a.pacc)
    KV4_REJECT("yskn_tb_attention: null buffer");
  if (a.kvh <= 0 || a.nh <= 0 || a.nh % a.kvh || a.nh / a.kvh > 8 || a.M <= 0 || a.M > 65535 || a.kvh > 65535 || a.splits <= 0 || a.max_ctx <= 0)
    KV4_REJECT("yskn_tb_attention: bad shape (kvh %d, nh %d, M %d, splits %d, max_ctx %d): at most 8 query heads per kv-head", a.kvh, a.nh, a.M, a.splits, a.max_ctx);
  if (a.pay_stride < 160 || a.pay_stride % 4 || (((uintptr_t)a.k_pay | (uintptr_t)a.v_pay) & 3)) KV4_REJECT("yskn_tb_attention: bad payload stride %d or alignment", a.pay_stride);
  const size_t stage = sizeof(TbWarpSm) * TBA_WARPS, merge = (size_t)TBA_WARPS * 8 * 258 * 4;
  const size_t smem = 2 * sizeof(TbTab) + (256 + 4) * 8 * 4 + (stage > merge ? stage : merge);
  TbAttnP P{a, a.nh / a.kvh};
  const dim3 grid(a.splits, a.kvh, a.M);
  if (act_dtype == YSKN_KV4_BF16) {
    static std::atomic<unsigned long long> attr{0};
    if (first_use_on_device(attr)) KV4_CUDA(cudaFuncSetAttribute(tb_attn32_kernel<YSKN_KV4_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tb_attn32_kernel<YSKN_KV4_BF16><<<grid, TBA_WARPS * 32, smem, st>>>(P);
  } else if (act_dtype == YSKN_KV4_F16) {
    static std::atomic<unsigned long long> attr{0};
    if (first_use_on_device(attr)) KV4_CUDA(cudaFuncSetAttribute(tb_attn32_kernel<YSKN_KV4_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    tb_attn32_kernel<YSKN_KV4_F16><<<grid, TBA_WARPS * 32, smem, st>>>(P);
  } else KV4_REJECT("yskn_tb_attention: q16 is bf16 or fp16 (act_dtype %d)", act_dtype);
  return launch_status("tb_attn32_kernel");
}

}  // namespace kv4
