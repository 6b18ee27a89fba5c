// KV4 quantize-and-append codec and the RoPE table (sm_100a).
//
// Bit-exact restatement, in new kernels, of the reference's
//   K shadow store            src/post_kernels.cu:48-54
//   per-token V int4          src/post_kernels.cu:64-82
//   32-token K group int4     src/attention_gqa.cu:143-154 (= src/post_kernels.cu:86-96)
//   (cos,sin) table           src/attention_gqa.cu:158-162
// Every arithmetic step that decides a stored bit uses an explicit round-to-nearest intrinsic, so the
// result does not depend on the compiler's FMA contraction (the reference relies on --fmad=false).
//
// Both kernels are HBM-bound byte movers: one warp owns one (row, kv-head) or one (group, kv-head),
// each lane owns HD/32 contiguous channels, so every load and store of a warp is one contiguous
// 128..512-byte segment.
#include "kv4_common.cuh"
#include <cmath>

namespace kv4 {
namespace {

__device__ __forceinline__ int quant4(float v, float lo, float inv) {
  int q = __float2int_rn(__fmul_rn(__fsub_rn(v, lo), inv));
  return q < 0 ? 0 : (q > 15 ? 15 : q);
}

// The 32-token group `gi` of kv-head `head`, by one warp: per channel min / max over the 32 shadow rows, fp16 scale and zero,
// int4 codes (src/attention_gqa.cu:143-154).  A lane touches only its own HD/32 channels of every row.
template <int HD>
__device__ __forceinline__ void group_quant_warp(const yskn_kv_layer& kv, int max_ctx, int gi, int head, int lane) {
  constexpr int CPL = HD / 32;
  const uint16_t* rows = kv.kshadow + ((size_t)head * max_ctx + (size_t)gi * 32) * HD + (size_t)lane * CPL;

  float lo[CPL], hi[CPL];
  #pragma unroll
  for (int e = 0; e < CPL; ++e) { lo[e] = 1e30f; hi[e] = -1e30f; }
  for (int t = 0; t < 32; ++t) {
    #pragma unroll
    for (int e = 0; e < CPL; e += 2) {
      const uint32_t u = *reinterpret_cast<const uint32_t*>(rows + (size_t)t * HD + e);
      const float a = h2f((uint16_t)u), b = h2f((uint16_t)(u >> 16));
      lo[e] = fminf(lo[e], a); hi[e] = fmaxf(hi[e], a); lo[e + 1] = fminf(lo[e + 1], b); hi[e + 1] = fmaxf(hi[e + 1], b);
    }
  }
  float inv[CPL];
  const size_t gb = (size_t)head * (max_ctx / 32) + gi;
  uint16_t* ks = kv.kscale + gb * HD + (size_t)lane * CPL;
  uint16_t* kz = kv.kzero + gb * HD + (size_t)lane * CPL;
  #pragma unroll
  for (int e = 0; e < CPL; e += 2) {
    uint32_t s2 = 0, z2 = 0;
    #pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float d = __fsub_rn(hi[e + k], lo[e + k]);
      inv[e + k] = hi[e + k] > lo[e + k] ? __fdiv_rn(15.f, d) : 0.f;
      s2 |= (uint32_t)f2h(__fdiv_rn(d, 15.f)) << (16 * k);
      z2 |= (uint32_t)f2h(lo[e + k]) << (16 * k);
    }
    *reinterpret_cast<uint32_t*>(ks + e) = s2;
    *reinterpret_cast<uint32_t*>(kz + e) = z2;
  }
  uint8_t* kq = kv.kq + gb * 32 * (HD / 2) + (size_t)lane * (CPL / 2);
  for (int t = 0; t < 32; ++t) {
    uint32_t packed = 0;
    #pragma unroll
    for (int e = 0; e < CPL; e += 2) {
      const uint32_t u = *reinterpret_cast<const uint32_t*>(rows + (size_t)t * HD + e);
      packed |= (uint32_t)quant4(h2f((uint16_t)u), lo[e], inv[e]) << (4 * e);
      packed |= (uint32_t)quant4(h2f((uint16_t)(u >> 16)), lo[e + 1], inv[e + 1]) << (4 * e + 4);
    }
    uint8_t* dst = kq + (size_t)t * (HD / 2);
    if (CPL == 8) *reinterpret_cast<uint32_t*>(dst) = packed;
    else if (CPL == 4) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)packed;
    else *dst = (uint8_t)packed;
  }
}

// One warp per (row, kv-head): K row -> fp16 shadow; V row -> int4 + fp16 scale/zero.  FUSE (one-row passes): a row that
// completes its 32-token group quantises the group in the same launch, as the reference's epilogue does at M = 1
// (src/post_kernels.cu:55-63, switched on by src/engine.cpp:186-187): the 31 older rows were stored by earlier passes and
// the newest one by this very lane, so no other launch and no barrier is needed.
template <int HD, int DT, bool FUSE>
__global__ void __launch_bounds__(128) kv4_append_rows_kernel(yskn_kv_append_args A) {
  constexpr int CPL = HD / 32;                       // channels per lane (2, 4 or 8)
  const int lane = threadIdx.x & 31, w = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (w >= A.M * A.kvh) return;
  const int r = w / A.kvh, head = w % A.kvh, pos = *A.d_pos + r;
  if (pos < 0 || pos >= A.max_ctx) return;
  const size_t in0 = ((size_t)r * A.kvh + head) * HD + (size_t)lane * CPL;

  uint16_t kh[CPL]; float y[CPL];
  #pragma unroll
  for (int e = 0; e < CPL; ++e) {
    kh[e] = f2h(act_load<DT>(A.k_in, in0 + e));
    y[e] = round_f16(act_load<DT>(A.v_in, in0 + e));
  }
  uint16_t* ksh = A.kv.kshadow + ((size_t)head * A.max_ctx + pos) * HD + (size_t)lane * CPL;
  #pragma unroll
  for (int e = 0; e < CPL; e += 2) *reinterpret_cast<uint32_t*>(ksh + e) = (uint32_t)kh[e] | ((uint32_t)kh[e + 1] << 16);

  float lo = y[0], hi = y[0];
  #pragma unroll
  for (int e = 1; e < CPL; ++e) { lo = fminf(lo, y[e]); hi = fmaxf(hi, y[e]); }
  #pragma unroll
  for (int o = 16; o; o >>= 1) { lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o)); }
  const float sc = __fdiv_rn(__fsub_rn(hi, lo), 15.f);
  const float inv = hi > lo ? __fdiv_rn(15.f, __fsub_rn(hi, lo)) : 0.f;
  const size_t slot = (size_t)head * A.max_ctx + pos;
  uint8_t* vq = A.kv.vq + slot * (HD / 2) + (size_t)lane * (CPL / 2);
  uint32_t packed = 0;
  #pragma unroll
  for (int e = 0; e < CPL; ++e) packed |= (uint32_t)quant4(y[e], lo, inv) << (4 * e);
  if (CPL == 8) *reinterpret_cast<uint32_t*>(vq) = packed;
  else if (CPL == 4) *reinterpret_cast<uint16_t*>(vq) = (uint16_t)packed;
  else *vq = (uint8_t)packed;
  if (lane == 0) { A.kv.vscale[slot] = f2h(sc); A.kv.vzero[slot] = f2h(lo); }
  if (FUSE && (pos & 31) == 31) group_quant_warp<HD>(A.kv, A.max_ctx, pos >> 5, head, lane);
}

// One warp per (candidate group, kv-head).  A group is quantised only in the pass that appends its
// 32nd token (src/attention_gqa.cu:145-146); until then its rows exist only in the fp16 shadow.
template <int HD>
__global__ void __launch_bounds__(128) kv4_group_quant_kernel(yskn_kv_quant_args A, int kvh) {
  const int lane = threadIdx.x & 31, w = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int ncand = (A.M + 31) / 32 + 1;
  if (w >= ncand * kvh) return;
  const int pos0 = *A.d_pos, last = pos0 + A.M - 1;
  const int gi = pos0 / 32 + w / kvh, head = w % kvh, gend = gi * 32 + 31;
  if (gend < pos0 || gend > last || gend >= A.max_ctx) return;
  group_quant_warp<HD>(A.kv, A.max_ctx, gi, head, lane);
}

// out[t][i] = (cos, sin)(float(t) * freq_i), freq_i = theta^(-2i/rd).  The fp32 product that defines the
// angle is kept (src/attention_gqa.cu:161); the exponent and the trigonometric functions are taken in double
// and rounded once, which makes the table reproducible on a CPU to the last bit in all but rare cases.
__global__ void kv4_rope_table_kernel(float2* out, int max_ctx, float theta, int rd) {
  const int half = rd / 2;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)max_ctx * half) return;
  const int t = (int)(idx / half), i = (int)(idx % half);
  const float freq = (float)pow((double)theta, -(double)(2 * i) / (double)rd);
  const float ang = __fmul_rn((float)t, freq);
  double s, c; sincos((double)ang, &s, &c);
  out[idx] = make_float2((float)c, (float)s);
}

template <int HD, bool FUSE> int append_dt(const yskn_kv_append_args& a, cudaStream_t st) {
  const int blocks = (a.M * a.kvh + 3) / 4;
  switch (a.in_dtype) {
    case YSKN_KV4_F16: kv4_append_rows_kernel<HD, YSKN_KV4_F16, FUSE><<<blocks, 128, 0, st>>>(a); break;
    case YSKN_KV4_BF16: kv4_append_rows_kernel<HD, YSKN_KV4_BF16, FUSE><<<blocks, 128, 0, st>>>(a); break;
    case YSKN_KV4_F32: kv4_append_rows_kernel<HD, YSKN_KV4_F32, FUSE><<<blocks, 128, 0, st>>>(a); break;
    default: KV4_REJECT("yskn_kv4_append: unknown in_dtype %d", a.in_dtype);
  }
  return launch_status("kv4_append_rows_kernel");
}

// A copy by a kernel, for the few kilobytes a decode step exchanges with the host: either side may be pinned (mapped) host
// memory.  Inside a captured pass a kernel node of this size runs in about 2 us where a memcpy node takes about 6.  Host
// memory is read past the caches (ld.global.cv), so a replayed graph sees what the host wrote since the last replay.
__global__ void __launch_bounds__(256) kv4_copy16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i < n16) dst[i] = __ldcv(src + i);
}

}  // namespace

int launch_copy16(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  if (bytes == 0) return 0;
  if (!dst || !src) KV4_REJECT("yskn_kv4_copy: null buffer");
  if ((bytes & 15) || (((uintptr_t)dst | (uintptr_t)src) & 15)) KV4_REJECT("yskn_kv4_copy: %zu bytes: size and both addresses must be multiples of 16", bytes);
  if (bytes > ((size_t)1 << 26)) KV4_REJECT("yskn_kv4_copy: %zu bytes: meant for small buffers (at most 64 MiB)", bytes);
  const size_t n16 = bytes / 16;
  kv4_copy16_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), n16);
  return launch_status("kv4_copy16_kernel");
}

int launch_rope_table(float* d_out, int max_ctx, float theta, int rd, cudaStream_t st) {
  if (!d_out || max_ctx <= 0 || rd <= 0 || (rd & 1)) KV4_REJECT("yskn_kv4_rope_table: bad arguments (max_ctx %d, rd %d)", max_ctx, rd);
  const long long n = (long long)max_ctx * (rd / 2);
  kv4_rope_table_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<float2*>(d_out), max_ctx, theta, rd);
  return launch_status("kv4_rope_table_kernel");
}

int launch_group_quant(const yskn_kv_quant_args& a, int kvh, int hd, cudaStream_t st) {
  if (a.M <= 0 || kvh <= 0 || !a.d_pos || a.max_ctx % 32) KV4_REJECT("yskn_kv4_group_quant: bad arguments (M %d, kvh %d, max_ctx %d)", a.M, kvh, a.max_ctx);
  const int blocks = (((a.M + 31) / 32 + 1) * kvh + 3) / 4;
  if (hd == 256) kv4_group_quant_kernel<256><<<blocks, 128, 0, st>>>(a, kvh);
  else if (hd == 128) kv4_group_quant_kernel<128><<<blocks, 128, 0, st>>>(a, kvh);
  else if (hd == 64) kv4_group_quant_kernel<64><<<blocks, 128, 0, st>>>(a, kvh);
  else KV4_REJECT("yskn_kv4_group_quant: unsupported head_dim %d (64, 128, 256)", hd);   // src/attention_gqa.cu:186
  return launch_status("kv4_group_quant_kernel");
}

int launch_append(const yskn_kv_append_args& a, cudaStream_t st) {
  if (!a.k_in || !a.v_in || !a.d_pos || a.M <= 0 || a.kvh <= 0 || a.max_ctx % 32)
    KV4_REJECT("yskn_kv4_append: bad arguments (M %d, kvh %d, max_ctx %d)", a.M, a.kvh, a.max_ctx);
  int rc;
  if (a.M == 1) {                                                // one launch: the row's warp also closes its group
    if (a.hd == 256) return append_dt<256, true>(a, st);
    if (a.hd == 128) return append_dt<128, true>(a, st);
    if (a.hd == 64) return append_dt<64, true>(a, st);
    KV4_REJECT("yskn_kv4_append: unsupported head_dim %d (64, 128, 256)", a.hd);
  }
  if (a.hd == 256) rc = append_dt<256, false>(a, st);
  else if (a.hd == 128) rc = append_dt<128, false>(a, st);
  else if (a.hd == 64) rc = append_dt<64, false>(a, st);
  else KV4_REJECT("yskn_kv4_append: unsupported head_dim %d (64, 128, 256)", a.hd);
  if (rc) return rc;
  yskn_kv_quant_args q; q.kv = a.kv; q.d_pos = a.d_pos; q.M = a.M; q.max_ctx = a.max_ctx;
  return launch_group_quant(q, a.kvh, a.hd, st);
}

}  // namespace kv4
