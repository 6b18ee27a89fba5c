// Family-B row codec, step 1: sign-Hadamard-256 rotation + INT8 rows with one fp32 scale per row.
//
// Semantics: the reference's src/kvx_codec.cuh as the shipping engine builds it (rotation on, INT8 payload;
// CMakeLists.txt:56): kvx_sign (:28-32), kvx_rotate (:35-49), kvx_store (:50-70); the decode direction is the one its
// probe runs (src/kvx_probe.cu:15-19).  Bit-exact: every operation is one IEEE fp32 operation in the reference's order.
//
// Mapping: eight lanes per row of 256 (a warp holds four rows); a lane keeps 32 elements in registers, so five of the eight
// butterfly stages pair registers and only three go through shuffles, and every load/store instruction of a row's lanes
// covers one contiguous run.  The stages run in the reference's order h = 1, 2, ... 128.  HBM-bound byte mover by design
// (1,284 B per fp32 row in + out, 772 B per fp16 row).
#include "kv4_common.cuh"

namespace kv4 {
namespace {

// Bit 0 of the reference's 32-bit multiply-xorshift hash of d + 1: set = the element's sign is flipped.
__host__ __device__ constexpr uint32_t kvx_sign_bit(int d) {
  uint32_t x = (uint32_t)d + 1u;
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x & 1u;
}
struct SignTable { uint32_t w[8]; };                       // 256 sign bits, bit d of the table = kvx_sign_bit(d)
constexpr SignTable make_signs() {
  SignTable t{};
  for (int d = 0; d < 256; ++d) t.w[d >> 5] |= kvx_sign_bit(d) << (d & 31);
  return t;
}
__constant__ SignTable c_signs = make_signs();
// Element layout of a row over 8 lanes: lane ll (0..7) holds v[4k + e] = element d = 32k + 4ll + e (k 0..7, e 0..3), so every
// load and store instruction of the 8 lanes covers one contiguous run of the row.  A warp holds 4 rows (lanes 8s .. 8s+7).
// Multiplying by +-1 is a sign-bit flip (exact, also for zeros and infinities).
__device__ __forceinline__ void apply_signs(float (&v)[32], int ll) {
  #pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t bits = c_signs.w[k] >> (4 * ll);
    #pragma unroll
    for (int e = 0; e < 4; ++e) v[4 * k + e] = __uint_as_float(__float_as_uint(v[4 * k + e]) ^ (((bits >> e) & 1u) << 31));
  }
}

// Butterflies + 1/16 in the reference's stage order h = 1, 2, ... 128.  Bits 0-1 of d are register bits (e), bits 2-4 the lane
// within the row (shuffles), bits 5-7 register bits again (k).  Lower index: a + b; upper: lower - upper.
__device__ __forceinline__ void hadamard256(float (&v)[32], int ll) {
  #pragma unroll
  for (int rb = 1; rb < 4; rb *= 2) {                      // h = 1, 2
    #pragma unroll
    for (int i = 0; i < 32; ++i)
      if (!(i & rb)) { const float lo = v[i], up = v[i + rb]; v[i] = __fadd_rn(lo, up); v[i + rb] = __fsub_rn(lo, up); }
  }
  #pragma unroll
  for (int m = 1; m < 8; m *= 2) {                         // h = 4, 8, 16
    const uint32_t flip = (ll & m) ? 0x80000000u : 0u;     // upper lane: other - self = other + (-self), exactly
    #pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float self = v[i], other = __shfl_xor_sync(0xffffffffu, self, m);
      v[i] = __fadd_rn(other, __uint_as_float(__float_as_uint(self) ^ flip));
    }
  }
  #pragma unroll
  for (int rb = 4; rb < 32; rb *= 2) {                     // h = 32, 64, 128
    #pragma unroll
    for (int i = 0; i < 32; ++i)
      if (!(i & rb)) { const float lo = v[i], up = v[i + rb]; v[i] = __fadd_rn(lo, up); v[i + rb] = __fsub_rn(lo, up); }
  }
  #pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __fmul_rn(v[i], 0.0625f);
}

template <int DT> __device__ __forceinline__ void load_row(const void* base, size_t row, int ll, bool live, float (&v)[32]) {
  #pragma unroll
  for (int k = 0; k < 8; ++k) {
    const size_t d = row * 256 + 32 * k + 4 * ll;
    if (DT == YSKN_KV4_F32) {
      const float4 a = live ? __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
      v[4 * k] = a.x; v[4 * k + 1] = a.y; v[4 * k + 2] = a.z; v[4 * k + 3] = a.w;
    } else {
      const uint2 u = live ? __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(base) + d)) : make_uint2(0u, 0u);
      v[4 * k] = DT == YSKN_KV4_F16 ? h2f((uint16_t)u.x) : bf2f((uint16_t)u.x); v[4 * k + 1] = DT == YSKN_KV4_F16 ? h2f((uint16_t)(u.x >> 16)) : bf2f((uint16_t)(u.x >> 16));
      v[4 * k + 2] = DT == YSKN_KV4_F16 ? h2f((uint16_t)u.y) : bf2f((uint16_t)u.y); v[4 * k + 3] = DT == YSKN_KV4_F16 ? h2f((uint16_t)(u.y >> 16)) : bf2f((uint16_t)(u.y >> 16));
    }
  }
}
template <int DT> __device__ __forceinline__ void store_row(void* base, size_t row, int ll, const float (&v)[32]) {
  #pragma unroll
  for (int k = 0; k < 8; ++k) {
    const size_t d = row * 256 + 32 * k + 4 * ll;
    if (DT == YSKN_KV4_F32) *reinterpret_cast<float4*>(static_cast<float*>(base) + d) = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
    else *reinterpret_cast<uint2*>(static_cast<uint16_t*>(base) + d) =
        make_uint2((uint32_t)act_store16<DT>(v[4 * k]) | ((uint32_t)act_store16<DT>(v[4 * k + 1]) << 16),
                   (uint32_t)act_store16<DT>(v[4 * k + 2]) | ((uint32_t)act_store16<DT>(v[4 * k + 3]) << 16));
  }
}

constexpr int ROWS_PER_BLOCK = 32;                         // 8 warps x 4 rows

// mode 0: rotate, 1: inverse rotate (fp32 in, fp32 out)
__global__ void __launch_bounds__(256) kvx_rotate_kernel(const float* x, float* y, long long rows, int inverse) {
  const int lane = threadIdx.x & 31, ll = lane & 7;
  const long long row = (long long)blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5) * 4 + (lane >> 3);
  const bool live = row < rows;
  float v[32];
  load_row<YSKN_KV4_F32>(x, (size_t)row, ll, live, v);
  if (!inverse) apply_signs(v, ll);
  hadamard256(v, ll);
  if (inverse) apply_signs(v, ll);
  if (live) store_row<YSKN_KV4_F32>(y, (size_t)row, ll, v);
}

// INT8 row from the rotated values: scale = max|v| / 127, q = rne(v / scale) clamped to +-127 (src/kvx_codec.cuh:50-70).
__device__ __forceinline__ void store_int8_row(const float (&v)[32], int ll, bool live, int8_t* q8, float* scales, size_t row) {
  float amax = 0.f;
  #pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  #pragma unroll
  for (int m = 4; m; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  const float sc = __fdiv_rn(amax, 127.f);
  // q = rne(fl(v / sc)).  v * (1 / sc) is within 3.8e-5 of the correctly rounded quotient (|q| <= 127), so rounding it gives
  // the same integer unless it lies that close to a half-integer; only those elements (about one in 10^4) take the exact division.
  const float inv = sc > 0.f ? __fdiv_rn(1.f, sc) : 0.f;
  #pragma unroll
  for (int k = 0; k < 8; ++k) {
    uint32_t w = 0u;
    #pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float xv = v[4 * k + e], t = __fmul_rn(xv, inv);
      int q = __float2int_rn(t);
      // distance of t from the integer it rounds to; near 0.5 (or NaN: 1/scale overflowed) -> the reference's own arithmetic.
      // |v| <= max|v| makes |v / scale| <= 127 (1 + 2^-23), so the reference's clamp to +-127 can only act on that path.
      if (!(fabsf(__fsub_rn(t, (float)q)) <= 0.5f - 6.2e-5f)) q = max(-127, min(127, sc > 0.f ? __float2int_rn(__fdiv_rn(xv, sc)) : 0));
      w |= ((uint32_t)q & 0xFFu) << (8 * e);
    }
    if (live) *reinterpret_cast<uint32_t*>(q8 + row * 256 + 32 * k + 4 * ll) = w;
  }
  if (live && ll == 0) scales[row] = sc;
}

template <int DT>
__global__ void __launch_bounds__(256) kvx_encode_kernel(const void* x, int8_t* q8, float* scales, long long rows) {
  const int lane = threadIdx.x & 31, ll = lane & 7;
  const long long row = (long long)blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5) * 4 + (lane >> 3);
  const bool live = row < rows;
  float v[32];
  load_row<DT>(x, (size_t)row, ll, live, v);
  apply_signs(v, ll);
  hadamard256(v, ll);
  store_int8_row(v, ll, live, q8, scales, (size_t)row);
}

template <int DT>
__global__ void __launch_bounds__(256) kvx_decode_kernel(const int8_t* q8, const float* scales, void* y, long long rows) {
  const int lane = threadIdx.x & 31, ll = lane & 7;
  const long long row = (long long)blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5) * 4 + (lane >> 3);
  const bool live = row < rows;
  const float sc = live ? __ldg(scales + row) : 0.f;
  float v[32];
  #pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t u = live ? __ldg(reinterpret_cast<const uint32_t*>(q8 + (size_t)row * 256 + 32 * k + 4 * ll)) : 0u;
    #pragma unroll
    for (int e = 0; e < 4; ++e) v[4 * k + e] = __fmul_rn((float)(int8_t)(uint8_t)(u >> (8 * e)), sc);
  }
  hadamard256(v, ll);
  apply_signs(v, ll);
  if (live) store_row<DT>(y, (size_t)row, ll, v);
}

// The attention block's row epilogue over INT8 rows: the reference's q35_attn_post_kernel (src/q35_kernels.cu:1013-1065) from
// the point where a thread holds its bf16-rounded projection value (:1029).  One work item = one row of 256: a query head
// (RMS norm, partial RoPE, rotation -> bf16 q16; its gate half is copied), a key head (the same -> INT8 row at the token's
// position) or a value head (rotation -> INT8 row).  Every operation is the reference's single IEEE operation in its order:
// the sum of squares is the reference's xor-shuffle tree per 32 channels (strides 16, 8, 4 = this layout's lane bits, strides
// 2, 1 = register pairs) followed by the in-order sum of the eight warp sums.  NRH = rotary width / 64.
__device__ __forceinline__ float rbf(float f) { return bf2f(f2bf(f)); }

template <int NRH>
__global__ void __launch_bounds__(256, 4) kvx_attn_post_kernel(yskn_kvx_attn_post_args A) {
  const int lane = threadIdx.x & 31, ll = lane & 7;
  const int per_tok = A.nh + 2 * A.kvh;
  const long long item = (long long)blockIdx.x * ROWS_PER_BLOCK + (threadIdx.x >> 5) * 4 + (lane >> 3);
  const bool live = item < (long long)A.M * per_tok;
  const int tok = live ? (int)(item / per_tok) : 0, u = live ? (int)(item % per_tok) : 0;
  const int kind = u < A.nh ? 0 : (u < A.nh + A.kvh ? 1 : 2);    // query / key / value head
  const int head = kind == 0 ? u : (kind == 1 ? u - A.nh : u - A.nh - A.kvh);
  const int pos = __ldg(A.d_pos) + tok;
  const uint16_t* src = kind == 0 ? A.q_rows + ((size_t)tok * A.nh + head) * 512
                                  : (kind == 1 ? A.k_rows : A.v_rows) + ((size_t)tok * A.kvh + head) * 256;
  float v[32];
  load_row<YSKN_KV4_BF16>(src, 0, ll, live, v);
  if (live && kind == 0) {                                       // the gate half of the head's projection, as it is
    #pragma unroll
    for (int k = 0; k < 8; ++k)
      *reinterpret_cast<uint2*>(A.gate16 + ((size_t)tok * A.nh + head) * 256 + 32 * k + 4 * ll) = __ldg(reinterpret_cast<const uint2*>(src + 256 + 32 * k + 4 * ll));
  }
  // ---- RMS norm (all lanes of a warp run the shuffles unless its four rows are all value heads, which keep their rows)
  float tot = 0.f;
  const bool any_norm = !__all_sync(0xffffffffu, kind == 2);
  #pragma unroll
  for (int k = 0; k < 8 && any_norm; ++k) {
    float t[4];
    #pragma unroll
    for (int e = 0; e < 4; ++e) t[e] = __fmul_rn(v[4 * k + e], v[4 * k + e]);
    #pragma unroll
    for (int m = 4; m; m >>= 1) {
      #pragma unroll
      for (int e = 0; e < 4; ++e) t[e] = __fadd_rn(t[e], __shfl_xor_sync(0xffffffffu, t[e], m));
    }
    tot = __fadd_rn(tot, __fadd_rn(__fadd_rn(t[0], t[2]), __fadd_rn(t[1], t[3])));
  }
  if (kind != 2) {
    const float x = __fadd_rn(__fdiv_rn(tot, 256.f), A.eps);
    const float r = A.pm ? __fdiv_rn(1.f, __fsqrt_rn(x)) : rsqrtf(x);
    const uint16_t* wn = kind == 0 ? A.qn_w : A.kn_w;
    #pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(wn + 32 * k + 4 * ll));
      const uint16_t wb[4] = {(uint16_t)w.x, (uint16_t)(w.x >> 16), (uint16_t)w.y, (uint16_t)(w.y >> 16)};
      #pragma unroll
      for (int e = 0; e < 4; ++e) v[4 * k + e] = rbf(__fmul_rn(__fmul_rn(v[4 * k + e], r), __fadd_rn(1.f, bf2f(wb[e]))));
    }
    // ---- rotate-half over the first 64*NRH channels: pair (d, d + 32*NRH) sits in one lane (registers k and k + NRH)
    #pragma unroll
    for (int k = 0; k < NRH; ++k) {
      const float4* rr = reinterpret_cast<const float4*>(A.rope + ((size_t)pos * (32 * NRH) + 32 * k + 4 * ll) * 2);
      const float4 c01 = live ? __ldg(rr) : make_float4(0.f, 0.f, 0.f, 0.f), c23 = live ? __ldg(rr + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float cs[4] = {c01.x, c01.z, c23.x, c23.z}, sn[4] = {c01.y, c01.w, c23.y, c23.w};
      #pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = v[4 * k + e], hi = v[4 * (k + NRH) + e];
        v[4 * k + e] = rbf(__fadd_rn(rbf(__fmul_rn(lo, cs[e])), rbf(__fmul_rn(-hi, sn[e]))));
        v[4 * (k + NRH) + e] = rbf(__fadd_rn(rbf(__fmul_rn(hi, cs[e])), rbf(__fmul_rn(lo, sn[e]))));
      }
    }
  }
  apply_signs(v, ll);
  hadamard256(v, ll);
  if (live && kind == 0) store_row<YSKN_KV4_BF16>(A.q16, (size_t)tok * A.nh + head, ll, v);
  const bool cache = live && kind != 0 && pos >= 0 && pos < A.max_ctx;     // a position outside the cache stores nothing
  store_int8_row(v, ll, cache, kind == 2 ? A.v8 : A.k8, kind == 2 ? A.vs : A.ks, (size_t)head * A.max_ctx + (cache ? pos : 0));
}

int grid_for(long long rows, unsigned* grid, const char* who) {
  if (rows < 0 || rows > (1ll << 34)) { set_error("%s: bad row count %lld", who, rows); return -1; }
  *grid = (unsigned)((rows + ROWS_PER_BLOCK - 1) / ROWS_PER_BLOCK);
  return 0;
}

}  // namespace

int launch_kvx_rotate(const float* x, float* y, long long rows, int inverse, cudaStream_t st) {
  if (rows == 0) return 0;
  if (!x || !y) KV4_REJECT("yskn_kvx_rotate: null buffer");
  if (((uintptr_t)x | (uintptr_t)y) & 15) KV4_REJECT("yskn_kvx_rotate: rows must be 16-byte aligned");
  unsigned grid; if (grid_for(rows, &grid, "yskn_kvx_rotate")) return -1;
  kvx_rotate_kernel<<<grid, 256, 0, st>>>(x, y, rows, inverse ? 1 : 0);
  return launch_status("kvx_rotate_kernel");
}

int launch_kvx_encode(const void* x, int x_dtype, int8_t* q8, float* scales, long long rows, cudaStream_t st) {
  if (rows == 0) return 0;
  if (!x || !q8 || !scales) KV4_REJECT("yskn_kvx_encode: null buffer");
  if (((uintptr_t)x & 15) || ((uintptr_t)q8 & 7)) KV4_REJECT("yskn_kvx_encode: x must be 16-byte and q8 8-byte aligned");
  unsigned grid; if (grid_for(rows, &grid, "yskn_kvx_encode")) return -1;
  if (x_dtype == YSKN_KV4_F32) kvx_encode_kernel<YSKN_KV4_F32><<<grid, 256, 0, st>>>(x, q8, scales, rows);
  else if (x_dtype == YSKN_KV4_F16) kvx_encode_kernel<YSKN_KV4_F16><<<grid, 256, 0, st>>>(x, q8, scales, rows);
  else if (x_dtype == YSKN_KV4_BF16) kvx_encode_kernel<YSKN_KV4_BF16><<<grid, 256, 0, st>>>(x, q8, scales, rows);
  else KV4_REJECT("yskn_kvx_encode: unknown dtype %d", x_dtype);
  return launch_status("kvx_encode_kernel");
}

int launch_kvx_decode(const int8_t* q8, const float* scales, void* y, int y_dtype, long long rows, cudaStream_t st) {
  if (rows == 0) return 0;
  if (!y || !q8 || !scales) KV4_REJECT("yskn_kvx_decode: null buffer");
  if (((uintptr_t)y & 15) || ((uintptr_t)q8 & 7)) KV4_REJECT("yskn_kvx_decode: y must be 16-byte and q8 8-byte aligned");
  unsigned grid; if (grid_for(rows, &grid, "yskn_kvx_decode")) return -1;
  if (y_dtype == YSKN_KV4_F32) kvx_decode_kernel<YSKN_KV4_F32><<<grid, 256, 0, st>>>(q8, scales, y, rows);
  else if (y_dtype == YSKN_KV4_F16) kvx_decode_kernel<YSKN_KV4_F16><<<grid, 256, 0, st>>>(q8, scales, y, rows);
  else if (y_dtype == YSKN_KV4_BF16) kvx_decode_kernel<YSKN_KV4_BF16><<<grid, 256, 0, st>>>(q8, scales, y, rows);
  else KV4_REJECT("yskn_kvx_decode: unknown dtype %d", y_dtype);
  return launch_status("kvx_decode_kernel");
}

int launch_kvx_attn_post(const yskn_kvx_attn_post_args& a, cudaStream_t st) {
  if (a.M == 0) return 0;
  if (!a.q_rows || !a.k_rows || !a.v_rows || !a.qn_w || !a.kn_w || !a.d_pos || !a.q16 || !a.gate16 || !a.k8 || !a.v8 || !a.ks || !a.vs)
    KV4_REJECT("yskn_kvx_attn_post: null buffer");
  if (a.M < 0 || a.nh <= 0 || a.kvh <= 0 || a.max_ctx <= 0) KV4_REJECT("yskn_kvx_attn_post: bad shape (M %d, nh %d, kvh %d, max_ctx %d)", a.M, a.nh, a.kvh, a.max_ctx);
  if (a.rd < 0 || a.rd > 256 || a.rd % 64) KV4_REJECT("yskn_kvx_attn_post: rotary width %d must be a multiple of 64 up to 256", a.rd);
  if (a.rd > 0 && !a.rope) KV4_REJECT("yskn_kvx_attn_post: rotary width %d needs a rope table", a.rd);
  if (((uintptr_t)a.q_rows | (uintptr_t)a.k_rows | (uintptr_t)a.v_rows | (uintptr_t)a.qn_w | (uintptr_t)a.kn_w | (uintptr_t)a.q16 | (uintptr_t)a.gate16 |
       (uintptr_t)a.k8 | (uintptr_t)a.v8) & 7)
    KV4_REJECT("yskn_kvx_attn_post: row arrays must be 8-byte aligned");
  if ((uintptr_t)a.rope & 15) KV4_REJECT("yskn_kvx_attn_post: the rope table must be 16-byte aligned");
  unsigned grid; if (grid_for((long long)a.M * (a.nh + 2 * a.kvh), &grid, "yskn_kvx_attn_post")) return -1;
  switch (a.rd / 64) {
    case 0: kvx_attn_post_kernel<0><<<grid, 256, 0, st>>>(a); break;
    case 1: kvx_attn_post_kernel<1><<<grid, 256, 0, st>>>(a); break;
    case 2: kvx_attn_post_kernel<2><<<grid, 256, 0, st>>>(a); break;
    case 3: kvx_attn_post_kernel<3><<<grid, 256, 0, st>>>(a); break;
    default: kvx_attn_post_kernel<4><<<grid, 256, 0, st>>>(a); break;
  }
  return launch_status("kvx_attn_post_kernel");
}

}  // namespace kv4
