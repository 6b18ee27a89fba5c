// Family-B row codec, step 1: sign-Hadamard-256 rotation + INT8 rows with one fp32 scale per row.
//
// Semantics: the reference's src/kvx_codec.cuh as the shipping engine builds it (rotation on, INT8 payload;
// CMakeLists.txt:56): kvx_sign (:28-32), kvx_rotate (:35-49), kvx_store (:50-70); the decode direction is the one its
// probe runs (src/kvx_probe.cu:15-19).  Bit-exact: every operation is one IEEE fp32 operation in the reference's order.
//
// Mapping: one warp per row of 256; lane L holds elements 8L .. 8L+7, so a row is read as two 16-byte loads per lane
// (fp32) or one (fp16/bf16) and written as one 8-byte store per lane.  The butterfly stages run in the reference's
// order h = 1, 2, ... 128: h = 1, 2, 4 pair registers of one lane, h = 8 ... 128 pair lanes L and L ^ (h / 8) through
// shuffles.  HBM-bound byte mover (1,284 B per fp32 row in + out, 772 B per fp16 row); the eight exact divisions per
// lane are the only heavy arithmetic.
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
// Multiplying by +-1 is a sign-bit flip (exact, also for zeros and infinities): element i of lane L is d = 8L + i.
__device__ __forceinline__ void apply_signs(float (&v)[8], int lane) {
  const uint32_t bits = (c_signs.w[lane >> 2] >> (8 * (lane & 3))) & 0xFFu;
  #pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(__float_as_uint(v[i]) ^ (((bits >> i) & 1u) << 31));
}

// Butterflies + 1/16 on the 256 elements a warp holds (v[i] = element 8*lane + i).  Lower index: a + b; upper: lower - upper.
__device__ __forceinline__ void hadamard256(float (&v)[8], int lane) {
  #pragma unroll
  for (int h = 1; h < 8; h *= 2) {
    #pragma unroll
    for (int i = 0; i < 8; ++i)
      if (!(i & h)) { const float lo = v[i], up = v[i + h]; v[i] = __fadd_rn(lo, up); v[i + h] = __fsub_rn(lo, up); }
  }
  #pragma unroll
  for (int m = 1; m < 32; m *= 2) {
    const uint32_t flip = (lane & m) ? 0x80000000u : 0u;          // upper lane: other - self = other + (-self), exactly
    #pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float self = v[i], other = __shfl_xor_sync(0xffffffffu, self, m);
      v[i] = __fadd_rn(other, __uint_as_float(__float_as_uint(self) ^ flip));
    }
  }
  #pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], 0.0625f);
}

template <int DT> __device__ __forceinline__ void load8(const void* base, size_t row, int lane, float (&v)[8]) {
  if (DT == YSKN_KV4_F32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + row * 256 + 8 * lane);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + row * 256 + 8 * lane));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[2 * k] = DT == YSKN_KV4_F16 ? h2f((uint16_t)w[k]) : bf2f((uint16_t)w[k]);
      v[2 * k + 1] = DT == YSKN_KV4_F16 ? h2f((uint16_t)(w[k] >> 16)) : bf2f((uint16_t)(w[k] >> 16));
    }
  }
}
template <int DT> __device__ __forceinline__ void store8(void* base, size_t row, int lane, const float (&v)[8]) {
  if (DT == YSKN_KV4_F32) {
    float4* p = reinterpret_cast<float4*>(static_cast<float*>(base) + row * 256 + 8 * lane);
    p[0] = make_float4(v[0], v[1], v[2], v[3]); p[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    uint32_t w[4];
    #pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = (uint32_t)act_store16<DT>(v[2 * k]) | ((uint32_t)act_store16<DT>(v[2 * k + 1]) << 16);
    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + row * 256 + 8 * lane) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// mode 0: rotate, 1: inverse rotate (fp32 in, fp32 out)
__global__ void __launch_bounds__(256) kvx_rotate_kernel(const float* x, float* y, long long rows, int inverse) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float v[8];
  load8<YSKN_KV4_F32>(x, (size_t)row, lane, v);
  if (!inverse) apply_signs(v, lane);
  hadamard256(v, lane);
  if (inverse) apply_signs(v, lane);
  store8<YSKN_KV4_F32>(y, (size_t)row, lane, v);
}

template <int DT>
__global__ void __launch_bounds__(256) kvx_encode_kernel(const void* x, int8_t* q8, float* scales, long long rows) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  float v[8];
  load8<DT>(x, (size_t)row, lane, v);
  apply_signs(v, lane);
  hadamard256(v, lane);
  float amax = 0.f;
  #pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  #pragma unroll
  for (int m = 16; m; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  const float sc = __fdiv_rn(amax, 127.f);
  // q = rne(fl(v / sc)).  v * (1 / sc) is within a few ulp of the exact quotient, so rounding it gives the same integer
  // unless it lies that close to a half-integer; only those elements (about one in 10^4) take the exact division.
  const float inv = sc > 0.f ? __fdiv_rn(1.f, sc) : 0.f;
  uint32_t w[2] = {0u, 0u};
  #pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float t = __fmul_rn(v[i], inv);
    const float frac = fabsf(__fsub_rn(t, truncf(t)));               // exact: |t| < 2^8 here, distance from the integer below in magnitude
    int q = __float2int_rn(t);
    if (fabsf(__fsub_rn(frac, 0.5f)) < 6.2e-5f || !(fabsf(t) < 200.f)) q = sc > 0.f ? __float2int_rn(__fdiv_rn(v[i], sc)) : 0;
    q = max(-127, min(127, q));
    w[i >> 2] |= (uint32_t)(uint8_t)(int8_t)q << (8 * (i & 3));
  }
  *reinterpret_cast<uint2*>(q8 + (size_t)row * 256 + 8 * lane) = make_uint2(w[0], w[1]);
  if (lane == 0) scales[row] = sc;
}

template <int DT>
__global__ void __launch_bounds__(256) kvx_decode_kernel(const int8_t* q8, const float* scales, void* y, long long rows) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint2 u = __ldg(reinterpret_cast<const uint2*>(q8 + (size_t)row * 256 + 8 * lane));
  const float sc = __ldg(scales + row);
  float v[8];
  #pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __fmul_rn((float)(int8_t)(uint8_t)((i < 4 ? u.x : u.y) >> (8 * (i & 3))), sc);
  hadamard256(v, lane);
  apply_signs(v, lane);
  store8<DT>(y, (size_t)row, lane, v);
}

int grid_for(long long rows, unsigned* grid, const char* who) {
  if (rows < 0 || rows > (1ll << 34)) { set_error("%s: bad row count %lld", who, rows); return -1; }
  *grid = (unsigned)((rows + 7) / 8);
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

}  // namespace kv4
