// Family-B decode attention over INT8 rows (the cache the row codec of kvx_codec.cu writes): split-K flash-decode on
// the tensor cores for sm_100a, plus the merge with the inverse rotation.
//
// Semantics: the reference's q35_attention_kernel<KV8> (src/q35_kernels.cu:1176-1281) and the tail of its combine
// (src/q35_kernels.cu:1400-1425).  K and V rows are INT8 [Hkv][max_ctx][256] with one fp32 scale per row (ks, vs); Q
// arrives already rotated (kvx_rotate) and is scaled by qscale at load; row r sits at pos = *d_pos + r and sees keys
// 0..pos, all of them INT8 (Family B has no fp16 shadow and rotates K before storing, so nothing happens at read time):
//   s_t = qscale * (q . k8_t) * ks_t,   p_t = softmax(s)_t,   O = sum_t p_t * vs_t * v8_t      (rotated basis)
// Partials (m, l, O) per split in the reference's layout pm/pl [M][S][Hq], pacc [M][S][Hq][256]; the merge divides,
// rotates back (inverse kvx_rotate), rounds to bf16/fp16 and applies the optional sigmoid gate.
//
// Kernel shape: one CTA per (split, kv-head, row); a warp takes 16-token tiles.  Bytes go straight from HBM into
// registers (16-byte loads, K of the next tile and V of this tile in flight while the tensor cores work), because an
// INT8 row needs no staging transform: a lane's 16 K bytes of token g are the A fragments of four k-steps once each byte
// b is read as the fp16 number 1152 + b (byte ^ 0x80 under exponent 2^10, one PRMT per fragment register); the constant
// 1152 leaves through a per-head bias (K) and through 1152 * sum(p') (V).  The contraction index of S is a fixed
// permutation of the channels (slot (w, s, 2j+x) <-> channel 16(4w+j)+4s+x), applied to Q once at set-up; for P.V a lane
// owns channels [32g, 32g+32) of token rows 2j, 2j+1, 2j+8, 2j+9 and PRMT pairs the two tokens of a k-slot.
// HBM-bound: 2,080 bytes per token (4 kv-heads x 2 x 260).
#include "kv4_common.cuh"

namespace kv4 {
namespace {

constexpr int KV8_HD = 256;
constexpr int KV8_WARPS = 8;
constexpr float KV8_LOG2E = 1.4426950408889634f, KV8_LN2 = 0.6931471805599453f;
constexpr uint32_t C64 = 0x64646464u;                      // high bytes of the fp16 pattern 0x64xx = 1024 + xx
constexpr float KV8_OFF = 1152.f;                          // 1024 + 128: a byte b is read as 1152 + b

struct Kv8P { yskn_kv8_attn_args a; int g; };

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) { uint32_t d; asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a)); return d; }
__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) { uint32_t d; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo)); return d; }
__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }   // streamed once

template <int DT>
__global__ void __launch_bounds__(KV8_WARPS * 32, 1) kv8_decode_kernel(const Kv8P P) {
  extern __shared__ __align__(16) uint8_t smem[];
  // [16 k-steps][32 lanes] uint2 Q fragments | bias[8] | merge area [warps][8 heads][258]
  uint2* s_q = reinterpret_cast<uint2*>(smem);
  float* s_bias = reinterpret_cast<float*>(smem + 16 * 32 * 8);
  float* s_merge = s_bias + 8;
  const yskn_kv8_attn_args& A = P.a;
  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z, G = P.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
  const int len = *A.d_pos + r + 1;                        // keys 0 .. pos
  const int tiles = (len + 15) / 16, per = (tiles + (int)gridDim.x - 1) / (int)gridDim.x;
  const int ti0 = min(tiles, split * per), ti1 = min(tiles, ti0 + per);

  // ---- set-up: Q as B fragments in the slot order of the K loads, scaled by qscale * log2(e); the per-head bias
  const float qs = A.qscale * KV8_LOG2E;
  for (int e = threadIdx.x; e < 16 * 32 * 2; e += KV8_WARPS * 32) {
    const int x = e & 1, ln = (e >> 1) & 31, kstep = e >> 6, w = kstep >> 2, s = kstep & 3, hh = ln >> 2, jj = ln & 3;
    const int c = 16 * (4 * w + jj) + 4 * s + 2 * x;
    float lo = 0.f, hi = 0.f;
    if (hh < G) {
      const size_t qb = ((size_t)r * A.nh + kvh * G + hh) * KV8_HD;
      lo = act_load<DT>(A.q16, qb + c) * qs; hi = act_load<DT>(A.q16, qb + c + 1) * qs;
    }
    reinterpret_cast<uint32_t*>(s_q)[e] = pack_h2(lo, hi);
  }
  __syncthreads();
  if (threadIdx.x < 8) {                                   // bias[h] = 1152 * sum over the fp16 values the MMAs multiply by
    float sum = 0.f;
    for (int kstep = 0; kstep < 16; ++kstep)
      for (int jj = 0; jj < 4; ++jj) {
        const uint2 u = s_q[kstep * 32 + threadIdx.x * 4 + jj];
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        sum += (a.x + a.y) + (b.x + b.y);
      }
    s_bias[threadIdx.x] = KV8_OFF * sum;
  }
  __syncthreads();
  const float bias0 = s_bias[2 * j], bias1 = s_bias[2 * j + 1];

  float acc[16][4];                                        // O^T: [m-tile][(channel 32g+2mt | +1) x (head 2j | 2j+1)]
  #pragma unroll
  for (int mt = 0; mt < 16; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
  float m[2] = {-1e30f, -1e30f}, l[2] = {0.f, 0.f}, zs[2] = {0.f, 0.f};   // heads 2j, 2j+1 (log2 domain); zs = sum of rounded p'

  const size_t plane = (size_t)kvh * A.max_ctx;
  const int8_t* kbase = A.k8 + plane * KV8_HD + 16 * j;    // + token*256 + 64*w : this lane's 16 channels of block w
  const int8_t* vbase = A.v8 + plane * KV8_HD + 32 * g;    // + token*256 (+16)  : this lane's 32 channels
  const float* ksb = A.ks + plane; const float* vsb = A.vs + plane;

  uint4 kx[4], ky[4];                                      // K of the current tile: token g (x) and g+8 (y), blocks w = 0..3
  auto load_k = [&](int ti) {
    const size_t t = (size_t)16 * ti + g;
    #pragma unroll
    for (int w = 0; w < 4; ++w) { kx[w] = ldg16(kbase + t * KV8_HD + 64 * w); ky[w] = ldg16(kbase + (t + 8) * KV8_HD + 64 * w); }
  };
  int ti = ti0 + warp;
  if (ti < ti1) load_k(ti);
  for (; ti < ti1; ti += KV8_WARPS) {
    const int tg = 16 * ti + g;
    const bool v0 = tg < len, v1 = tg + 8 < len;
    // ---- V of this tile and the scales: in flight while S is computed
    uint4 vr[4][2];
    {
      const size_t ta = (size_t)16 * ti + 2 * j;
      const size_t tt[4] = {ta, ta + 1, ta + 8, ta + 9};
      #pragma unroll
      for (int q = 0; q < 4; ++q) { vr[q][0] = ldg16(vbase + tt[q] * KV8_HD); vr[q][1] = ldg16(vbase + tt[q] * KV8_HD + 16); }
    }
    const float ks0 = v0 ? __ldg(ksb + tg) : 0.f, ks1 = v1 ? __ldg(ksb + tg + 8) : 0.f;
    const float vs0 = v0 ? __ldg(vsb + tg) : 0.f, vs1 = v1 ? __ldg(vsb + tg + 8) : 0.f;
    // ---- S^T[16 tokens x 8 heads] = K . Q^T, two accumulation chains
    float sa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    #pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t xw[4] = {kx[w].x ^ 0x80808080u, kx[w].y ^ 0x80808080u, kx[w].z ^ 0x80808080u, kx[w].w ^ 0x80808080u};
      const uint32_t yw[4] = {ky[w].x ^ 0x80808080u, ky[w].y ^ 0x80808080u, ky[w].z ^ 0x80808080u, ky[w].w ^ 0x80808080u};
      #pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint2 qb = s_q[(4 * w + s) * 32 + lane];
        mma16816(sa[s & 1], __byte_perm(xw[s], C64, 0x4140), __byte_perm(yw[s], C64, 0x4140),
                 __byte_perm(xw[s], C64, 0x4342), __byte_perm(yw[s], C64, 0x4342), qb.x, qb.y);
      }
    }
    if (ti + KV8_WARPS < ti1) load_k(ti + KV8_WARPS);       // K of this warp's next tile: in flight during softmax and P.V
    // ---- softmax over the tile (log2 domain); rows g, g+8; heads 2j, 2j+1
    const float s00 = v0 ? (sa[0][0] + sa[1][0] - bias0) * ks0 : -INFINITY, s01 = v0 ? (sa[0][1] + sa[1][1] - bias1) * ks0 : -INFINITY;
    const float s10 = v1 ? (sa[0][2] + sa[1][2] - bias0) * ks1 : -INFINITY, s11 = v1 ? (sa[0][3] + sa[1][3] - bias1) * ks1 : -INFINITY;
    float t0 = fmaxf(s00, s10), t1 = fmaxf(s01, s11);
    #pragma unroll
    for (int o = 4; o <= 16; o <<= 1) { t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, o)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, o)); }
    if (__any_sync(0xffffffffu, t0 > m[0] + 8.f || t1 > m[1] + 8.f)) {   // lazy rescale: the running max may lag by 2^8
      const float n0 = fmaxf(m[0], t0), n1 = fmaxf(m[1], t1), a0 = ex2(m[0] - n0), a1 = ex2(m[1] - n1);
      m[0] = n0; m[1] = n1; l[0] *= a0; l[1] *= a1; zs[0] *= a0; zs[1] *= a1;
      #pragma unroll
      for (int mt = 0; mt < 16; ++mt) { acc[mt][0] *= a0; acc[mt][1] *= a1; acc[mt][2] *= a0; acc[mt][3] *= a1; }
    }
    const float p00 = v0 ? ex2(s00 - m[0]) : 0.f, p01 = v0 ? ex2(s01 - m[1]) : 0.f;
    const float p10 = v1 ? ex2(s10 - m[0]) : 0.f, p11 = v1 ? ex2(s11 - m[1]) : 0.f;
    l[0] += p00 + p10; l[1] += p01 + p11;
    // the row scale of V goes into P (fp16); the 1152 offset of the V operand leaves through the sum of the ROUNDED p'
    const uint32_t pp0 = pack_h2(p00 * vs0, p01 * vs0), pp1 = pack_h2(p10 * vs1, p11 * vs1);
    const float2 pr0 = __half22float2(*reinterpret_cast<const __half2*>(&pp0)), pr1 = __half22float2(*reinterpret_cast<const __half2*>(&pp1));
    zs[0] += pr0.x + pr1.x; zs[1] += pr0.y + pr1.y;
    const uint32_t pb0 = movmatrix_t(pp0), pb1 = movmatrix_t(pp1);     // B regs: (tokens 2j,2j+1 | head g), (tokens 2j+8,2j+9 | head g)
    // ---- O^T += V^T P^T: m-tile mt = channels (32g + 2mt, 32g + 2mt + 1) as rows (g, g+8)
    #pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t wa[4] = {vr[0][h].x, vr[0][h].y, vr[0][h].z, vr[0][h].w}, wb[4] = {vr[1][h].x, vr[1][h].y, vr[1][h].z, vr[1][h].w};
      const uint32_t wc[4] = {vr[2][h].x, vr[2][h].y, vr[2][h].z, vr[2][h].w}, wd[4] = {vr[3][h].x, vr[3][h].y, vr[3][h].z, vr[3][h].w};
      #pragma unroll
      for (int wi = 0; wi < 4; ++wi)
        #pragma unroll
        for (int half = 0; half < 2; ++half) {                           // bytes (0,1) then (2,3) of the word
          const uint32_t sel = half ? 0x7362u : 0x5140u;                 // [A.b, B.b, A.b', B.b']
          const uint32_t ab = __byte_perm(wa[wi], wb[wi], sel) ^ 0x80808080u, cd = __byte_perm(wc[wi], wd[wi], sel) ^ 0x80808080u;
          mma16816(acc[8 * h + 2 * wi + half], __byte_perm(ab, C64, 0x4140), __byte_perm(ab, C64, 0x4342),
                   __byte_perm(cd, C64, 0x4140), __byte_perm(cd, C64, 0x4342), pb0, pb1);
        }
    }
  }

  // ---- this warp's (m, l, O) per head: sums over the token lanes, the operand offset removed
  #pragma unroll
  for (int o = 4; o <= 16; o <<= 1) {
    l[0] += __shfl_xor_sync(0xffffffffu, l[0], o); l[1] += __shfl_xor_sync(0xffffffffu, l[1], o);
    zs[0] += __shfl_xor_sync(0xffffffffu, zs[0], o); zs[1] += __shfl_xor_sync(0xffffffffu, zs[1], o);
  }
  {
    float* mine = s_merge + (size_t)warp * 8 * 258;
    #pragma unroll
    for (int mt = 0; mt < 16; ++mt) {
      const int c = 32 * g + 2 * mt;
      mine[(2 * j) * 258 + 2 + c] = acc[mt][0] - KV8_OFF * zs[0]; mine[(2 * j + 1) * 258 + 2 + c] = acc[mt][1] - KV8_OFF * zs[1];
      mine[(2 * j) * 258 + 2 + c + 1] = acc[mt][2] - KV8_OFF * zs[0]; mine[(2 * j + 1) * 258 + 2 + c + 1] = acc[mt][3] - KV8_OFF * zs[1];
    }
    if (g == 0) { mine[(2 * j) * 258] = m[0]; mine[(2 * j) * 258 + 1] = l[0]; mine[(2 * j + 1) * 258] = m[1]; mine[(2 * j + 1) * 258 + 1] = l[1]; }
  }
  __syncthreads();
  // ---- merge the warps and store the split's partial (m in the natural-log domain, as the reference's partials)
  for (int e = threadIdx.x; e < G * KV8_HD; e += KV8_WARPS * 32) {
    const int hh = e / KV8_HD, d = e % KV8_HD;
    float M2 = -1e30f;
    #pragma unroll
    for (int w = 0; w < KV8_WARPS; ++w) M2 = fmaxf(M2, s_merge[((size_t)w * 8 + hh) * 258]);
    float L2 = 0.f, o = 0.f;
    #pragma unroll
    for (int w = 0; w < KV8_WARPS; ++w) {
      const float* src = s_merge + ((size_t)w * 8 + hh) * 258;
      const float sc = src[0] > -1e29f ? ex2(src[0] - M2) : 0.f;
      L2 += sc * src[1]; o += sc * src[2 + d];
    }
    const size_t pidx = ((size_t)r * A.splits + split) * A.nh + kvh * G + hh;
    if (d == 0) { A.pm[pidx] = M2 > -1e29f ? M2 * KV8_LN2 : -1e30f; A.pl[pidx] = L2; }
    A.pacc[pidx * KV8_HD + d] = o;
  }
}

// ---- merge of the splits + inverse rotation + rounding (+ gate): one block per (head, row), one thread per channel
template <int DT>
__global__ void __launch_bounds__(256) kv8_combine_kernel(const float* pm, const float* pl, const float* pacc, int S, int M, int nh,
                                                         const void* gate, void* o16, int inverse_rotate) {
  __shared__ float s_w[64], s_buf[256];
  __shared__ float s_L;
  const int head = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
  auto slot = [&](int s) -> size_t { return ((size_t)r * S + s) * nh + head; };
  float M2 = -1e30f;
  for (int s = 0; s < S; ++s) M2 = fmaxf(M2, __ldcg(pm + slot(s)));
  if (d < S) { const float pmv = __ldcg(pm + slot(d)); s_w[d] = pmv > -1e29f ? expf(pmv - M2) : 0.f; }
  __syncthreads();
  if (d == 0) { float L2 = 0.f; for (int s = 0; s < S; ++s) L2 += s_w[s] * __ldcg(pl + slot(s)); s_L = L2; }
  float o = 0.f;
  for (int s = 0; s < S; ++s) o += s_w[s] * __ldcg(pacc + slot(s) * KV8_HD + d);
  __syncthreads();
  float y = __fdiv_rn(o, s_L);
  if (inverse_rotate) {                                    // inverse kvx_rotate (src/kvx_codec.cuh:35-49): butterflies, x 1/16, then the sign
    s_buf[d] = y;
    __syncthreads();
    for (int h = 1; h < 256; h *= 2) {
      const float a = s_buf[d], b = s_buf[d ^ h];
      __syncthreads();
      s_buf[d] = (d & h) ? __fsub_rn(b, a) : __fadd_rn(a, b);
      __syncthreads();
    }
    uint32_t x = (uint32_t)d + 1u;
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    y = __fmul_rn(s_buf[d], 0.0625f);
    if (x & 1u) y = -y;
  }
  const size_t e = ((size_t)r * nh + head) * KV8_HD + d;
  auto rnd = [](float v) -> float { return DT == YSKN_KV4_BF16 ? bf2f(f2bf(v)) : h2f(f2h(v)); };
  y = rnd(y);
  if (gate) {                                              // y * sigmoid(gate), each factor and the product rounded (src/q35_kernels.cu:1423-1424)
    const float gt = act_load<DT>(gate, e);
    const float sg = rnd(__fdiv_rn(1.f, __fadd_rn(1.f, expf(-gt))));
    y = rnd(__fmul_rn(y, sg));
  }
  static_cast<uint16_t*>(o16)[e] = act_store16<DT>(y);
}

}  // namespace

int launch_kv8_attention(const yskn_kv8_attn_args& a, int act_dtype, cudaStream_t st) {
  if (!a.q16 || !a.k8 || !a.v8 || !a.ks || !a.vs || !a.d_pos || !a.pm || !a.pl || !a.pacc) KV4_REJECT("yskn_kv8_attention: null buffer");
  if (a.kvh <= 0 || a.nh <= 0 || a.nh % a.kvh || a.nh / a.kvh > 8 || a.M <= 0 || a.M > 65535 || a.kvh > 65535 || a.splits <= 0 || a.max_ctx <= 0 || a.max_ctx % 64)
    KV4_REJECT("yskn_kv8_attention: bad shape (kvh %d, nh %d, M %d, splits %d, max_ctx %d): at most 8 query heads per kv-head, max_ctx a multiple of 64",
               a.kvh, a.nh, a.M, a.splits, a.max_ctx);
  if (((uintptr_t)a.k8 | (uintptr_t)a.v8) & 15) KV4_REJECT("yskn_kv8_attention: k8 and v8 must be 16-byte aligned");
  const size_t smem = 16 * 32 * 8 + 8 * 4 + (size_t)KV8_WARPS * 8 * 258 * 4;
  Kv8P P{a, a.nh / a.kvh};
  const dim3 grid(a.splits, a.kvh, a.M);
  if (act_dtype == YSKN_KV4_BF16) {
    static std::atomic<unsigned long long> attr{0};
    if (first_use_on_device(attr)) KV4_CUDA(cudaFuncSetAttribute(kv8_decode_kernel<YSKN_KV4_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kv8_decode_kernel<YSKN_KV4_BF16><<<grid, KV8_WARPS * 32, smem, st>>>(P);
  } else if (act_dtype == YSKN_KV4_F16) {
    static std::atomic<unsigned long long> attr{0};
    if (first_use_on_device(attr)) KV4_CUDA(cudaFuncSetAttribute(kv8_decode_kernel<YSKN_KV4_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kv8_decode_kernel<YSKN_KV4_F16><<<grid, KV8_WARPS * 32, smem, st>>>(P);
  } else KV4_REJECT("yskn_kv8_attention: q16 is bf16 or fp16 (act_dtype %d)", act_dtype);
  return launch_status("kv8_decode_kernel");
}

int launch_kv8_combine(const float* pm, const float* pl, const float* pacc, int splits, int M, int nh, const void* gate, void* o16,
                       int act_dtype, int inverse_rotate, cudaStream_t st) {
  if (!pm || !pl || !pacc || !o16) KV4_REJECT("yskn_kv8_combine: null buffer");
  if (splits <= 0 || splits > 64 || M <= 0 || nh <= 0) KV4_REJECT("yskn_kv8_combine: bad shape (splits %d of at most 64, M %d, nh %d)", splits, M, nh);
  const dim3 grid(nh, M);
  if (act_dtype == YSKN_KV4_BF16) kv8_combine_kernel<YSKN_KV4_BF16><<<grid, 256, 0, st>>>(pm, pl, pacc, splits, M, nh, gate, o16, inverse_rotate);
  else if (act_dtype == YSKN_KV4_F16) kv8_combine_kernel<YSKN_KV4_F16><<<grid, 256, 0, st>>>(pm, pl, pacc, splits, M, nh, gate, o16, inverse_rotate);
  else KV4_REJECT("yskn_kv8_combine: o16 is bf16 or fp16 (act_dtype %d)", act_dtype);
  return launch_status("kv8_combine_kernel");
}

}  // namespace kv4
