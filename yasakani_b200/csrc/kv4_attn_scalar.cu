// Generic KV4 GQA attention on CUDA cores (sm_100a): any M, any G <= 8, head_dim 64/128/256, any even
// rotary width.  This is the shape-complete path; the tensor-core kernels take over the shapes they cover.
//
// Semantics follow the reference's attention_gqa_kernel (src/attention_gqa.cu:17-118): row r sits at
// pos = *d_pos + r and sees keys 0..pos; split s covers keys [s*per, min(len,(s+1)*per)) with
// per = ceil(len/splits); keys of 32-token groups before the row's own group are int4
// (nib*scale + zero, separate multiply and add), keys of the own group come from the fp16 shadow; K is
// rotated at read time with the caller's (cos,sin) table; V is always int4 per token; partials are
// (m, l, un-normalised O) per (row, split, head).
// Extras of the 27B engine's argument set (yskn_kv4_attn_ext; src/q35_atx.cu:111-119): with a row -> depth table `wk`, row r
// sits at position *d_pos + wk[r], sees the cached keys below that position and its own key, which is stored in cache slot
// *d_pos + r (read from the shadow, rotated by the row's position); rows that see fewer than long_len keys use
// splits_short splits and leave the remaining partial slots empty (pm = -1e30).
//
// Work split: grid (splits, Hkv, M); four warps stride the tokens of the split; a lane owns HD/32
// contiguous channels, so one token's packed K or V row is a single coalesced 64/128-byte warp load.
#include "kv4_common.cuh"

namespace kv4 {
namespace {

template <int G, int HD, int DT>
__global__ void __launch_bounds__(128) kv4_attn_scalar_kernel(yskn_attn_g_args A, int rd, Shard sh, yskn_kv4_attn_ext X) {
  constexpr int CPL = HD / 32;
  __shared__ float s_m[4][G], s_l[4][G];
  __shared__ float s_acc[4][G][HD];
  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // pos/len/cur_group are LOCAL to this shard: local token t is global token t + sh.start (1 GPU: start 0)
  const int base = *A.d_pos, dp = X.wk ? (int)X.wk[r] : r;
  const int pos = base + dp - sh.start, own = base + r - sh.start;   // the row's position; the slot of its own key (== pos without wk)
  const int len = max(0, min(pos + 1, sh.len));
  const int S = (X.splits_short > 0 && base + dp + 1 < X.long_len) ? X.splits_short : A.splits;   // src/q35_atx.cu:113
  const int per = (len + S - 1) / S;
  const int t0 = min(len, split * per), t1 = split < S ? min(len, t0 + per) : t0, cur_group = pos / 32;
  const int c0 = lane * CPL;                          // first channel of this lane
  const int half = rd / 2, lanes_off = half / CPL;    // rotary partner distance in lanes
  const bool rot = c0 < rd, lower = c0 < half;

  float q[G][CPL], acc[G][CPL], m[G], l[G];
  #pragma unroll
  for (int i = 0; i < G; ++i) {
    m[i] = -1e30f; l[i] = 0.f;
    #pragma unroll
    for (int e = 0; e < CPL; ++e) {
      q[i][e] = __fmul_rn(act_load<DT>(A.q16, ((size_t)r * A.nh + kvh * G + i) * HD + c0 + e), A.qscale);
      acc[i][e] = 0.f;
    }
  }

  for (int t = t0 + warp; t < t1; t += 4) {
    float kd[CPL], vd[CPL];
    if (t / 32 < cur_group) {
      const size_t gb = (size_t)kvh * (A.max_ctx / 32) + t / 32;
      const uint8_t* kb = A.kv.kq + (gb * 32 + (t & 31)) * (HD / 2) + c0 / 2;
      #pragma unroll
      for (int e = 0; e < CPL; e += 2) {
        const uint8_t b = kb[e / 2];
        const uint32_t s2 = *reinterpret_cast<const uint32_t*>(A.kv.kscale + gb * HD + c0 + e);
        const uint32_t z2 = *reinterpret_cast<const uint32_t*>(A.kv.kzero + gb * HD + c0 + e);
        kd[e] = __fadd_rn(__fmul_rn((float)(b & 15), h2f((uint16_t)s2)), h2f((uint16_t)z2));
        kd[e + 1] = __fadd_rn(__fmul_rn((float)(b >> 4), h2f((uint16_t)(s2 >> 16))), h2f((uint16_t)(z2 >> 16)));
      }
    } else {
      const uint16_t* ks = A.kv.kshadow + ((size_t)kvh * A.max_ctx + (t == pos ? own : t)) * HD + c0;
      #pragma unroll
      for (int e = 0; e < CPL; e += 2) {
        const uint32_t u = *reinterpret_cast<const uint32_t*>(ks + e);
        kd[e] = h2f((uint16_t)u); kd[e + 1] = h2f((uint16_t)(u >> 16));
      }
    }
    if (rd > 0) {                                     // rotate-half over the first rd channels
      #pragma unroll
      for (int e = 0; e < CPL; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, kd[e], lanes_off);
        if (rot) {
          const float2 cs = *reinterpret_cast<const float2*>(A.rope + ((size_t)(t + sh.start) * half + ((c0 + e) % half)) * 2);
          kd[e] = lower ? (kd[e] * cs.x - other * cs.y) : (other * cs.y + kd[e] * cs.x);
        }
      }
    }
    {
      const size_t slot = (size_t)kvh * A.max_ctx + (t == pos ? own : t);
      const float vs = h2f(A.kv.vscale[slot]), vz = h2f(A.kv.vzero[slot]);
      const uint8_t* vb = A.kv.vq + slot * (HD / 2) + c0 / 2;
      #pragma unroll
      for (int e = 0; e < CPL; e += 2) { const uint8_t b = vb[e / 2]; vd[e] = (float)(b & 15) * vs + vz; vd[e + 1] = (float)(b >> 4) * vs + vz; }
    }
    #pragma unroll
    for (int i = 0; i < G; ++i) {
      float s = 0.f;
      #pragma unroll
      for (int e = 0; e < CPL; ++e) s += q[i][e] * kd[e];
      #pragma unroll
      for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mn = fmaxf(m[i], s), a = expf(m[i] - mn), b = expf(s - mn);
      l[i] = l[i] * a + b;
      #pragma unroll
      for (int e = 0; e < CPL; ++e) acc[i][e] = acc[i][e] * a + b * vd[e];
      m[i] = mn;
    }
  }

  #pragma unroll
  for (int i = 0; i < G; ++i) {
    if (lane == 0) { s_m[warp][i] = m[i]; s_l[warp][i] = l[i]; }
    #pragma unroll
    for (int e = 0; e < CPL; ++e) s_acc[warp][i][c0 + e] = acc[i][e];
  }
  __syncthreads();
  for (int i = warp; i < G; i += 4) {                 // merge the four warps, one head per warp
    float M2 = s_m[0][i];
    #pragma unroll
    for (int w = 1; w < 4; ++w) M2 = fmaxf(M2, s_m[w][i]);
    float L2 = 0.f, o[CPL];
    #pragma unroll
    for (int e = 0; e < CPL; ++e) o[e] = 0.f;
    #pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sc = (s_m[w][i] > -1e29f) ? expf(s_m[w][i] - M2) : 0.f;
      L2 += sc * s_l[w][i];
      #pragma unroll
      for (int e = 0; e < CPL; ++e) o[e] += sc * s_acc[w][i][c0 + e];
    }
    const size_t p = ((size_t)r * A.splits + split) * A.nh + kvh * G + i;
    if (lane == 0) { A.pm[p] = M2; A.pl[p] = L2; }
    #pragma unroll
    for (int e = 0; e < CPL; ++e) A.pacc[p * HD + c0 + e] = o[e];
  }
}

template <int G, int HD> int launch_gd(const yskn_attn_g_args& a, int rd, int dt, Shard sh, const yskn_kv4_attn_ext& x, cudaStream_t st) {
  const dim3 grid(a.splits, a.kvh, a.M);
  if (dt == YSKN_KV4_F16) kv4_attn_scalar_kernel<G, HD, YSKN_KV4_F16><<<grid, 128, 0, st>>>(a, rd, sh, x);
  else kv4_attn_scalar_kernel<G, HD, YSKN_KV4_BF16><<<grid, 128, 0, st>>>(a, rd, sh, x);
  return launch_status("kv4_attn_scalar_kernel");
}
template <int HD> int launch_d(const yskn_attn_g_args& a, int g, int rd, int dt, Shard sh, const yskn_kv4_attn_ext& x, cudaStream_t st) {
  switch (g) {
    case 1: return launch_gd<1, HD>(a, rd, dt, sh, x, st);
    case 2: return launch_gd<2, HD>(a, rd, dt, sh, x, st);
    case 3: return launch_gd<3, HD>(a, rd, dt, sh, x, st);
    case 4: return launch_gd<4, HD>(a, rd, dt, sh, x, st);
    case 5: return launch_gd<5, HD>(a, rd, dt, sh, x, st);
    case 6: return launch_gd<6, HD>(a, rd, dt, sh, x, st);
    case 7: return launch_gd<7, HD>(a, rd, dt, sh, x, st);
    case 8: return launch_gd<8, HD>(a, rd, dt, sh, x, st);
  }
  KV4_REJECT("yskn_kv4_attention: unsupported group size %d (1..8)", g);
}

}  // namespace

int launch_attention_scalar(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, Shard sh, cudaStream_t st, const yskn_kv4_attn_ext* ext) {
  yskn_kv4_attn_ext x{0, 0, 0, nullptr};
  if (ext) x = *ext;
  const int cpl = hd / 32;
  if (rd < 0 || rd > hd || (rd & 1) || (rd > 0 && ((rd / 2) % cpl || ((rd / 2 / cpl) & (rd / 2 / cpl - 1)))))
    KV4_REJECT("yskn_kv4_attention: unsupported rotary width %d for head_dim %d", rd, hd);   // src/attention_gqa.cu:174
  if (hd == 256) return launch_d<256>(a, g, rd, act_dtype, sh, x, st);
  if (hd == 128) return launch_d<128>(a, g, rd, act_dtype, sh, x, st);
  if (hd == 64) return launch_d<64>(a, g, rd, act_dtype, sh, x, st);
  KV4_REJECT("yskn_kv4_attention: unsupported head_dim %d (64, 128, 256)", hd);
}

}  // namespace kv4
