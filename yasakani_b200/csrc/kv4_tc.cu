// Multi-row KV4 attention on the 5th-generation tensor cores (tcgen05 + TMEM) for sm_100a: the verify pass
// (up to 64 query rows against a long cache) and causal prefill (thousands of rows).
//
// Semantics: the reference's Family-A attention for M rows (src/attention_gqa.cu:17-118, src/attention_kv4q.cu:381-448):
// row r sits at pos = *d_pos + r, sees keys 0..pos, reads 32-token groups before its own group as int4 and its own
// group from the fp16 shadow, K rotated at read time, V int4 per token.  Tile shapes and the split of the key range
// follow the reference's tensor-core verify kernels in spirit (rows = (token, head) pairs packed into MMA tiles per
// kv-head, split-K partials in the same [M][splits][Hq] layout; src/q35_fa.cu:48-303, src/q35_atx.cu:92-793).
//
// Two kernels.
//  1. kv4_tc_prep_kernel dequantises the cache once per pass into a caller-owned fp16 workspace, as the reference's
//     kv_dequant_kernel does into fp32 (src/attention_kv4q.cu:198-243): Kd = rotated int4 keys of every complete
//     group, Vd = int4 values of every token, Ks = rotated fp16-shadow keys of the groups the new rows live in.
//     fp32 arithmetic, one rounding to fp16.  HBM-bound byte mover: one warp per (token, kv-head).
//  2. kv4_tc_attn_kernel: a pair of CTAs (cluster of two, tcgen05 cta_group::2) = 256 query rows ((token, head) pairs
//     of one kv-head, 128 per CTA) x one split of the keys, in tiles of 128 keys.  Per CTA:
//       warp 8      TMA producer: its Q rows once, then its half of every K tile (64 keys) and V tile (HD/2 channels)
//                   into two mbarrier rings, one tiled copy each; the copies report to the leader CTA's barriers
//       warp 9      (leader CTA only) one thread issues every tcgen05.mma of the pair: S = Q.K^T (M256 N128 K16 steps, Q and
//                   K from shared memory, K-major, 128-byte swizzle) into one of two TMEM buffers, and O += P.V (M256
//                   N=HD, P from tensor memory, V as MN-major operand); commits arrive on both CTAs' barriers
//       warps 0-7   two threads per query row (64 of the tile's 128 keys each): tcgen05.ld of the S row, masks, online
//                   softmax in the log2 domain with a lazy rescale of O, P -> fp16 -> tensor memory over the S columns
//                   just read; final (m, l, O) store, or the finished fp16 row when there is a single split
//     S of tile i+2 is issued right after P.V of tile i, so the tensor pipe works while the softmax warps run.
//     Tiles that contain a row's own group ("edge" tiles) get S twice, from Kd and from Ks, and each row picks per
//     32-key group: int4 keys for groups before its own, shadow keys (causally masked) for its own.
//
//  The attention kernel has four forms (template FORM): 0 = operand tiles by TMA from the workspace, as above (3 = the same
//  with bf16 queries and output rows: the softmax warps convert the queries, there is no Q copy); 1 = no
//  workspace and no prep launch, converter warps build the tiles from the packed KV4 cache inside the kernel; 2 = the same over
//  Family-B INT8 rows.  The converting forms run 16 warps: 0-7 softmax, 8 Q copy + MMA issue, 9-11 V tiles, 12-15 K tiles.
//
// Rows are independent of one another inside every step (an MMA output row depends on its own A row only, the lazy
// rescale multiplies other rows by exactly 1), tiles start at multiples of 128 keys and split boundaries depend on
// *d_pos and `splits` only, so a row's result does not depend on how many rows the pass holds.
//
// Every wait is bounded; a wait that runs out sets the device status word (4/5/6 = softmax / MMA / producer) and the CTA
// frees its TMEM and returns.
#include "kv4_common.cuh"
#include <cuda.h>
#include <cstring>
#include <mutex>
#include <unordered_map>

namespace kv4 {

__device__ int g_tc_status = 0;              // 0 ok; 4/5/6 = a bounded wait ran out in the softmax warps / MMA warp / producer


namespace {

constexpr int TC_BN = 128;                                 // keys per tile of the attention kernel

// ------------------------------------------------------------------------------------------------ prep kernel
struct PrepP {
  yskn_kv_layer kv; const int* d_pos; int M; int max_ctx; int kvh; const float* rope; int rd;
  uint16_t* kd; uint16_t* vd; uint16_t* ks; int ks_rows; int valid_tokens;
  int t_begin;                                             // first token the grid covers: nothing below it needs (re)writing
};

// Nibble e of a packed word as an exact float: the nibble placed in the low mantissa bits of 2^23 reads as 8388608 + n.
__device__ __forceinline__ float nib_f32(uint32_t w, int e) {
  return __fsub_rn(__uint_as_float(((w >> (4 * e)) & 15u) | 0x4B000000u), 8388608.f);
}
__device__ __forceinline__ uint32_t tc_pack(float lo, float hi);

// CPL nibbles (CPL/2 bytes) or CPL fp16 values of one lane in a single load
template <int CPL> __device__ __forceinline__ uint32_t load_packed(const uint8_t* p) {
  if (CPL == 8) return __ldg(reinterpret_cast<const uint32_t*>(p));
  return (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p));
}
template <int CPL> __device__ __forceinline__ void load_halves(const uint16_t* p, uint32_t (&o)[CPL / 2]) {
  if (CPL == 8) { const uint4 u = __ldg(reinterpret_cast<const uint4*>(p)); o[0] = u.x; o[1] = u.y; o[CPL / 2 - 2] = u.z; o[CPL / 2 - 1] = u.w; }
  else { const uint2 u = __ldg(reinterpret_cast<const uint2*>(p)); o[0] = u.x; o[CPL / 2 - 1] = u.y; }
}

// One warp per (token t, kv-head); lane owns HD/32 contiguous channels.
template <int HD>
__global__ void __launch_bounds__(128) kv4_tc_prep_kernel(PrepP P) {
  constexpr int CPL = HD / 32;
  const int lane = threadIdx.x & 31;
  const int t = P.t_begin + (int)blockIdx.x * 4 + (int)(threadIdx.x >> 5), head = blockIdx.y;   // grid (tokens / 4, kv-heads)
  const int pos0 = *P.d_pos, end = pos0 + P.M;                      // tokens [0, end) exist
  const int end_tile = min(P.max_ctx, (end + TC_BN - 1) / TC_BN * TC_BN);   // tiles read whole rows of keys: keep V finite there
  if (t >= end_tile) return;
  const int c0 = lane * CPL, half = P.rd / 2, lanes_off = half > 0 ? half / CPL : 1;
  const bool rot = c0 < P.rd, lower = c0 < half;
  const size_t row = (size_t)head * P.max_ctx + t;
  auto store = [&](uint16_t* dst, const float (&v)[CPL]) {        // one 16-byte (hd 256) or 8-byte (hd 128) store per lane
    uint32_t w2[CPL / 2];
    #pragma unroll
    for (int e = 0; e < CPL; e += 2) w2[e / 2] = tc_pack(v[e], v[e + 1]);      // one conversion per pair
    if (CPL == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(w2[0], w2[1], w2[CPL / 2 - 2], w2[CPL / 2 - 1]);
    else *reinterpret_cast<uint2*>(dst) = make_uint2(w2[0], w2[CPL / 2 - 1]);
  };
  auto rotate = [&](float (&k)[CPL]) {
    if (P.rd <= 0) return;
    // (cos, sin) of this lane's CPL frequencies: consecutive table entries (rd / 2 is a power of two).  Lanes outside the
    // rotary width read entry 0 and keep their values by a select, so the loop has no divergent branches.
    const float4* rp = reinterpret_cast<const float4*>(P.rope + ((size_t)t * half + (rot ? (c0 & (half - 1)) : 0)) * 2);
    float4 cs2[CPL / 2];
    #pragma unroll
    for (int e = 0; e < CPL / 2; ++e) cs2[e] = __ldg(rp + e);
    #pragma unroll
    for (int e = 0; e < CPL; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, k[e], lanes_off);
      const float cx = (e & 1) ? cs2[e / 2].z : cs2[e / 2].x, sy = (e & 1) ? cs2[e / 2].w : cs2[e / 2].y;
      const float r = lower ? (k[e] * cx - other * sy) : (other * sy + k[e] * cx);
      k[e] = rot ? r : k[e];
    }

  };
  // ---- V: every token below `end`, zero rows up to the tile boundary
  if (t >= P.valid_tokens) {
    float v[CPL];
    if (t < end) {
      const float vs = h2f(P.kv.vscale[row]), vz = h2f(P.kv.vzero[row]);
      const uint32_t vw = load_packed<CPL>(P.kv.vq + row * (HD / 2) + c0 / 2);      // this lane's CPL nibbles in one load
      #pragma unroll
      for (int e = 0; e < CPL; e += 2) { v[e] = nib_f32(vw, e) * vs + vz; v[e + 1] = nib_f32(vw, e + 1) * vs + vz; }
    } else {
      #pragma unroll
      for (int e = 0; e < CPL; ++e) v[e] = 0.f;
    }
    store(P.vd + row * HD + c0, v);
  }
  // ---- Kd: tokens of complete groups (32g+31 < end), rotated
  const int gi = t / 32;
  if (gi * 32 + 31 < end && t >= (P.valid_tokens / 32) * 32) {       // a group completed since the last pass is (re)written whole
    const size_t gb = (size_t)head * (P.max_ctx / 32) + gi;
    const uint32_t kw = load_packed<CPL>(P.kv.kq + (gb * 32 + (t & 31)) * (HD / 2) + c0 / 2);
    uint32_t sw[CPL / 2], zw[CPL / 2];                                 // this lane's CPL scales and zeros in one load each
    load_halves<CPL>(P.kv.kscale + gb * HD + c0, sw); load_halves<CPL>(P.kv.kzero + gb * HD + c0, zw);
    float k[CPL];
    #pragma unroll
    for (int e = 0; e < CPL; e += 2) {
      const uint32_t s2 = sw[e / 2], z2 = zw[e / 2];
      k[e] = __fadd_rn(__fmul_rn(nib_f32(kw, e), h2f((uint16_t)s2)), h2f((uint16_t)z2));
      k[e + 1] = __fadd_rn(__fmul_rn(nib_f32(kw, e + 1), h2f((uint16_t)(s2 >> 16))), h2f((uint16_t)(z2 >> 16)));
    }
    rotate(k);
    store(P.kd + row * HD + c0, k);
  }
  // ---- Ks: rotated shadow keys from the tile that holds *d_pos onwards (row index relative to that tile)
  const int ks0 = (pos0 / TC_BN) * TC_BN;
  if (t >= ks0 && t - ks0 < P.ks_rows) {
    float k[CPL];
    if (t < end) {
      uint32_t sw2[CPL / 2];
      load_halves<CPL>(P.kv.kshadow + row * HD + c0, sw2);
      #pragma unroll
      for (int e = 0; e < CPL; e += 2) { const uint32_t u = sw2[e / 2]; k[e] = h2f((uint16_t)u); k[e + 1] = h2f((uint16_t)(u >> 16)); }
      rotate(k);
    } else {
      #pragma unroll
      for (int e = 0; e < CPL; ++e) k[e] = 0.f;
      rotate(k);                                                     // keeps the shuffles convergent
    }
    store(P.ks + ((size_t)head * P.ks_rows + (t - ks0)) * HD + c0, k);
  }
}


// ------------------------------------------------------------------------------------------------ PTX helpers
constexpr uint32_t TC_WAIT_LIMIT = 1u << 22;
constexpr float TC_LOG2E = 1.4426950408889634f, TC_LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool bar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {          // bounded; false = gave up
  for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) if (bar_try(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// Address of the leader CTA's copy (rank 0 of the pair) of a shared-memory location, in the cluster window.
__device__ __forceinline__ uint32_t leader_addr(uint32_t local) { uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(local)); return r; }
// What the arrival publishes lives in tensor memory and is ordered by the tcgen05 fences around it, so the default
// (CTA-scope) release is enough; a cluster-scope release costs several hundred cycles per call.
__device__ __forceinline__ void bar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Data that a CTA's converter warps wrote into its own shared memory with ordinary stores is read by the tensor core of the
// same SM: each writer orders its stores for the async proxy (fence.proxy.async), the warp then arrives on the leader's
// barrier and the issuing thread waits on it, both with the default release / acquire; no other SM ever reads these bytes
// with ordinary loads.
__device__ __forceinline__ void cluster_sync_all() {                 // every thread of both CTAs
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, int z, int w, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
               ::"r"(dst), "l"(m), "r"(x), "r"(y), "r"(z), "r"(w), "r"(cluster_bar) : "memory");
}
// One tiled copy into this CTA's shared memory that reports its bytes to a barrier of the pair's leader.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* m, int x, int y, int z, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(m), "r"(x), "r"(y), "r"(z), "r"(cluster_bar) : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100): start address, leading and stride byte offsets
// in 16-byte units.  K-major operands: 8-row x 128-byte atoms, SBO = 1024 between atoms along M/N, LBO unused.
// MN-major operands: 128-byte rows hold 64 M/N-elements of one k; SBO = 1024 between groups of 8 k; LBO = distance
// between 64-element blocks along M/N.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: fp16 A and B, fp32 accumulator, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, bool b_mn_major) {
  return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// A operand (128 rows x 16 k, fp16 pairs in 8 columns) from tensor memory, B from shared memory.
__device__ __forceinline__ void umma2_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// One instruction drives the tensor cores of both SMs of the pair (M = 256: 128 rows in each CTA's tensor memory).
__device__ __forceinline__ void umma2_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in BOTH CTAs once all MMAs issued so far are done.
__device__ __forceinline__ void umma2_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                 "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
                 "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  #pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {            // two loads in flight, one wait
  uint32_t r[64];
  #pragma unroll
  for (int h = 0; h < 2; ++h)
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[32 * h + 0]), "=r"(r[32 * h + 1]), "=r"(r[32 * h + 2]), "=r"(r[32 * h + 3]), "=r"(r[32 * h + 4]), "=r"(r[32 * h + 5]), "=r"(r[32 * h + 6]),
                   "=r"(r[32 * h + 7]), "=r"(r[32 * h + 8]), "=r"(r[32 * h + 9]), "=r"(r[32 * h + 10]), "=r"(r[32 * h + 11]), "=r"(r[32 * h + 12]), "=r"(r[32 * h + 13]),
                   "=r"(r[32 * h + 14]), "=r"(r[32 * h + 15]), "=r"(r[32 * h + 16]), "=r"(r[32 * h + 17]), "=r"(r[32 * h + 18]), "=r"(r[32 * h + 19]), "=r"(r[32 * h + 20]),
                   "=r"(r[32 * h + 21]), "=r"(r[32 * h + 22]), "=r"(r[32 * h + 23]), "=r"(r[32 * h + 24]), "=r"(r[32 * h + 25]), "=r"(r[32 * h + 26]), "=r"(r[32 * h + 27]),
                   "=r"(r[32 * h + 28]), "=r"(r[32 * h + 29]), "=r"(r[32 * h + 30]), "=r"(r[32 * h + 31])
                 : "r"(taddr + 32 * h) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  #pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
                 "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])),
                 "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
                 "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                 "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])),
                 "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
                 "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31])) : "memory");
}
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]),
                 "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                 "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float tc_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t tc_pack(float lo, float hi) { uint32_t d; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo)); return d; }

// ------------------------------------------------------------------------------------------------ int4 -> fp16 operand rows
// A packed 32-bit word holds the nibbles of eight consecutive channels.  One logic op reads nibbles (x, x + 4) in place as
// the fp16 pair (off + n_x, off + n_{x+4}) (off = 1024 under exponent 2^10 for bits 0..3 of a half, 64 under 2^6 for bits
// 4..7); the offset is removed by an exact fp16 subtraction, so n[x] holds the two nibbles as exact small integers.
__device__ __forceinline__ uint32_t tc_hadd2(uint32_t a, uint32_t b) { uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t tc_hfma2(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
__device__ __forceinline__ uint32_t tc_hmul2(uint32_t a, uint32_t b) { uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ void tc_nibs(uint32_t w, uint32_t (&n)[4]) {
  const uint32_t w8 = w >> 8;
  n[0] = tc_hadd2((w & 0x000F000Fu) | 0x64006400u, 0xE400E400u); n[1] = tc_hadd2((w & 0x00F000F0u) | 0x54005400u, 0xD400D400u);
  n[2] = tc_hadd2((w8 & 0x000F000Fu) | 0x64006400u, 0xE400E400u); n[3] = tc_hadd2((w8 & 0x00F000F0u) | 0x54005400u, 0xD400D400u);
}
// eight consecutive fp16 (v.x = (e0, e1) .. v.w = (e6, e7)) <-> registers o[x] = (e_x, e_{x+4})
__device__ __forceinline__ void tc_row_to_pairs(const uint4& v, uint32_t (&o)[4]) {
  o[0] = __byte_perm(v.x, v.z, 0x5410); o[1] = __byte_perm(v.x, v.z, 0x7632); o[2] = __byte_perm(v.y, v.w, 0x5410); o[3] = __byte_perm(v.y, v.w, 0x7632);
}
__device__ __forceinline__ uint4 tc_pairs_to_row(const uint32_t (&r)[4]) {
  return make_uint4(__byte_perm(r[0], r[1], 0x5410), __byte_perm(r[2], r[3], 0x5410), __byte_perm(r[0], r[1], 0x7632), __byte_perm(r[2], r[3], 0x7632));
}
// Global loads as ordered asm statements: the compiler keeps them where they are written, ahead of the arithmetic.
__device__ __forceinline__ uint32_t tc_ldg32(const void* p) { uint32_t v; asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p)); return v; }
__device__ __forceinline__ uint32_t tc_ldg16(const void* p) { unsigned short v; asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p)); return v; }
__device__ __forceinline__ uint4 tc_ldg128(const void* p) {
  uint4 v; asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v;
}
__device__ __forceinline__ void tc_prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void tc_sts128(uint32_t a, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// bf16 queries of one CTA (128 operand rows = (token, head) pairs) as fp16 rows in the swizzled Q blocks; rows without a
// query are zero.  Thread t of nt; eight 16-byte loads are in flight per thread before the first one is converted.
template <int HD>
__device__ __forceinline__ void tc_stage_q_bf16(uint32_t sq, int q_block, const uint16_t* q16, int tok0, int G, int TOK, int M, int nh, int head0,
                                                int t, int nt) {
  constexpr int NW = HD / 8, B = 8;
  for (int base = t; base < 128 * NW; base += B * nt) {
    uint4 u[B];
    #pragma unroll
    for (int b = 0; b < B; ++b) {
      const int it = base + b * nt, row = it / NW, w = it % NW, tk = tok0 + row / G;
      u[b] = make_uint4(0u, 0u, 0u, 0u);
      if (it < 128 * NW && row < TOK * G && tk < M) u[b] = tc_ldg128(q16 + ((size_t)tk * nh + head0 + row % G) * HD + 8 * w);
    }
    #pragma unroll
    for (int b = 0; b < B; ++b) {
      const int it = base + b * nt, row = it / NW, w = it % NW;
      if (it >= 128 * NW) break;
      const uint32_t uu[4] = {u[b].x, u[b].y, u[b].z, u[b].w};
      uint32_t o4[4];
      #pragma unroll
      for (int e = 0; e < 4; ++e) o4[e] = tc_pack(__uint_as_float(uu[e] << 16), __uint_as_float(uu[e] & 0xffff0000u));
      tc_sts128(sq + (w >> 3) * q_block + row * 128 + (((w & 7) ^ (row & 7)) << 4), make_uint4(o4[0], o4[1], o4[2], o4[3]));
    }
  }
}
// ------------------------------------------------------------------------------------------------ attention kernel
constexpr int TC_SW = 8;                                   // softmax warps: warp w owns rows 32*(w%4).., key columns 64*(w/4)..
constexpr int TC_KW = 4, TC_VW = 3, TC_CW = TC_KW + TC_VW;  // converter warps of the fused forms: K half tiles, V half tiles
// + producer warp, + MMA issuer warp; the fused form adds the converter warps and fills up to four warpgroups (16 warps x 128
// registers at launch), so that setmaxnreg can move registers from the softmax warps (120 each) and the V converters (112) to the K converters (160)
constexpr int tc_threads(bool fused) { return fused ? 512 : (TC_SW + 2) * 32; }
static_assert(TC_SW == 8 && TC_SW + 1 + TC_CW <= 16, "warpgroups 0-1 = softmax warps, warpgroups 2-3 = Q copy + MMA issuer (one warp), converters");
constexpr int TC_THREADS = tc_threads(false);

// A pair of CTAs (a cluster of two, tcgen05 cta_group::2) works on 256 query rows with MMAs of M = 256: each CTA keeps
// its 128 rows of S, P and O in its own tensor memory, its Q rows in shared memory, and stages HALF of every K tile
// (64 of the 128 keys) and half of every V tile (HD/2 of the channels); the tensor cores of both SMs read both halves.
// Why these shapes: one thread issues every MMA of the pair and an MMA costs it 50-65 cycles whatever its size, and
// M128 N64 steps run at two thirds of the rate of N128 steps, so S tiles are 128 keys wide (N = 128) -- which fills
// tensor memory (2 x 128 S columns + 256 O columns) and sends Q to shared memory; an SM takes in only 40-50 bytes per
// clock from L2, so each SM stages half a tile.
template <int HD> struct TcLay {
  static constexpr int KBLK = HD / 64;                     // 64-channel (128-byte) operand blocks
  static constexpr int Q_BLOCK = 128 * 128;                // 128 rows x 128 bytes
  static constexpr int Q_BYTES = KBLK * Q_BLOCK;           // [block][row][128 B]
  static constexpr int K_BLOCK = (TC_BN / 2) * 128;        // this CTA's 64 keys x 128 bytes
  static constexpr int K_HALF = KBLK * K_BLOCK;            // [block][key][128 B]
  static constexpr int V_BLOCK = TC_BN * 128;              // 128 keys x 128 bytes
  static constexpr int V_HALF = (KBLK / 2) * V_BLOCK;      // this CTA's HD/2 channels: [block][key][128 B]
  static constexpr int NK = 3, NV = 2;                     // ring depths
  static constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = OFF_K + NK * K_HALF, OFF_BAR = OFF_V + NV * V_HALF;
  static constexpr int OFF_XCH = OFF_BAR + 256;            // float val[2 tile parities][2 column halves][128 rows], u16 seq[2][128]
  static constexpr int TOTAL = OFF_XCH + 2 * 2 * 128 * 4 + 2 * 128 * 2;
  // TMEM columns (32-bit): two S buffers of 128 fp32 columns and O.  P (fp16 pairs) is written over the S columns its
  // thread has read: 32 columns at +0 for keys 0-63, 32 at +64 for keys 64-127.
  static constexpr uint32_t TM_S0 = 0, TM_S1 = TC_BN, TM_O = 2 * TC_BN;
  static constexpr int TM_COLS = 512;
  static_assert(TOTAL <= 227 * 1024, "shared memory budget");
  static_assert(2 * TC_BN + HD <= 512, "TMEM columns");
  static_assert(K_HALF % 1024 == 0 && V_HALF % 1024 == 0 && Q_BYTES % 1024 == 0, "swizzle atoms");
};

struct TcP {
  const int* d_pos; int M, splits, G, nh, max_ctx, ks_rows; float qscale;
  float* pm; float* pl; float* pacc;
  uint16_t* o16; const uint16_t* bv;                       // splits == 1 and o16 set: store the finished rows, no partials
  yskn_kv_layer kv; const float* rope; int rd;             // the fused form reads the packed cache itself
  const uint16_t* q16; int bf16;                           // fused form with bf16 activations: the converter warps also stage Q (as fp16)
  const int8_t* k8; const int8_t* v8; const float* ks8; const float* vs8;     // FORM 2: INT8 rows and their scales
};

// FORM 0: K and V tiles come by TMA from the fp16 workspace that kv4_tc_prep_kernel wrote.
// FORM 3: FORM 0 for bf16 activations, a form of its own so that the fp16 kernel carries none of its code.
// FORM 1: no workspace.  Seven converter warps per CTA read the packed cache rows of each tile straight from global memory
// (the int4 words, their scale and zero rows, the rope table rows of the rotary channels; for edge tiles also the fp16
// shadow rows), convert them and store the fp16 operand rows into the same 128-byte-swizzled stages the TMA would have
// filled; "full" then counts the converter warps of both CTAs instead of bytes.  A pass reads 1/4 of the bytes of the
// workspace form and needs no launch in front.
// FORM 2: the converting form over Family-B INT8 rows (k8, v8 [Hkv][max_ctx][256] with one fp32 scale per row; the
// reference's q35_attention_kernel<KV8> semantics, src/q35_kernels.cu:1176-1281, for many rows): every key is an INT8 row,
// nothing is rotated at read time and there is no shadow, so every tile has one K item and the tiles that hold the new
// rows are masked causally.  A byte is read as the fp16 number 1152 + b by one byte permute, the offset leaves by an exact
// subtraction, and the row's scale (rounded to fp16) is multiplied in.
template <int HD, int FORM>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(tc_threads(FORM == 1 || FORM == 2), 1)
kv4_tc_attn_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapKd,
                   const __grid_constant__ CUtensorMap mapVd, const __grid_constant__ CUtensorMap mapKs, const TcP P) {
  using L = TcLay<HD>;
  constexpr bool FUSED = FORM == 1 || FORM == 2, I8 = FORM == 2;
  const bool act_bf16 = FUSED ? P.bf16 != 0 : FORM == 3;              // a compile-time constant in the workspace forms
  static_assert(!I8 || HD == 256, "INT8 rows have 256 channels");
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sb = s_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                           // 0 = leader: issues the MMAs, owns the "full"/"ready" barriers
  // barriers (8 bytes each), same offsets in both CTAs:
  //   leader's copy only: kfull[NK] vfull[NV] pready[2] qfull     each CTA's copy: kempty[NK] vempty[NV] sready[2] pvdone[2]
  const uint32_t B0 = sb + L::OFF_BAR;
  const uint32_t b_kfull = B0, b_kempty = B0 + 32, b_vfull = B0 + 64, b_vempty = B0 + 96, b_sready = B0 + 128, b_pready = B0 + 144,
                 b_pvdone = B0 + 160, b_q = B0 + 176;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_BAR + 184);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::OFF_BAR + 188);
  const uint32_t lead_kfull = leader_addr(b_kfull), lead_vfull = leader_addr(b_vfull), lead_pready = leader_addr(b_pready), lead_q = leader_addr(b_q);

  if (sb & 1023u) { if (threadIdx.x == 0) atomicExch(&g_tc_status, 3); return; }   // same in both CTAs: nobody is left waiting
  if (threadIdx.x == 0) {
    for (int i = 0; i < L::NK; ++i) { bar_init(b_kfull + 8 * i, FUSED ? 2 * TC_KW : 1); bar_init(b_kempty + 8 * i, 1); }
    for (int i = 0; i < L::NV; ++i) { bar_init(b_vfull + 8 * i, FUSED ? 2 * TC_VW : 1); bar_init(b_vempty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { bar_init(b_sready + 8 * i, 1); bar_init(b_pready + 8 * i, 2 * TC_SW); bar_init(b_pvdone + 8 * i, 1); }
    bar_init(b_q, act_bf16 ? (FUSED ? 2 * TC_KW : 2 * TC_SW) : 1);   // bf16 queries are staged by warps, not by TMA
    *s_abort = 0;
    for (int i = 0; i < 128; ++i) reinterpret_cast<volatile uint32_t*>(smem + L::OFF_XCH + 2 * 2 * 128 * 4)[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == TC_SW + 1) {                                           // the same warp of both CTAs allocates for the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sb + L::OFF_BAR + 184), "n"(L::TM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                                // both CTAs' barriers exist before anyone signals the other
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // Programmatic dependent launch: the grid may be scheduled while its predecessor in the stream drains, and everything above
  // (barriers, tensor memory, the cluster handshake) touches nothing the predecessor wrote.  From here on the position, the
  // queries and the cache (or the workspace the prep kernel fills) are read; the merge kernel that follows may be scheduled
  // early in turn and waits for this grid before it reads the partials.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- geometry: uniform over the pair except tok0
  const int G = P.G, TOK = 128 / G, kvh = blockIdx.z, S = P.splits, split = blockIdx.y;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;               // heaviest query tiles first; gridDim.x is even
  const int tok0 = qt * TOK;                                         // this CTA's first token
  const int tokA = (qt & ~1) * TOK;                                  // the pair's first token (always < M)
  const int pos0 = *P.d_pos;
  const int pmax = pos0 + min(tokA + 2 * TOK, P.M) - 1;              // last key any row of the pair sees
  const int nt_all = pmax / TC_BN + 1;
  const int per = (pos0 / TC_BN + 1 + S - 1) / S;                    // split width in tiles: a function of *d_pos and S only
  const int j0 = min(split * per, nt_all), j1 = split == S - 1 ? nt_all : min((split + 1) * per, nt_all);
  const int n = j1 - j0;
  const int jb = (pos0 + tokA) / TC_BN;                              // tiles below jb hold only groups before every row's own group
  const int nbulk = max(0, min(n, jb - j0));
  const int npipe = I8 ? n : nbulk;                                  // tiles with a single K item, run through the two S buffers in turn
  const int ks0 = (pos0 / TC_BN) * TC_BN;


  auto role_producer = [&]() {
    // ======================================================================= TMA producer (one per CTA)
    // Q once, then two rings: K halves are free again as soon as their S MMAs are done, V halves only after P.V.
    // Every copy reports to the leader's "full" barrier; the leader posts the byte count of both CTAs' parts.
    if (lane == 0 && n > 0 && !(FUSED && act_bf16)) {
      if (!act_bf16) {                                                 // bf16 queries are converted and written by warps instead
        if (rank == 0) bar_expect_tx(b_q, 2 * L::KBLK * G * TOK * 128);
        for (int kb = 0; kb < L::KBLK; ++kb) tma_load_4d_pair(sb + L::OFF_Q + kb * L::Q_BLOCK, &mapQ, 64 * kb, 0, kvh, tok0, lead_q);
      }
      int kit = 0; bool ok = true;
      for (int i = 0; i < n && ok && !FUSED; ++i) {
        const int j = j0 + i;
        for (int half = 0; half < (i >= nbulk ? 2 : 1) && ok; ++half, ++kit) {      // Kd; edge tiles: then Ks
          const int st = kit % L::NK;
          if (kit >= L::NK && !bar_wait(b_kempty + 8 * st, (kit / L::NK - 1) & 1)) { atomicExch(&g_tc_status, 6); *s_abort = 1; ok = false; break; }
          if (*s_abort) { ok = false; break; }
          if (rank == 0) bar_expect_tx(b_kfull + 8 * st, 2 * L::K_HALF);
          const int row = (half == 0 ? kvh * P.max_ctx + j * TC_BN : kvh * P.ks_rows + j * TC_BN - ks0) + (TC_BN / 2) * (int)rank;
          tma_load_3d_pair(sb + L::OFF_K + st * L::K_HALF, half == 0 ? &mapKd : &mapKs, 0, row, 0, lead_kfull + 8 * st);
        }
        if (!ok) break;
        const int st = i % L::NV;                                    // V of tile i; its buffer was last read by P.V of tile i-NV
        if (i >= L::NV && !bar_wait(b_vempty + 8 * st, (i / L::NV - 1) & 1)) { atomicExch(&g_tc_status, 6); *s_abort = 1; ok = false; break; }
        if (rank == 0) bar_expect_tx(b_vfull + 8 * st, 2 * L::V_HALF);
        tma_load_3d_pair(sb + L::OFF_V + st * L::V_HALF, &mapVd, 0, kvh * P.max_ctx + j * TC_BN, (L::KBLK / 2) * (int)rank, lead_vfull + 8 * st);
      }
    }
  };
  // the converting forms have no K / V copies to issue: the warp that requested Q goes on to issue the MMAs
  constexpr int CONV0 = TC_SW + 1;
  auto role_mma = [&]() {
    // ======================================================================= MMA issuer (one thread of the leader CTA)
    // The tensor pipe runs this thread's MMAs in issue order, so S of tile i+2, issued after P.V of tile i, may
    // overwrite the TMEM buffer that P.V reads P from without a barrier in between.
    if (lane == 0 && n > 0 && rank == 0) {
      constexpr uint32_t ID_S = instr_desc(256, TC_BN, false), ID_PV = instr_desc(256, HD, true);
      bool ok = true;
      auto fail = [&]() { atomicExch(&g_tc_status, 5); *s_abort = 1; ok = false; };
      const uint64_t qdesc0 = smem_desc(sb + L::OFF_Q, 16, 1024), kdesc0 = smem_desc(sb + L::OFF_K, 16, 1024),
                     vdesc0 = smem_desc(sb + L::OFF_V, L::V_BLOCK, 1024);
      auto issue_s = [&](int item, int buf) {                        // S[buf] = Q . K(item)^T
        const int st = item % L::NK;
        if (!bar_wait(b_kfull + 8 * st, (item / L::NK) & 1)) { fail(); return; }
        tc_fence_after();
        const uint64_t kd = kdesc0 + (uint64_t)((st * L::K_HALF) >> 4);
        // The workspace form (prefill) lives on this thread's issue rate: everything unrolled.  The converting forms keep
        // their code inside the instruction cache: one expansion per lambda and a rolled loop, whose iteration is kept to a
        // handful of instructions by stepping the two descriptors (an MMA cost this thread ~220 cycles with the
        // descriptors recomputed in every iteration, and the thread then paced the whole kernel).
        if constexpr (FUSED) {
          const uint32_t dcol = tmem + (buf ? L::TM_S1 : L::TM_S0);
          uint64_t qd = qdesc0, kdd = kd;
          #pragma unroll 1
          for (int t = 0; t < 4 * L::KBLK; ++t) {
            umma2_ss(dcol, qd, kdd, ID_S, t ? 1u : 0u);
            const bool last = (t & 3) == 3;                          // next 64-channel block: the next operand block of Q and of K
            qd += last ? (uint64_t)((L::Q_BLOCK - 96) >> 4) : 2ull;
            kdd += last ? (uint64_t)((L::K_BLOCK - 96) >> 4) : 2ull;
          }
        } else {
        #pragma unroll
        for (int kb = 0; kb < L::KBLK; ++kb)
          #pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma2_ss(tmem + (buf ? L::TM_S1 : L::TM_S0), qdesc0 + (uint64_t)((kb * L::Q_BLOCK + ks * 32) >> 4),
                     kd + (uint64_t)((kb * L::K_BLOCK + ks * 32) >> 4), ID_S, (kb | ks) ? 1u : 0u);
        }
        umma2_commit(b_sready + 8 * buf);
        umma2_commit(b_kempty + 8 * st);                             // the K halves may be overwritten once these MMAs are done
      };
      auto issue_pv = [&](int tile_i, int buf) {                     // O (+)= P . V(tile_i), P from TMEM (over S[buf])
        const int st = tile_i % L::NV;
        if (!bar_wait(b_pready + 8 * (tile_i & 1), (tile_i >> 1) & 1)) { fail(); return; }
        if (!bar_wait(b_vfull + 8 * st, (tile_i / L::NV) & 1)) { fail(); return; }
        tc_fence_after();
        const uint64_t vd = vdesc0 + (uint64_t)((st * L::V_HALF) >> 4);
        const uint32_t pcol = tmem + (buf ? L::TM_S1 : L::TM_S0);
        if constexpr (FUSED) {
          uint32_t pa = pcol; uint64_t vdd = vd;
          #pragma unroll 1
          for (int ks = 0; ks < TC_BN / 16; ++ks) {                  // P columns: keys 0-63 at +0.., keys 64-127 at +64..
            umma2_ts(tmem + L::TM_O, pa, vdd, ID_PV, (tile_i | ks) ? 1u : 0u);
            pa += ks == 3 ? 64u - 24u : 8u; vdd += 128ull;
          }
        } else {
        #pragma unroll
        for (int ks = 0; ks < TC_BN / 16; ++ks)                      // P columns: keys 0-63 at +0.., keys 64-127 at +64..
          umma2_ts(tmem + L::TM_O, pcol + 64 * (ks >> 2) + 8 * (ks & 3), vd + (uint64_t)((ks * 2048) >> 4), ID_PV, (tile_i | ks) ? 1u : 0u);
        }
        umma2_commit(b_pvdone + 8 * (tile_i & 1));                   // O may be rescaled
        umma2_commit(b_vempty + 8 * st);                             // the V halves may be overwritten
      };
      if (!bar_wait(b_q, 0)) fail();
      tc_fence_after();
      // Bulk tiles: S(0), S(1), then P.V(i), S(i+2), ...: S of the next two tiles is done or in flight while the softmax
      // warps work on this one.  Edge tiles: S from the int4 keys, S from the shadow keys, then P.V.
      if constexpr (FUSED) {                                         // the same order as one loop with a single expansion of each lambda
        int s_next = 0, pv_next = 0;
        const int s_total = npipe + 2 * (n - npipe);
        while (ok && pv_next < n) {
          bool do_s = false; int buf = 0;
          if (s_next < npipe) { do_s = s_next < pv_next + 2; buf = s_next & 1; }
          else if (pv_next >= npipe) { const int e = s_next - (npipe + 2 * (pv_next - npipe)); do_s = s_next < s_total && e < 2; buf = e; }
          if (do_s) { issue_s(s_next, buf); ++s_next; }
          else { issue_pv(pv_next, pv_next < npipe ? (pv_next & 1) : 0); ++pv_next; }
        }
      } else {
        if (ok && npipe > 0) issue_s(0, 0);
        if (ok && npipe > 1) issue_s(1, 1);
        for (int i = 0; i < npipe && ok; ++i) {
          issue_pv(i, i & 1);
          if (ok && i + 2 < npipe) issue_s(i + 2, i & 1);
        }
        for (int i = npipe, kit = npipe; i < n && ok; ++i, kit += 2) {
          issue_s(kit, 0); if (!ok) break;
          issue_s(kit + 1, 1); if (!ok) break;
          issue_pv(i, 0);
        }
      }
    }
  };
  auto role_conv = [&](const bool is_k) {
    // ======================================================================= converter warps (fused form)
    // Four warps convert the K half tiles, three the V half tiles, each role with its own ring, so neither waits for the
    // other.  Every global load of a phase is issued before the first dependent instruction (ordered asm statements) and
    // the loads of the next tile are in flight while the current one is converted: a thread pays the memory latency once.
    constexpr int NKT = TC_KW * 32, NVT = TC_VW * 32, NWD = HD / 8, NWV = HD / 16;   // threads per role; packed words per K row; per V row in this CTA's channel half
    // warps 9-11 (warpgroup 2) convert V, warps 12-15 (warpgroup 3) convert K: ct = 0 .. NKT-1 for K, NKT .. NKT+NVT-1 for V
    const int ct = is_k ? (int)threadIdx.x - (TC_SW + 4) * 32 : (int)threadIdx.x - CONV0 * 32 + TC_KW * 32;
    const int end = pos0 + P.M;                                      // tokens [0, end) exist
    const size_t row0 = (size_t)kvh * P.max_ctx, grp0 = (size_t)kvh * (P.max_ctx / 32);
    bool ok = true;
    auto publish = [&](uint32_t lead_bar) {                          // this warp's part of the stage is written
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive_cluster(lead_bar);
    };
    auto stage_wait = [&](uint32_t bar_empty, int item, int depth) { // the stage's previous contents have been consumed
      if (item >= depth && !bar_wait(bar_empty, (item / depth - 1) & 1)) { atomicExch(&g_tc_status, 6); *s_abort = 1; ok = false; }
      if (*s_abort) ok = false;
    };

    // INT8 rows: item = (key, 16-byte chunk = 16 channels) -> two 16-byte chunks of fp16; cur holds this tile's items, each
    // next-tile item is requested right before the same item of this tile is converted
    struct I8In { uint4 w; uint32_t s; };
    auto i8_convert = [&](const I8In& I, bool live, uint4& lo, uint4& hi) {      // channels 0-7 and 8-15 of the chunk
      // the row's scale as a sum of two fp16 numbers: b * scale = fma(b, hi, b * lo) is then rounded once, without the
      // per-row relative error of up to 2^-11 that a scale rounded to fp16 alone would put on all 256 channels of the row
      const float sf = __uint_as_float(I.s), sh = __half2float(__float2half_rn(sf));
      const uint32_t s_hi = tc_pack(sh, sh), s_lo = tc_pack(sf - sh, sf - sh);
      const uint32_t ww[4] = {I.w.x ^ 0x80808080u, I.w.y ^ 0x80808080u, I.w.z ^ 0x80808080u, I.w.w ^ 0x80808080u};
      uint32_t r[8];
      #pragma unroll
      for (int e = 0; e < 4; ++e) {                                  // byte b -> 0x64bb = 1152 + b (b two's complement, top bit flipped)
        const uint32_t n0 = tc_hadd2(__byte_perm(ww[e], 0x64646464u, 0x4140), 0xE480E480u), n1 = tc_hadd2(__byte_perm(ww[e], 0x64646464u, 0x4342), 0xE480E480u);
        r[2 * e] = tc_hfma2(n0, s_hi, tc_hmul2(n0, s_lo));
        r[2 * e + 1] = tc_hfma2(n1, s_hi, tc_hmul2(n1, s_lo));
      }
      lo = live ? make_uint4(r[0], r[1], r[2], r[3]) : make_uint4(0u, 0u, 0u, 0u);
      hi = live ? make_uint4(r[4], r[5], r[6], r[7]) : make_uint4(0u, 0u, 0u, 0u);
    };
    if (n > 0 && is_k) {
      // ------------------------------------------------------------------- K role
      if constexpr (I8) {
        constexpr int NKI = ((TC_BN / 2) * 16 + NKT - 1) / NKT;      // 64 keys x 16 chunks over the K threads
        if (P.bf16) {
          tc_stage_q_bf16<HD>(sb + L::OFF_Q, L::Q_BLOCK, P.q16, tok0, G, TOK, P.M, P.nh, kvh * G, ct, NKT);
          publish(lead_q);
        }
        // The items of all tiles form one stream (NKI per tile); two are in flight ahead of the one being converted.  Rolled
        // loops: the kernel's code has to stay inside the instruction cache.
        auto k8_load = [&](int q, I8In& I) {                         // q-th item of this thread's stream
          const int it = ct + NKT * (q % NKI), t = (j0 + q / NKI) * TC_BN + (TC_BN / 2) * (int)rank + (it >> 4);
          if (q < n * NKI && it < (TC_BN / 2) * 16 && t < P.max_ctx) {
            I.w = tc_ldg128(P.k8 + (row0 + t) * HD + 16 * (it & 15));
            I.s = tc_ldg32(P.ks8 + row0 + t);
          }
        };
        auto k8_prefetch = [&](int tk) {                             // L2 prefetch of a half tile: 64 rows of 256 bytes, two lines each
          if (tk >= P.max_ctx) return;
          tc_prefetch_l2(P.k8 + (row0 + tk + (ct >> 1)) * HD + 128 * (ct & 1));
          if (ct < 2) tc_prefetch_l2(P.ks8 + row0 + tk + 32 * ct);
        };
        I8In cur, n1, n2;
        k8_load(0, cur); k8_load(1, n1);
        if (n > 1) k8_prefetch((j0 + 1) * TC_BN + (TC_BN / 2) * (int)rank);
        int q = 0;
        for (int i = 0; i < n && ok; ++i) {
          const int tk0 = (j0 + i) * TC_BN + (TC_BN / 2) * (int)rank, st = i % L::NK;
          const uint32_t sk = sb + L::OFF_K + st * L::K_HALF;
          if (i + 2 < n) k8_prefetch(tk0 + 2 * TC_BN);
          stage_wait(b_kempty + 8 * st, i, L::NK);
          if (!ok) break;
          #pragma unroll 1
          for (int u = 0; u < NKI; ++u, ++q) {
            k8_load(q + 2, n2);
            const int it = ct + NKT * u, k = it >> 4, c = it & 15;
            if (it < (TC_BN / 2) * 16) {
              uint4 lo, hi;
              i8_convert(cur, tk0 + k < P.max_ctx, lo, hi);
              tc_sts128(sk + (c >> 2) * L::K_BLOCK + k * 128 + ((((2 * c) & 7) ^ (k & 7)) << 4), lo);
              tc_sts128(sk + (c >> 2) * L::K_BLOCK + k * 128 + ((((2 * c + 1) & 7) ^ (k & 7)) << 4), hi);
            }
            cur = n1; n1 = n2;
          }
          publish(lead_kfull + 8 * st);
        }
      } else {
      const int nrw = P.rd / 8, nrp = nrw / 2, half = P.rd / 2;      // rotary words; word pairs (w, w + nrp), a power of two; frequencies
      const int lp = nrp > 0 ? __ffs(nrp) - 1 : 0, nrot = (TC_BN / 2) * nrp;
      const int npl = NWD - nrw;                                     // plain word columns
      const uint32_t* kq32 = reinterpret_cast<const uint32_t*>(P.kv.kq);
      auto k_addr = [&](uint32_t sk, int w, int k) { return sk + (w >> 3) * L::K_BLOCK + k * 128 + (((w & 7) ^ (k & 7)) << 4); };
      // Plain items: (word column, octet of keys); item x of a tile = column nrw + x % npl, keys 8 (x / npl) .. +7, so that
      // consecutive lanes take consecutive columns of one octet.  A thread's items of all tiles form one stream (NPI per tile).
      constexpr int NPI = (NWD * 8 + NKT - 1) / NKT;
      const int np1 = npl > 0 ? npl : 1, nplain = npl * 8;
      struct PlainIn { uint32_t w[8]; uint4 s, z; };
      auto plain_load = [&](int q, PlainIn& I) {                     // q-th item of the stream
        const int x = ct + NKT * (q % NPI), tk = (j0 + q / NPI) * TC_BN + (TC_BN / 2) * (int)rank;
        if (q < n * NPI && x < nplain && tk < P.max_ctx) {
          const int col = nrw + x % np1, key = 8 * (x / np1);
          const uint32_t* src = kq32 + (row0 + tk + key) * (HD / 8) + col;
          #pragma unroll
          for (int e = 0; e < 8; ++e) I.w[e] = tc_ldg32(src + e * (HD / 8));
          const size_t gb = (grp0 + (tk + key) / 32) * HD + 8 * col;
          I.s = tc_ldg128(P.kv.kscale + gb); I.z = tc_ldg128(P.kv.kzero + gb);
        }
      };
      auto plain_store = [&](int u, uint32_t sk, const PlainIn& I) {
        const int x = ct + NKT * u;
        if (x >= nplain) return;
        const int col = nrw + x % np1, key = 8 * (x / np1);
        uint32_t sc[4], zz[4];
        tc_row_to_pairs(I.s, sc); tc_row_to_pairs(I.z, zz);
        const uint32_t base = sk + (col >> 3) * L::K_BLOCK + key * 128;      // key is a multiple of 8: (key + e) & 7 = e
        const uint32_t cx = (uint32_t)(col & 7);
        #pragma unroll
        for (int h = 0; h < 8; h += 4) {                               // four words converted, then four stores: independent chains interleave
          uint4 out[4];
          #pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t nb[4], r[4];
            tc_nibs(I.w[h + e], nb);
            #pragma unroll
            for (int x2 = 0; x2 < 4; ++x2) r[x2] = tc_hfma2(nb[x2], sc[x2], zz[x2]);
            out[e] = tc_pairs_to_row(r);
          }
          #pragma unroll
          for (int e = 0; e < 4; ++e) tc_sts128(base + (h + e) * 128 + ((cx ^ (uint32_t)(h + e)) << 4), out[e]);
        }
      };
      struct RotIn { uint32_t wa, wb; uint4 sa, za, sb, zb; uint4 r[4]; };   // shadow items keep their two fp16 rows in sa, za
      // one rotary item = key k, word pair (p, p + nrp): 8 + 8 channels (c, c + rd/2) and their 8 (cos, sin) pairs
      auto rot_load = [&](int it, int tk0, bool shadow, RotIn& R) {
        const int k = it >> lp, p = it & (nrp - 1), q = p + nrp, t = tk0 + k;
        if (shadow) {
          R.sa = tc_ldg128(P.kv.kshadow + (row0 + t) * HD + 8 * p); R.za = tc_ldg128(P.kv.kshadow + (row0 + t) * HD + 8 * q);
        } else {
          const uint32_t* rowp = kq32 + (row0 + t) * (HD / 8);
          R.wa = tc_ldg32(rowp + p); R.wb = tc_ldg32(rowp + q);
          const size_t gb = (grp0 + t / 32) * HD;
          R.sa = tc_ldg128(P.kv.kscale + gb + 8 * p); R.za = tc_ldg128(P.kv.kzero + gb + 8 * p);
          R.sb = tc_ldg128(P.kv.kscale + gb + 8 * q); R.zb = tc_ldg128(P.kv.kzero + gb + 8 * q);
        }
        const float* rp = P.rope + ((size_t)t * half + 8 * p) * 2;
        #pragma unroll
        for (int e = 0; e < 4; ++e) R.r[e] = tc_ldg128(rp + 4 * e);
      };
      // fp16 pairs throughout: registers x hold channels (x, x + 4) of the word, like the nibble reads
      auto rot_store = [&](int it, int tk0, bool shadow, uint32_t sk, const RotIn& R) {
        const int k = it >> lp, p = it & (nrp - 1), q = p + nrp, t = tk0 + k;
        uint32_t a[4], b[4];
        if (shadow) {
          tc_row_to_pairs(R.sa, a); tc_row_to_pairs(R.za, b);
          if (t >= end) { a[0] = a[1] = a[2] = a[3] = 0u; b[0] = b[1] = b[2] = b[3] = 0u; }
        } else {
          uint32_t na[4], nb[4], sa[4], za[4], sb4[4], zb[4];
          tc_nibs(R.wa, na); tc_nibs(R.wb, nb);
          tc_row_to_pairs(R.sa, sa); tc_row_to_pairs(R.za, za); tc_row_to_pairs(R.sb, sb4); tc_row_to_pairs(R.zb, zb);
          #pragma unroll
          for (int x = 0; x < 4; ++x) { a[x] = tc_hfma2(na[x], sa[x], za[x]); b[x] = tc_hfma2(nb[x], sb4[x], zb[x]); }
        }
        // R.r[e/2] = (cos e, sin e, cos e+1, sin e+1) as fp32 bits; C[x] = (cos x, cos x+4), S[x] = (sin x, sin x+4)
        const uint32_t C[4] = {tc_pack(__uint_as_float(R.r[0].x), __uint_as_float(R.r[2].x)), tc_pack(__uint_as_float(R.r[0].z), __uint_as_float(R.r[2].z)),
                               tc_pack(__uint_as_float(R.r[1].x), __uint_as_float(R.r[3].x)), tc_pack(__uint_as_float(R.r[1].z), __uint_as_float(R.r[3].z))};
        const uint32_t S[4] = {tc_pack(__uint_as_float(R.r[0].y), __uint_as_float(R.r[2].y)), tc_pack(__uint_as_float(R.r[0].w), __uint_as_float(R.r[2].w)),
                               tc_pack(__uint_as_float(R.r[1].y), __uint_as_float(R.r[3].y)), tc_pack(__uint_as_float(R.r[1].w), __uint_as_float(R.r[3].w))};
        uint32_t lo[4], hi[4];
        #pragma unroll
        for (int x = 0; x < 4; ++x) {
          lo[x] = tc_hfma2(a[x], C[x], tc_hmul2(b[x], S[x]) ^ 0x80008000u);      // a cos - b sin
          hi[x] = tc_hfma2(a[x], S[x], tc_hmul2(b[x], C[x]));                    // a sin + b cos
        }
        tc_sts128(k_addr(sk, p, k), tc_pairs_to_row(lo));
        tc_sts128(k_addr(sk, q, k), tc_pairs_to_row(hi));
      };
      auto zero_k = [&](uint32_t sk) {                               // a half tile past max_ctx: nothing to read
        for (int it = ct; it < (TC_BN / 2) * NWD; it += NKT) tc_sts128(k_addr(sk, it % NWD, it / NWD), make_uint4(0u, 0u, 0u, 0u));
      };
      if (P.bf16) {
        // bf16 activations: this CTA's query rows (token, head) as fp16 operand rows; rows without a query are zero
        tc_stage_q_bf16<HD>(sb + L::OFF_Q, L::Q_BLOCK, P.q16, tok0, G, TOK, P.M, P.nh, kvh * G, ct, NKT);
        publish(lead_q);
      }
      // Rotary items in the compact mapping (rotary width of at most 64 channels): a thread owns one word pair (p, p + nrp) of
      // one 32-key group and up to two keys of it, so the group's scale / zero chunks are loaded once per tile; its items of
      // all tiles form one stream (RCI per tile).  Wider rotary parts take the items one after the other (rot_load / rot_store).
      const bool compact = nrp >= 1 && nrp <= 4;
      constexpr int RCI = 2;                                         // keys per thread: 32 / tpc <= 2 with 128 K threads
      const int tpc = compact ? NKT / (2 * nrp) : 1;                 // threads per (pair, group); keys c and c + tpc of the group
      const int cp = ct & (nrp - 1), cg = compact ? (ct >> lp) & 1 : 0, cc = compact ? ct / (2 * nrp) : 0;
      struct RotS { uint4 sa, za, sb, zb; };                         // the group's scale / zero chunks of the two words
      struct RotI { uint32_t wa, wb; uint4 r[4]; };                  // one key: the two words and the 8 (cos, sin) pairs
      auto rots_load = [&](int tk0, RotS& R) {
        const size_t gb = (grp0 + tk0 / 32 + cg) * HD;
        R.sa = tc_ldg128(P.kv.kscale + gb + 8 * cp); R.za = tc_ldg128(P.kv.kzero + gb + 8 * cp);
        R.sb = tc_ldg128(P.kv.kscale + gb + 8 * (cp + nrp)); R.zb = tc_ldg128(P.kv.kzero + gb + 8 * (cp + nrp));
      };
      auto roti_load = [&](int q, RotI& R) {                         // q-th item of the stream
        const int kk = cc + tpc * (q % RCI), tk = (j0 + q / RCI) * TC_BN + (TC_BN / 2) * (int)rank;
        if (q < n * RCI && kk < 32 && tk < P.max_ctx) {
          const int t = tk + 32 * cg + kk;
          const uint32_t* rowp = kq32 + (row0 + t) * (HD / 8);
          R.wa = tc_ldg32(rowp + cp); R.wb = tc_ldg32(rowp + cp + nrp);
          const float* rp = P.rope + ((size_t)t * half + 8 * cp) * 2;
          #pragma unroll
          for (int e = 0; e < 4; ++e) R.r[e] = tc_ldg128(rp + 4 * e);
        }
      };
      auto roti_store = [&](int u, uint32_t sk, const RotS& Sc, const RotI& R) {
        const int kk = cc + tpc * u;
        if (kk >= 32) return;
        const int p = cp, q = cp + nrp, k = 32 * cg + kk;
        uint32_t sa[4], za[4], sb4[4], zb[4], na[4], nb[4], a[4], b[4], lo[4], hi[4];
        tc_row_to_pairs(Sc.sa, sa); tc_row_to_pairs(Sc.za, za); tc_row_to_pairs(Sc.sb, sb4); tc_row_to_pairs(Sc.zb, zb);
        tc_nibs(R.wa, na); tc_nibs(R.wb, nb);
        #pragma unroll
        for (int x = 0; x < 4; ++x) { a[x] = tc_hfma2(na[x], sa[x], za[x]); b[x] = tc_hfma2(nb[x], sb4[x], zb[x]); }
        const uint4* r = R.r;                                        // r[e/2] = (cos e, sin e, cos e+1, sin e+1) as fp32 bits
        const uint32_t C[4] = {tc_pack(__uint_as_float(r[0].x), __uint_as_float(r[2].x)), tc_pack(__uint_as_float(r[0].z), __uint_as_float(r[2].z)),
                               tc_pack(__uint_as_float(r[1].x), __uint_as_float(r[3].x)), tc_pack(__uint_as_float(r[1].z), __uint_as_float(r[3].z))};
        const uint32_t S[4] = {tc_pack(__uint_as_float(r[0].y), __uint_as_float(r[2].y)), tc_pack(__uint_as_float(r[0].w), __uint_as_float(r[2].w)),
                               tc_pack(__uint_as_float(r[1].y), __uint_as_float(r[3].y)), tc_pack(__uint_as_float(r[1].w), __uint_as_float(r[3].w))};
        #pragma unroll
        for (int x = 0; x < 4; ++x) {
          lo[x] = tc_hfma2(a[x], C[x], tc_hmul2(b[x], S[x]) ^ 0x80008000u);      // a cos - b sin
          hi[x] = tc_hfma2(a[x], S[x], tc_hmul2(b[x], C[x]));                    // a sin + b cos
        }
        tc_sts128(k_addr(sk, p, k), tc_pairs_to_row(lo));
        tc_sts128(k_addr(sk, q, k), tc_pairs_to_row(hi));
      };
      PlainIn pc, pn;                                                // plain stream: current item, next item
      RotI rc, rn;                                                   // rotary stream (compact mapping)
      plain_load(0, pc);
      if (compact) roti_load(0, rc);
      int pq = 0, rq = 0, kit = 0;
      // L2 prefetch of a half tile two tiles ahead (64 packed rows, the scale and zero rows of its two groups; one line per
      // thread), so that the register loads a phase ahead find their lines in L2
      auto k_prefetch = [&](int tk) {
        if (tk >= P.max_ctx) return;
        if (ct < TC_BN / 2) tc_prefetch_l2(P.kv.kq + (row0 + tk + ct) * (HD / 2));
        else if (ct < TC_BN / 2 + 4 * (HD / 64)) {
          const int x = ct - TC_BN / 2, arr = x & 1, grp = (x >> 1) & 1, line = x >> 2;      // line < HD/64 (128-byte lines of an HD x fp16 row)
          tc_prefetch_l2((arr ? P.kv.kzero : P.kv.kscale) + (grp0 + tk / 32 + grp) * HD + 64 * line);
        }
      };
      if (n > 1) k_prefetch(j0 * TC_BN + TC_BN + (TC_BN / 2) * (int)rank);
      for (int i = 0; i < n && ok; ++i) {
        const int j = j0 + i;
        const int tk0 = j * TC_BN + (TC_BN / 2) * (int)rank;         // first key of this CTA's half of the K tile
        const bool kin = tk0 < P.max_ctx;                            // max_ctx is a multiple of 64: the half tile is inside or outside as a whole
        if (i + 2 < n) k_prefetch(tk0 + 2 * TC_BN);
        // ---- item 1: the int4 keys.  The converters never idle, so a request must be made a whole phase before its data
        //      is used: each plain item is requested while the one before it is converted (the first of a tile during the
        //      previous tile's last plain item, i.e. a whole rotary phase ahead), each rotary item likewise (the first of a
        //      tile a whole plain phase ahead), the tile's rotary scales before its plain phase.  Rolled loops, one expansion
        //      of each conversion: the kernel's code has to stay inside the instruction cache.
        {
          const int st = kit % L::NK;
          const uint32_t sk = sb + L::OFF_K + st * L::K_HALF;
          RotS RS;
          if (kin && compact) rots_load(tk0, RS);
          stage_wait(b_kempty + 8 * st, kit, L::NK);
          if (!ok) break;
          if (!kin) { zero_k(sk); pq += NPI; rq += RCI; plain_load(pq, pc); if (compact) roti_load(rq, rc); }
          else {
            #pragma unroll 1
            for (int u = 0; u < NPI; ++u, ++pq) {
              plain_load(pq + 1, pn);
              plain_store(u, sk, pc);
              pc = pn;
            }
            if (compact) {
              #pragma unroll 1
              for (int u = 0; u < RCI; ++u, ++rq) {
                roti_load(rq + 1, rn);
                roti_store(u, sk, RS, rc);
                rc = rn;
              }
            } else {
              RotIn R1;
              #pragma unroll 1
              for (int it = ct; it < nrot; it += NKT) { rot_load(it, tk0, false, R1); rot_store(it, tk0, false, sk, R1); }
            }
          }
          publish(lead_kfull + 8 * st);
          ++kit;
        }
        // ---- item 2 (edge tiles): the fp16 shadow keys
        if (i >= nbulk) {
          const int st = kit % L::NK;
          const uint32_t sk = sb + L::OFF_K + st * L::K_HALF;
          stage_wait(b_kempty + 8 * st, kit, L::NK);
          if (!ok) break;
          if (!kin) zero_k(sk);
          else {
            // plain channels: a copy, kept as a small loop (edge tiles are few; the kernel's code must stay inside the
            // instruction cache)
            #pragma unroll 1
            for (int it = ct; it < (TC_BN / 2) * NWD; it += NKT) {
              const int k = it / NWD, w = it % NWD;
              if (w < nrw) continue;
              uint4 x = make_uint4(0u, 0u, 0u, 0u);
              if (tk0 + k < end) x = tc_ldg128(P.kv.kshadow + (row0 + tk0 + k) * HD + 8 * w);
              tc_sts128(k_addr(sk, w, k), x);
            }
            RotIn R1;
            #pragma unroll 1
            for (int it = ct; it < nrot; it += NKT) { rot_load(it, tk0, true, R1); rot_store(it, tk0, true, sk, R1); }
          }
          publish(lead_kfull + 8 * st);
          ++kit;
        }
      }
      }
    } else if (n > 0) {
      // ------------------------------------------------------------------- V role: this CTA's HD/2 channels of all 128 keys of a tile.
      if constexpr (I8) {
        constexpr int NVI8 = (TC_BN * 8 + NVT - 1) / NVT;            // 128 keys x 8 chunks (this CTA's 128 channels) over the V threads
        const int vt = ct - NKT;
        auto v8_load = [&](int q, I8In& I) {                         // q-th item of this thread's stream (NVI8 per tile)
          const int it = vt + NVT * (q % NVI8), t = (j0 + q / NVI8) * TC_BN + (it >> 3);
          if (q < n * NVI8 && it < TC_BN * 8 && t < end) {
            I.w = tc_ldg128(P.v8 + (row0 + t) * HD + 128 * (int)rank + 16 * (it & 7));
            I.s = tc_ldg32(P.vs8 + row0 + t);
          }
        };
        auto v8_prefetch = [&](int j) {                              // L2 prefetch of a tile's 128 half rows (one line each) and scales
          for (int x = vt; x < TC_BN; x += NVT) if (j * TC_BN + x < end) tc_prefetch_l2(P.v8 + (row0 + j * TC_BN + x) * HD + 128 * (int)rank);
          if (vt < 4 && j * TC_BN + 32 * vt < end) tc_prefetch_l2(P.vs8 + row0 + j * TC_BN + 32 * vt);
        };
        I8In cur, n1, n2;
        v8_load(0, cur); v8_load(1, n1);
        if (n > 1) v8_prefetch(j0 + 1);
        int q = 0;
        for (int i = 0; i < n && ok; ++i) {
          const int j = j0 + i, st = i % L::NV;
          const uint32_t sv = sb + L::OFF_V + st * L::V_HALF;
          if (i + 2 < n) v8_prefetch(j + 2);
          stage_wait(b_vempty + 8 * st, i, L::NV);
          if (!ok) break;
          #pragma unroll 1
          for (int u = 0; u < NVI8; ++u, ++q) {
            v8_load(q + 2, n2);
            const int it = vt + NVT * u, k = it >> 3, c = it & 7;
            if (it < TC_BN * 8) {
              uint4 lo, hi;
              i8_convert(cur, j * TC_BN + k < end, lo, hi);          // tokens that do not exist yet read as zero
              tc_sts128(sv + (c >> 2) * L::V_BLOCK + k * 128 + ((((2 * c) & 7) ^ (k & 7)) << 4), lo);
              tc_sts128(sv + (c >> 2) * L::V_BLOCK + k * 128 + ((((2 * c + 1) & 7) ^ (k & 7)) << 4), hi);
            }
            cur = n1; n1 = n2;
          }
          publish(lead_vfull + 8 * st);
        }
      } else {
      // Item = (key, 16-byte part of the key's half row = 32 channels); tokens that do not exist yet read as zero.
      constexpr int PARTS = NWV / 4, NVI = (TC_BN * PARTS + NVT - 1) / NVT;
      const int vt = ct - NKT;
      struct VIn { uint4 w; uint32_t s, z; };
      // The items of all tiles form one stream (tile by tile, NVI items each); two items are in flight ahead of the one being
      // converted.  A rolled loop: the lines are in L2 already (prefetched two tiles ahead), and small code matters more
      // here than the last cycles of latency.
      auto v_item_load = [&](int q, VIn& I) {                        // q-th item of this thread's stream
        const int j = j0 + q / NVI, it = vt + NVT * (q % NVI), t = j * TC_BN + it / PARTS;
        if (q < n * NVI && it < TC_BN * PARTS && t < end) {
          I.w = tc_ldg128(P.kv.vq + (row0 + t) * (HD / 2) + (HD / 4) * (int)rank + 16 * (it % PARTS));
          I.s = tc_ldg16(P.kv.vscale + row0 + t); I.z = tc_ldg16(P.kv.vzero + row0 + t);
        }
      };
      auto v_prefetch = [&](int j) {                                 // L2 prefetch of a tile's half rows and per-token scales
        for (int x = vt; x < TC_BN; x += NVT) if (j * TC_BN + x < end) tc_prefetch_l2(P.kv.vq + (row0 + j * TC_BN + x) * (HD / 2) + (HD / 4) * (int)rank);
        if (vt < 4 && j * TC_BN + 64 * (vt & 1) < end) tc_prefetch_l2((vt & 2 ? P.kv.vzero : P.kv.vscale) + row0 + j * TC_BN + 64 * (vt & 1));
      };
      VIn cur, n1, n2;
      v_item_load(0, cur); v_item_load(1, n1);
      if (n > 1) v_prefetch(j0 + 1);
      int q = 0;
      for (int i = 0; i < n && ok; ++i) {
        const int j = j0 + i, st = i % L::NV;
        const uint32_t sv = sb + L::OFF_V + st * L::V_HALF;
        if (i + 2 < n) v_prefetch(j + 2);
        stage_wait(b_vempty + 8 * st, i, L::NV);
        if (!ok) break;
        #pragma unroll 1
        for (int u = 0; u < NVI; ++u, ++q) {
          v_item_load(q + 2, n2);
          const int it = vt + NVT * u, k = it / PARTS, part = it % PARTS;
          if (it < TC_BN * PARTS) {
            // no branches inside an item: a token that does not exist yet gets scale = zero = 0 (nibbles are finite whatever
            // the word holds), and the four words are converted before the four stores, so their chains interleave
            const bool live = j * TC_BN + k < end;
            const uint32_t s2 = live ? cur.s | (cur.s << 16) : 0u, z2 = live ? cur.z | (cur.z << 16) : 0u;
            const uint32_t ww[4] = {cur.w.x, cur.w.y, cur.w.z, cur.w.w};
            uint4 out[4];
            #pragma unroll
            for (int e = 0; e < 4; ++e) {
              uint32_t nb[4], r[4];
              tc_nibs(ww[e], nb);
              #pragma unroll
              for (int x = 0; x < 4; ++x) r[x] = tc_hfma2(nb[x], s2, z2);
              out[e] = tc_pairs_to_row(r);
            }
            const uint32_t base = sv + (part >> 1) * L::V_BLOCK + k * 128, kx = (uint32_t)(k & 7), c0 = 4 * (part & 1);   // chunk 4*part + e of the half row
            #pragma unroll
            for (int e = 0; e < 4; ++e) tc_sts128(base + (((c0 + e) ^ kx) << 4), out[e]);
          }
          cur = n1; n1 = n2;
        }
        publish(lead_vfull + 8 * st);
      }
      }
    }
  };
  auto role_softmax = [&]() {
    // ======================================================================= softmax warps: two threads per query row
    const int quad = warp & 3, hf = warp >> 2;                       // TMEM lane quadrant; which 64 of the tile's 128 key columns
    const int rho = quad * 32 + lane;                                // row of the tile = TMEM lane
    const int tok = tok0 + rho / G, head = rho % G;
    const bool valid = rho < TOK * G && tok < P.M;
    const int pr = pos0 + tok, cr = pr / 32;                         // row position and its own group
    const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
    const float cs = P.qscale * TC_LOG2E;
    if constexpr (FORM == 3) {
      if (n > 0) {
        // bf16 activations in the workspace form: these eight warps write this CTA's query rows as fp16 operand rows
        // (the converting forms leave that to their K converters); rows without a query are zero
        tc_stage_q_bf16<HD>(sb + L::OFF_Q, L::Q_BLOCK, P.q16, tok0, G, TOK, P.M, P.nh, kvh * G, threadIdx.x, 32 * TC_SW);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) bar_arrive_cluster(lead_q);
      }
    }
    // The row's two threads swap one float per tile through shared memory: value first, then a sequence number the
    // partner polls (bounded, like every wait here; a named barrier could not give up).
    volatile float* xval = reinterpret_cast<volatile float*>(smem + L::OFF_XCH);
    volatile uint16_t* xseq = reinterpret_cast<volatile uint16_t*>(smem + L::OFF_XCH + 2 * 2 * 128 * 4);   // tags modulo 2^16
    auto swap_with_partner = [&](float v, int tag) -> float {       // tag = 1, 2, 3, ... in program order
      xval[((tag & 1) * 2 + hf) * 128 + rho] = v;
      __threadfence_block();
      xseq[hf * 128 + rho] = (uint16_t)tag;
      for (uint32_t it = 0; it < TC_WAIT_LIMIT; ++it) {             // until the partner is at this tag (or one ahead)
        if ((uint16_t)(xseq[(hf ^ 1) * 128 + rho] - (uint16_t)tag) < 0x8000u) { __threadfence_block(); return xval[((tag & 1) * 2 + (hf ^ 1)) * 128 + rho]; }
      }
      atomicExch(&g_tc_status, 4); *s_abort = 1;
      return v;
    };
    float m = -1e30f, l = 0.f;                                       // m is common to the row's two threads, l is this half's sum
    int srd[2] = {0, 0};                                             // how often each S buffer has been read
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) {
      const int j = j0 + i;
      const bool edge = i >= npipe;
      const int buf = edge ? 0 : (i & 1);
      const uint32_t scol = trow + (buf ? L::TM_S1 : L::TM_S0) + 64 * hf;   // this thread's 64 S columns; P goes over the first 32
      float x[64];                                                   // raw scores of this thread's 64 keys
      if (!bar_wait(b_sready + 8 * buf, srd[buf] & 1)) { atomicExch(&g_tc_status, 4); *s_abort = 1; ok = false; break; }
      tc_fence_after();
      tmem_ld64(scol, x);
      ++srd[buf];
      if (edge) {
        if (!bar_wait(b_sready + 8, srd[1] & 1)) { atomicExch(&g_tc_status, 4); *s_abort = 1; ok = false; break; }
        tc_fence_after();
        ++srd[1];
        // each 32-key quarter is one group: before the row's own -> int4 keys; own group -> shadow keys up to the row; later -> nothing
        #pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float a[32];
          tmem_ld32(trow + L::TM_S1 + 64 * hf + 32 * h2, a);
          const int gk = 4 * j + 2 * hf + h2, tb = j * TC_BN + 64 * hf + 32 * h2;
          #pragma unroll
          for (int k = 0; k < 32; ++k) x[32 * h2 + k] = gk < cr ? x[32 * h2 + k] : (gk == cr && tb + k <= pr) ? a[k] : -INFINITY;
        }
      }
      if (I8 && i >= nbulk) {                                        // INT8 rows: the tiles that hold the new rows are masked causally
        const int tb = j * TC_BN + 64 * hf;
        #pragma unroll
        for (int k = 0; k < 64; ++k) x[k] = tb + k <= pr ? x[k] : -INFINITY;
      }
      // ---- online softmax in the log2 domain on p = 2^(x*cs - m); lazy rescale (the running max may lag by up to 2^8)
      float tmax = fmaxf(x[0], x[1]);
      #pragma unroll
      for (int k = 2; k < 64; k += 2) tmax = fmaxf(tmax, fmaxf(x[k], x[k + 1]));
      tmax = fmaxf(tmax, swap_with_partner(tmax, i + 1)) * cs;        // the row's two threads swap their maxima
      const bool bump = valid && tmax > m + 8.f;
      const float mn = bump ? tmax : m, alpha = bump ? tc_ex2(m - mn) : 1.f;
      m = mn; l *= alpha;
      uint32_t pk[32];
      {
        const float nm = -m;
        float ls0 = 0.f, ls1 = 0.f;
        #pragma unroll
        for (int k = 0; k < 64; k += 4) {
          const float p0 = tc_ex2(fmaf(x[k], cs, nm)), p1 = tc_ex2(fmaf(x[k + 1], cs, nm));        // exp2(-inf) = 0 for masked keys
          const float p2 = tc_ex2(fmaf(x[k + 2], cs, nm)), p3 = tc_ex2(fmaf(x[k + 3], cs, nm));
          ls0 += p0 + p1; ls1 += p2 + p3; pk[k / 2] = tc_pack(p0, p1); pk[k / 2 + 1] = tc_pack(p2, p3);
        }
        l += ls0 + ls1;
      }
      if (__any_sync(0xffffffffu, !valid) && !valid) {               // rows of the tile that hold no query: P = 0, state untouched
        #pragma unroll
        for (int k = 0; k < 32; ++k) pk[k] = 0u;
        l = 0.f;
      }
      // ---- O may be rescaled once P.V of tile i-1 is done (P.V of this tile waits for the signal below)
      if (i > 0 && __any_sync(0xffffffffu, bump)) {                  // rows that did not bump multiply by exactly 1
        if (!bar_wait(b_pvdone + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1)) { atomicExch(&g_tc_status, 4); *s_abort = 1; ok = false; break; }
        tc_fence_after();
        #pragma unroll 1
        for (int c = hf; c < HD / 32; c += 2) {                      // the row's two threads take alternate 32-column chunks of O
          float o[32];
          tmem_ld32(trow + L::TM_O + 32 * c, o);
          #pragma unroll
          for (int k = 0; k < 32; ++k) o[k] *= alpha;
          tmem_st32(trow + L::TM_O + 32 * c, o);
        }
      }
      tmem_st32u(scol, pk);                                          // P as the A operand of P.V, over S columns this thread has read
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) bar_arrive_cluster(lead_pready + 8 * (i & 1));
    }
    // ---- this split's result per (row, head): (m, l, O) partial, or the finished row when there is one split
    if (ok && n > 0 && !bar_wait(b_pvdone + 8 * ((n - 1) & 1), ((n - 1) >> 1) & 1)) { atomicExch(&g_tc_status, 4); *s_abort = 1; ok = false; }
    tc_fence_after();
    if (ok) l += swap_with_partner(l, n + 1);                        // the row's sum = the two halves' sums
    if (ok && !*s_abort) {
      const size_t pidx = ((size_t)tok * S + split) * P.nh + kvh * G + head;
      const bool direct = P.o16 != nullptr && S == 1;                // one split: this CTA holds the whole row, finish it here
      if (valid && !direct && hf == 0) { P.pm[pidx] = (n > 0 && m > -1e29f) ? m * TC_LN2 : -1e30f; P.pl[pidx] = n > 0 ? l : 0.f; }
      #pragma unroll 1
      for (int c = hf; c < HD / 32; c += 2) {
        float o[32];
        if (n > 0) tmem_ld32(trow + L::TM_O + 32 * c, o);
        else {
          #pragma unroll
          for (int k = 0; k < 32; ++k) o[k] = 0.f;
        }
        if (valid && direct) {                                       // y = round_f16(o / l) (+ V bias), as the merge kernel
          const size_t oi = ((size_t)tok * P.nh + kvh * G + head) * HD + 32 * c;
          uint32_t w[16];
          #pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float y0 = round_f16(o[k] / l), y1 = round_f16(o[k + 1] / l);
            if (act_bf16) {
              if (P.bv) { y0 = __fadd_rn(y0, bf2f(P.bv[kvh * HD + 32 * c + k])); y1 = __fadd_rn(y1, bf2f(P.bv[kvh * HD + 32 * c + k + 1])); }
              w[k / 2] = (uint32_t)f2bf(y0) | ((uint32_t)f2bf(y1) << 16);
              continue;
            }
            if (P.bv) { y0 = __fadd_rn(y0, h2f(P.bv[kvh * HD + 32 * c + k])); y1 = __fadd_rn(y1, h2f(P.bv[kvh * HD + 32 * c + k + 1])); }
            w[k / 2] = (uint32_t)f2h(y0) | ((uint32_t)f2h(y1) << 16);
          }
          uint4* dst = reinterpret_cast<uint4*>(P.o16 + oi);
          #pragma unroll
          for (int k = 0; k < 4; ++k) dst[k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
        } else if (valid) {
          float4* dst = reinterpret_cast<float4*>(P.pacc + pidx * HD + 32 * c);
          #pragma unroll
          for (int k = 0; k < 8; ++k) dst[k] = make_float4(o[4 * k], o[4 * k + 1], o[4 * k + 2], o[4 * k + 3]);
        }
      }
    }
  };
  // ---- roles.  In the converting forms each warpgroup first sets its register budget (120 / 120 / 112 / 160 per thread: 512
  //      per scheduler lane) and the role code sits under that branch, so that each role is compiled for its own budget.
  if constexpr (FUSED) {
    if (warp < TC_SW) { asm volatile("setmaxnreg.dec.sync.aligned.u32 120;"); role_softmax(); }
    else if (warp < TC_SW + 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 112;");
      if (warp == TC_SW) { role_producer(); role_mma(); } else role_conv(false);
    } else { asm volatile("setmaxnreg.inc.sync.aligned.u32 160;"); role_conv(true); }
  } else {
    if (warp == TC_SW) role_producer();
    else if (warp == TC_SW + 1) role_mma();
    else role_softmax();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                                // neither CTA's shared or tensor memory is in use by the other any more
  if (warp == TC_SW + 1) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(L::TM_COLS) : "memory");
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn tc_encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// Encoded maps are kept per (kind, base, extents): a decode loop calls with the same buffers every step and
// cuTensorMapEncodeTiled costs a few microseconds of host time per map.
struct TcMapKey {
  int kind; const void* base; uint64_t a, b, c, d;
  bool operator==(const TcMapKey& o) const { return kind == o.kind && base == o.base && a == o.a && b == o.b && c == o.c && d == o.d; }
};
struct TcMapHash {
  size_t operator()(const TcMapKey& k) const {
    size_t h = std::hash<const void*>()(k.base) ^ (size_t)k.kind * 0x9E3779B97F4A7C15ull;
    for (uint64_t v : {k.a, k.b, k.c, k.d}) h = (h ^ v) * 0x100000001B3ull;
    return h;
  }
};
template <class Make> bool tc_cached_map(CUtensorMap* out, const TcMapKey& key, Make make) {
  static std::mutex mu; static std::unordered_map<TcMapKey, CUtensorMap, TcMapHash> cache;
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  if (!make(out)) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// fp16 array [rows][hd] viewed as (64 channels, rows, hd/64 channel blocks): one copy of a box (64, box_rows, box_blocks)
// lands in shared memory as [block][row][128 bytes], 128-byte swizzle -- the tensor core's operand layout.
bool tc_map_rows(CUtensorMap* out, const void* base, uint64_t rows, int hd, int box_rows, int box_blocks) {
  return tc_cached_map(out, TcMapKey{0, base, rows, (uint64_t)hd, (uint64_t)box_rows, (uint64_t)box_blocks}, [&](CUtensorMap* m) {
    EncodeFn fn = tc_encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {64, rows, (cuuint64_t)(hd / 64)}, strides[2] = {(cuuint64_t)hd * 2, 128};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_blocks}, es[3] = {1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  });
}

// q16 [M][kvh][G][hd] viewed as 4-D; box = 64 channels x G heads x 1 kv-head x TOK tokens: rows land as (token, head).
bool tc_map_q(CUtensorMap* out, const void* q16, int M, int kvh, int G, int hd) {
  return tc_cached_map(out, TcMapKey{1, q16, (uint64_t)M, (uint64_t)kvh, (uint64_t)G, (uint64_t)hd}, [&](CUtensorMap* m) {
    EncodeFn fn = tc_encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)G, (cuuint64_t)kvh, (cuuint64_t)M};
    const cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)G * hd * 2, (cuuint64_t)kvh * G * hd * 2};
    const cuuint32_t box[4] = {64, (cuuint32_t)G, 1, (cuuint32_t)(128 / G)}, es[4] = {1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(q16), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  });
}

// Launch with programmatic stream serialization allowed (the kernel waits in griddepcontrol.wait after its set-up).
template <class K>
int tc_launch_pdl(K kern, dim3 grid, int threads, int smem_bytes, cudaStream_t st, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2,
                  const CUtensorMap& m3, const TcP& P) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smem_bytes; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  KV4_CUDA(cudaLaunchKernelEx(&cfg, kern, m0, m1, m2, m3, P));
  return 0;
}

struct TcWs { uint16_t* kd; uint16_t* vd; uint16_t* ks; int ks_rows; size_t bytes; };
TcWs carve(void* ws, int kvh, int hd, int max_ctx, int M) {
  TcWs w; const size_t plane = (size_t)kvh * max_ctx * hd * 2;
  w.ks_rows = TC_BN * ((M + TC_BN - 1) / TC_BN + 1);
  w.kd = static_cast<uint16_t*>(ws);
  w.vd = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(ws) + plane);
  w.ks = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(ws) + 2 * plane);
  w.bytes = 2 * plane + (size_t)kvh * w.ks_rows * hd * 2;
  return w;
}

template <int HD>
int launch_tc_hd(const yskn_attn_g_args& a, int g, int rd, int bf16, const TcWs& w, int valid_tokens, uint16_t* o16, const uint16_t* bv, cudaStream_t st) {
  using L = TcLay<HD>;
  // Tokens below valid_tokens are in the workspace already (the caller guarantees valid_tokens <= *d_pos); the group that
  // holds valid_tokens may have been completed since, and the shadow rows start at the 128-token tile of *d_pos.
  const int t_begin = (valid_tokens / TC_BN) * TC_BN;
  PrepP pp{a.kv, a.d_pos, a.M, a.max_ctx, a.kvh, a.rope, rd, w.kd, w.vd, w.ks, w.ks_rows, valid_tokens, t_begin};
  const int span = a.max_ctx - t_begin;
  if (span <= 0) KV4_REJECT("yskn_kv4_attention_tc: valid_tokens %d is beyond max_ctx %d", valid_tokens, a.max_ctx);
  kv4_tc_prep_kernel<HD><<<dim3((unsigned)((span + 3) / 4), (unsigned)a.kvh), 128, 0, st>>>(pp);
  if (int rc = launch_status("kv4_tc_prep_kernel")) return rc;
  CUtensorMap mq, mkd, mvd, mks;
  const uint64_t rows = (uint64_t)a.kvh * a.max_ctx;
  if (bf16) memset(&mq, 0, sizeof(mq));                               // the softmax warps stage Q
  if ((!bf16 && !tc_map_q(&mq, a.q16, a.M, a.kvh, g, HD)) || !tc_map_rows(&mkd, w.kd, rows, HD, TC_BN / 2, L::KBLK) ||
      !tc_map_rows(&mvd, w.vd, rows, HD, TC_BN, L::KBLK / 2) || !tc_map_rows(&mks, w.ks, (uint64_t)a.kvh * w.ks_rows, HD, TC_BN / 2, L::KBLK))
    KV4_REJECT("yskn_kv4_attention_tc: cuTensorMapEncodeTiled failed or is unavailable");
  auto kern = bf16 ? kv4_tc_attn_kernel<HD, 3> : kv4_tc_attn_kernel<HD, 0>;
  static std::atomic<unsigned long long> attr[2] = {{0}, {0}};
  if (first_use_on_device(attr[bf16 != 0])) KV4_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  const int tok = 128 / g, qtiles = ((a.M + tok - 1) / tok + 1) & ~1;        // CTA pairs: an even number of query tiles
  TcP P{a.d_pos, a.M, a.splits, g, a.nh, a.max_ctx, w.ks_rows, a.qscale, a.pm, a.pl, a.pacc, o16, bv, a.kv, a.rope, rd,
        static_cast<const uint16_t*>(a.q16), bf16, nullptr, nullptr, nullptr, nullptr};
  if (int rc = tc_launch_pdl(kern, dim3(qtiles, a.splits, a.kvh), TC_THREADS, L::TOTAL, st, mq, mkd, mvd, mks, P)) return rc;
  return launch_status("kv4_tc_attn_kernel");
}

// The fused form: one launch, no workspace.
template <int HD>
int launch_tc_fused_hd(const yskn_attn_g_args& a, int g, int rd, int bf16, uint16_t* o16, const uint16_t* bv, cudaStream_t st) {
  using L = TcLay<HD>;
  CUtensorMap mq;
  if (bf16) memset(&mq, 0, sizeof(mq));                               // the converter warps stage Q
  else if (!tc_map_q(&mq, a.q16, a.M, a.kvh, g, HD)) KV4_REJECT("yskn_kv4_attention: cuTensorMapEncodeTiled failed or is unavailable");
  auto kern = kv4_tc_attn_kernel<HD, 1>;
  static std::atomic<unsigned long long> attr{0};
  if (first_use_on_device(attr)) KV4_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  const int tok = 128 / g, qtiles = ((a.M + tok - 1) / tok + 1) & ~1;
  TcP P{a.d_pos, a.M, a.splits, g, a.nh, a.max_ctx, 0, a.qscale, a.pm, a.pl, a.pacc, o16, bv, a.kv, a.rope, rd, static_cast<const uint16_t*>(a.q16), bf16,
        nullptr, nullptr, nullptr, nullptr};
  if (int rc = tc_launch_pdl(kern, dim3(qtiles, a.splits, a.kvh), tc_threads(true), L::TOTAL, st, mq, mq, mq, mq, P)) return rc;
  return launch_status("kv4_tc_attn_kernel (fused)");
}

}  // namespace

bool attention_tc_supports(int g, int hd, int rd, int act_dtype) {
  return g >= 1 && g <= 8 && (hd == 256 || hd == 128) && rd >= 0 && rd <= hd && rd % 2 == 0 && (act_dtype == YSKN_KV4_F16 || act_dtype == YSKN_KV4_BF16) &&
         (rd == 0 || ((rd / 2) % (hd / 32) == 0 && (((rd / 2) / (hd / 32)) & ((rd / 2) / (hd / 32) - 1)) == 0));
}

size_t attention_tc_workspace_bytes(int kvh, int hd, int max_ctx, int M) { return carve(nullptr, kvh, hd, max_ctx, M).bytes; }

int launch_attention_tc(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, void* workspace, size_t workspace_bytes,
                        int valid_tokens, uint16_t* o16_direct, const uint16_t* bv, cudaStream_t st) {
  if (!workspace && workspace_bytes == 0) return launch_attention_tc_fused(a, g, hd, rd, act_dtype, o16_direct, bv, st);   // no workspace: convert inside the kernel
  if (!attention_tc_supports(g, hd, rd, act_dtype))
    KV4_REJECT("yskn_kv4_attention_tc: unsupported (g %d, hd %d, rd %d, act_dtype %d): fp16 or bf16 activations, hd 128/256", g, hd, rd, act_dtype);
  const TcWs w = carve(workspace, a.kvh, hd, a.max_ctx, a.M);
  if (!workspace || workspace_bytes < w.bytes) KV4_REJECT("yskn_kv4_attention_tc: workspace of %zu bytes needed, %zu given", w.bytes, workspace_bytes);
  if (((uintptr_t)workspace | (uintptr_t)a.q16) & 15) KV4_REJECT("yskn_kv4_attention_tc: workspace and q16 must be 16-byte aligned");
  if (valid_tokens < 0) valid_tokens = 0;
  if (o16_direct && ((uintptr_t)o16_direct & 15)) KV4_REJECT("yskn_kv4_prefill_tc: o16 must be 16-byte aligned");
  if (!o16_direct && ((uintptr_t)a.pacc & 15)) KV4_REJECT("yskn_kv4_attention_tc: pacc must be 16-byte aligned");
  const int bf16 = act_dtype == YSKN_KV4_BF16;
  return hd == 256 ? launch_tc_hd<256>(a, g, rd, bf16, w, valid_tokens, o16_direct, bv, st) : launch_tc_hd<128>(a, g, rd, bf16, w, valid_tokens, o16_direct, bv, st);
}

// Many-row attention straight from the packed cache (no workspace, one launch).  Same shapes as the workspace form, and the
// rotary width must be a whole number of 16-channel word pairs.
bool attention_tc_fused_supports(int g, int hd, int rd, int act_dtype) {
  return (act_dtype == YSKN_KV4_F16 || act_dtype == YSKN_KV4_BF16) && attention_tc_supports(g, hd, rd, YSKN_KV4_F16) && rd % 16 == 0;
}

int launch_attention_tc_fused(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, uint16_t* o16_direct, const uint16_t* bv, cudaStream_t st) {
  if (!attention_tc_fused_supports(g, hd, rd, act_dtype))
    KV4_REJECT("yskn_kv4_attention: fused tensor-core form does not cover (g %d, hd %d, rd %d, act_dtype %d)", g, hd, rd, act_dtype);
  const uintptr_t al = (uintptr_t)a.q16 | (uintptr_t)a.kv.kq | (uintptr_t)a.kv.vq | (uintptr_t)a.kv.kscale | (uintptr_t)a.kv.kzero | (uintptr_t)a.kv.kshadow |
                       (uintptr_t)a.rope | (o16_direct ? (uintptr_t)o16_direct : (uintptr_t)a.pacc);
  if (al & 15) KV4_REJECT("yskn_kv4_attention: q16, cache arrays, rope table and pacc / o16 must be 16-byte aligned");
  const int bf16 = act_dtype == YSKN_KV4_BF16;
  return hd == 256 ? launch_tc_fused_hd<256>(a, g, rd, bf16, o16_direct, bv, st) : launch_tc_fused_hd<128>(a, g, rd, bf16, o16_direct, bv, st);
}

// Many-row attention over Family-B INT8 rows on the tcgen05 kernel (FORM 2): partials in the layout of yskn_kv8_attention.
int launch_kv8_attention_tc(const yskn_kv8_attn_args& a, int act_dtype, cudaStream_t st) {
  if (!a.q16 || !a.k8 || !a.v8 || !a.ks || !a.vs || !a.d_pos || !a.pm || !a.pl || !a.pacc) KV4_REJECT("yskn_kv8_attention_tc: null buffer");
  if (a.kvh <= 0 || a.nh <= 0 || a.nh % a.kvh || a.nh / a.kvh > 8 || a.M <= 0 || a.M > 65535 || a.kvh > 65535 || a.splits <= 0 || a.splits > 65535 ||
      a.max_ctx <= 0 || a.max_ctx % 64)
    KV4_REJECT("yskn_kv8_attention_tc: bad shape (kvh %d, nh %d, M %d, splits %d, max_ctx %d)", a.kvh, a.nh, a.M, a.splits, a.max_ctx);
  if (act_dtype != YSKN_KV4_F16 && act_dtype != YSKN_KV4_BF16) KV4_REJECT("yskn_kv8_attention_tc: q16 is fp16 or bf16 (act_dtype %d)", act_dtype);
  if (((uintptr_t)a.k8 | (uintptr_t)a.v8 | (uintptr_t)a.q16 | (uintptr_t)a.pacc) & 15) KV4_REJECT("yskn_kv8_attention_tc: k8, v8, q16 and pacc must be 16-byte aligned");
  using L = TcLay<256>;
  const int g = a.nh / a.kvh, bf16 = act_dtype == YSKN_KV4_BF16;
  CUtensorMap mq;
  if (bf16) memset(&mq, 0, sizeof(mq));
  else if (!tc_map_q(&mq, a.q16, a.M, a.kvh, g, 256)) KV4_REJECT("yskn_kv8_attention_tc: cuTensorMapEncodeTiled failed or is unavailable");
  auto kern = kv4_tc_attn_kernel<256, 2>;
  static std::atomic<unsigned long long> attr{0};
  if (first_use_on_device(attr)) KV4_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
  const int tok = 128 / g, qtiles = ((a.M + tok - 1) / tok + 1) & ~1;
  TcP P{a.d_pos, a.M, a.splits, g, a.nh, a.max_ctx, 0, a.qscale, a.pm, a.pl, a.pacc, nullptr, nullptr, yskn_kv_layer{}, nullptr, 0,
        a.q16, bf16, a.k8, a.v8, a.ks, a.vs};
  if (int rc = tc_launch_pdl(kern, dim3(qtiles, a.splits, a.kvh), tc_threads(true), L::TOTAL, st, mq, mq, mq, mq, P)) return rc;
  return launch_status("kv4_tc_attn_kernel (INT8 rows)");
}

int tc_status_fetch(int* out) {
  int v = 0;
  KV4_CUDA(cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)));
  const int zero = 0;
  KV4_CUDA(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
  *out = v; return 0;
}

}  // namespace kv4
