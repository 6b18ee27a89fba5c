// KV4 GQA flash-decode for sm_100a: TMA-staged packed cache, int4 -> fp16 in registers, warp-level
// tensor-core tiles, online softmax by warp shuffles, split-K partials.
//
// Semantics: the reference's attention_gqa_kernel (src/attention_gqa.cu:17-118) -- row r at *d_pos + r sees keys
// 0..pos; 32-token groups before the row's own group are read as int4 (k = nib*scale + zero), the own group from
// the fp16 shadow; K is rotated at read time; V is int4 per token; output = (m, l, un-normalised O) per split.
// Results agree with the reference to the attention tolerance, not bit for bit: the split boundaries are whole
// 32-token groups and the products run on tensor cores with fp16 operands.
//
// Why tensor cores for an HBM-bound kernel: one cached token costs 292 bytes but 2*G*HD = 3072 multiply-adds
// (G 6, HD 256); at 75 % of HBM bandwidth that is ~50 T multiply-adds/s, more than the fp32 pipes deliver.
//
// Work split.  grid (splits, Hkv, M), one CTA per SM when splits*Hkv*M = 148.  A CTA owns a run of 128-token units
// (four 32-token groups) of one kv-head.  One producer warp streams each unit into an mbarrier ring with seven
// copies: K 128 x HD/2 bytes and V 128 x HD/2 bytes by tiled TMA (128-byte swizzle), four K scale rows, four K zero
// rows, 128 V scales, 128 V zeros (bulk copies) and the four rope rows of the groups' first positions (one strided
// TMA tile).  Few, large copies matter: the number of copies in flight per SM is limited, not only their bytes.
// Seven consumer warps take the groups round-robin and keep their own (m, l, O) state.  A group is two 16-token
// MMA tiles:
//   S^T[16 tok x 8 heads]  = K[16 tok x HD] . Q^T[HD x 8 heads]          (m16n8k16, HD/16 steps)
//   O^T[HD x 8 heads]     += V^T[HD x 16 tok] . P^T[16 tok x 8 heads]    (HD/16 m-tiles)
// so one K/V tile serves all G <= 8 query heads of the group, and the packed bytes go from shared memory straight
// into A-fragment registers:
//   * a 32-bit word holds 8 nibbles; one LOP3 reads nibbles (x, x+4) in place as the half2 (off+n_x, off+n_{x+4}):
//     bits 0..3 of a half count in steps of 1 under exponent 2^10 (off 1024), bits 4..7 under 2^6 (off 64).  That is
//     exactly one A register because the contraction order over channels is free.  K's per-channel scale is folded
//     into Q once per group (q' = q*scale); the zero points and the offsets become a per-head bias,
//     sum q*zero - sum off*q', formed by two more MMA rows so that the offsets cancel against the rounded q'.
//   * for V the contraction runs over tokens: a transposed 8x8 shared-memory load (ldmatrix.trans) hands a lane the same
//     four channels of two consecutive tokens in one register, which is the pairing an A register wants.  V's per-token
//     scale is folded into P and its zero point into a per-head scalar.  The even channels' offset of 1024 is removed by
//     an exact fp16 subtraction before the MMA: the tensor core's fp32 accumulators truncate, and a sum that carries
//     1024 * sum(p) loses about 2e-3 of the output at 262,144 tokens (measured, on the even channels only); the odd
//     channels' offset of 64 stays and is cancelled by an MMA row of ones over the same rounded P.
//   * RoPE: Q is rotated back by the group's first position (one table row per group), the remaining angle
//     (0..31 tokens) is applied to the rotary channels of K with the table's first 32 rows.  cos/sin of
//     (t0 + dt) are thereby formed by angle addition from the caller's table entries for t0 and dt.  The table's own
//     angle at t is the fp32 product t*freq, which differs from the sum of the two entries' angles by up to one ulp of
//     t*freq (0.03 rad at t = 262,144 for the highest frequency): a per-token perturbation of the score of about 1e-3,
//     random in sign, that changed no digit of the measured error at 262,144 tokens (a build that read the table row of
//     every token for the eight highest frequencies gave the same error and ran 16 % slower).
// Lane (g = lane/4, j = lane%4) owns words w = 4i + j of a packed K row, so a rotary pair (c, c + RD/2) stays
// in one lane.
//
// Every wait is bounded: a wait that runs out sets a device status word and the CTA drains and returns.
#include "kv4_common.cuh"
#include <cuda.h>
#include <mutex>
#include <type_traits>
#include <unordered_map>
#include <cstring>
#include <vector>

namespace kv4 {

__device__ int g_decode_status = 0;          // 0 ok; 1 = a consumer wait ran out; 2 = a producer wait ran out

namespace {

#ifndef KV4_DECODE_NCW
#define KV4_DECODE_NCW 7                     // consumer warps per CTA
#endif
#ifndef KV4_DECODE_MAXREG
#define KV4_DECODE_MAXREG 255                // 2 warps per SM sub-partition, one CTA of 8 warps per SM.  Measured at 262,144 tokens:
                                             // 4 / 6 / 8 / 12 / 16 warps (255 / 255 / 255 / 168 / 128 registers) = 127 / 111 / 83.5 / 90.2 / 107 us per step
#endif
constexpr int NSTAGE = 5;                    // ring depth (128-token units in flight per CTA)
constexpr int NCW = KV4_DECODE_NCW;
constexpr int NTHREADS = (NCW + 1) * 32;
constexpr uint32_t WAIT_LIMIT = 1u << 22;    // polls of try_wait before giving up (each poll suspends up to ~us)
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

template <int HD, int RD> struct Lay {
  static constexpr int UG = 4;                             // groups per unit (one ring stage)
  static constexpr int ROWB = HD / 2;                      // bytes of one packed row
  static constexpr int KB = 32 * ROWB;                     // packed K (or V) bytes of one group
  static constexpr int SCB = HD * 2;                       // one fp16 scale row
  static constexpr int ROPEB = RD / 2 * 8;                 // one rope row
  static constexpr int SHADOW = 32 * HD * 2;               // fp16 rows of the open group (= UG*KB: it takes K's place)
  static constexpr int OFF_K = 0, OFF_V = UG * KB, OFF_KS = 2 * UG * KB, OFF_KZ = OFF_KS + UG * SCB, OFF_VS = OFF_KZ + UG * SCB,
                       OFF_VZ = OFF_VS + UG * 64, OFF_ROPE = OFF_VZ + UG * 64;
  static constexpr int STAGE = (OFF_ROPE + UG * ROPEB + 1023) / 1024 * 1024;
  static constexpr int NW = HD / 32;                       // packed words per lane per row
  static constexpr int NR = RD / 32;                       // of which rotary (first NR); pairs (i, i + NR/2)
  static constexpr int NP = NR / 2;
  static constexpr int QFRAG = NW * 32 * 16;               // Q as B fragments: [i][lane] x 16 bytes
  static constexpr int RELT = 4 * (NP ? NP : 1) * 2 * 32 * 16;   // relative rotation: [tile][half][i][xpair][lane] x 16 B
  static constexpr int OFF_STAGES = 0;
  static constexpr int OFF_QFRAG = NSTAGE * STAGE;
  static constexpr int OFF_RELT = OFF_QFRAG + QFRAG;
  static constexpr int OFF_BARS = OFF_RELT + RELT;         // full[NSTAGE], empty[NSTAGE]
  static constexpr int OFF_MISC = OFF_BARS + 2 * NSTAGE * 8;
  static constexpr int TOTAL = OFF_MISC + 64;
  static constexpr int MERGE = NCW * 8 * (HD + 2) * 4;     // aliases the stage ring after the loop
  static_assert(MERGE <= NSTAGE * STAGE, "merge buffer must fit in the ring");
  static_assert(SHADOW == UG * KB, "the open group's fp16 rows take the place of the unit's packed K");
  static_assert(NR % 2 == 0 && NR <= NW, "rotary width must be a multiple of 64 and at most head_dim");
  static_assert(TOTAL <= 227 * 1024, "shared memory budget of one CTA");
};

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_t(uint32_t a, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) { uint32_t d; asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a)); return d; }
__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) { uint32_t d; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo)); return d; }
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) { uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
__device__ __forceinline__ uint32_t hadd2(uint32_t a, uint32_t b) { uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t hneg2(uint32_t a) { return a ^ 0x80008000u; }
// A 32-bit word of a packed row holds nibbles 0..7.  Register X pairs nibbles (X, X+4) as the two halves of a
// half2 WITHOUT moving them: nibbles at bits 0..3 of a half read as 1024 + n under exponent 2^10 (0x6400), nibbles at
// bits 4..7 as 64 + n under exponent 2^6 (0x5400).  One shift (w >> 8) serves X = 2, 3.  The constant offsets are
// removed exactly: on the Q side by an MMA row of the same constants, on the rotary path by an exact subtraction.
constexpr uint32_t OFF_E = 0x64006400u, OFF_O = 0x54005400u;       // (1024,1024), (64,64)
constexpr uint32_t NEG_E = 0xE400E400u, NEG_O = 0xD400D400u;       // their negatives
// (a & m) | c as ONE LOP3.  LOP3 takes a single immediate, so with two literal constants the compiler emits AND then OR
// (measured: 562 LOP3 per group instead of ~280); the masks and offsets are therefore kept in registers that the
// compiler cannot fold (NibK).
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t m, uint32_t c) {
  uint32_t d; asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(m), "r"(c)); return d;
}
struct NibK { uint32_t m0, m1, e, o; };                          // 0x000F000F, 0x00F000F0, OFF_E, OFF_O
__device__ __forceinline__ NibK nib_consts() {
  NibK k;
  asm volatile("mov.u32 %0, 0x000F000F;\n mov.u32 %1, 0x00F000F0;\n mov.u32 %2, 0x64006400;\n mov.u32 %3, 0x54005400;"
               : "=r"(k.m0), "=r"(k.m1), "=r"(k.e), "=r"(k.o));
  return k;
}
__device__ __forceinline__ void nib_regs(uint32_t w, uint32_t (&o)[4], const NibK& c) {
  const uint32_t w8 = w >> 8;
  o[0] = and_or(w, c.m0, c.e); o[1] = and_or(w, c.m1, c.o);
  o[2] = and_or(w8, c.m0, c.e); o[3] = and_or(w8, c.m1, c.o);
}
// eight consecutive fp16 (r.x = (e0,e1) .. r.w = (e6,e7)) -> register X pairing elements (X, X+4)
__device__ __forceinline__ void pair_regs(const uint4& r, uint32_t (&o)[4]) {
  o[0] = __byte_perm(r.x, r.z, 0x5410); o[1] = __byte_perm(r.x, r.z, 0x7632);
  o[2] = __byte_perm(r.y, r.w, 0x5410); o[3] = __byte_perm(r.y, r.w, 0x7632);
}
__device__ __forceinline__ float lds_h(uint32_t a) {
  unsigned short v; asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a)); return __half2float(__ushort_as_half(v));
}

// ---------------------------------------------------------------- kernel
struct DecodeP {
  yskn_attn_g_args A;
  Shard sh;
  int g;
  int early;          // the caller's promise (yskn_kv4_attn_ext): *d_pos and every cache row below it are final before the
                      // preceding kernel of the stream ends, so they may be read ahead of griddepcontrol.wait
  yskn_kv4_ms_rows ms;  // rows of several sequences (ms.pos != nullptr): row r reads the cache ms.layers[ms.slot[r]] at position ms.pos[r]
};

template <int HD, int RD, int DT>
__global__ void __maxnreg__(KV4_DECODE_MAXREG)
kv4_decode_mma_kernel(const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                      const __grid_constant__ CUtensorMap mapR, const DecodeP P) {
  using L = Lay<HD, RD>;
  constexpr int NW = L::NW, NR = L::NR, NP = L::NP, NRd = NR > 0 ? NR : 1;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const yskn_attn_g_args& A = P.A;
  const int split = blockIdx.x, kvh = blockIdx.y, r = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, j = lane & 3;
  const int G = P.g;
  // Programmatic dependent launch in both directions (src/pdl.cuh:15-30 is the reference's form of this): this grid may be
  // scheduled while the previous kernel of the stream drains and waits here before it reads anything that kernel wrote
  // (position, query, appended rows); the merge kernel that follows may be scheduled early in turn and waits for this grid
  // to finish before it reads the partials.
  // With `early` (the reference's Q35AttnArgs.early, src/q35_kernels.cu:1195-1206) the position is read and the producer
  // fills the ring with rows below the base position BEFORE the wait: those rows were final before the predecessor started.
  const bool early = P.early != 0;
  if (!early) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }

  // ---- which groups this CTA owns (local token indices of this shard)
  const bool multi = P.ms.pos != nullptr;                       // rows of several sequences: per-row position and cache
  const int base_local = multi ? P.ms.pos[r] : *A.d_pos - P.sh.start;   // row 0's local position: rows below it are never written again
  const int pos = multi ? base_local : base_local + r;
  const int len = max(0, min(pos + 1, P.sh.len));
  const int cg = pos >= 0 ? pos / 32 : 0;                       // first group that is not read as int4
  const int nq = min(cg, len / 32);                             // int4 groups, all fully visible
  const bool has_tail = len > nq * 32;                          // the open group lives in this shard
  const int nu4 = (nq + L::UG - 1) / L::UG;                     // int4 units of four groups (the last may hold fewer)
  const int units = nu4 + (has_tail ? 1 : 0);                   // the open group is a unit of its own, the last one
  const int per = (units + (int)gridDim.x - 1) / (int)gridDim.x;
  const int u0 = min(units, split * per), u1 = min(units, u0 + per), nu = u1 - u0;

  const uint32_t bar_full = sbase + L::OFF_BARS, bar_empty = bar_full + NSTAGE * 8;
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::OFF_MISC);
  if (sbase & 1023u) { if (threadIdx.x == 0) atomicExch(&g_decode_status, 3); return; }   // the swizzled tiles need a 1 KB base
  if (threadIdx.x == 0) {
    // a stage is free again once the consumers of its four groups have arrived (units with fewer groups are never reused)
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, L::UG); }
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  float* mbuf = reinterpret_cast<float*>(smem);                 // merge buffer, aliases the ring after the loop

  if (warp == NCW) {
    // =========================================================== producer warp
    if (nu > 0) {
      const size_t row0 = (size_t)kvh * A.max_ctx;              // first row of this kv-head in the [Hkv*max_ctx] arrays
      const int slot = multi ? P.ms.slot[r] : 0;
      const yskn_kv_layer kvl = multi ? P.ms.layers[slot] : A.kv;
      const CUtensorMap* const mk = multi ? static_cast<const CUtensorMap*>(P.ms.maps) + 2 * slot : &mapK;
      const CUtensorMap* const mv = multi ? static_cast<const CUtensorMap*>(P.ms.maps) + 2 * slot + 1 : &mapV;
      int issued = 0;
      bool waited = !early;
      for (int k = 0; k < nu; ++k) {
        const int s = k % NSTAGE, u = u0 + k;
        // an early unit: one of the first ring fills, int4 only, every token below the base position
        if (!waited && (k >= NSTAGE || (has_tail && u == nu4) || min(nq, (u + 1) * L::UG) * 32 > max(0, min(base_local, P.sh.len)))) {
          asm volatile("griddepcontrol.wait;" ::: "memory");
          asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
          waited = true;
        }
        int go = 1;
        if (lane == 0) {
          if (k >= NSTAGE && !mbar_wait(bar_empty + 8 * s, ((k / NSTAGE) - 1) & 1)) { atomicExch(&g_decode_status, 2); *s_abort = 1; }
          if (*s_abort) go = 0;
        }
        go = __shfl_sync(0xffffffffu, go, 0);
        if (!go) break;
        const bool tail = has_tail && u == nu4;
        const int ngr = tail ? 1 : min(L::UG, nq - u * L::UG);   // groups in this unit
        const int g0 = tail ? nq : u * L::UG;                    // its first group (local index)
        const uint32_t st = sbase + L::OFF_STAGES + s * L::STAGE, bar = bar_full + 8 * s;
        if (lane == 0) mbar_expect_tx(bar, 2 * L::UG * L::KB + ngr * (2 * L::SCB * (tail ? 0 : 1) + 128) + L::UG * L::ROPEB);   // SHADOW == UG*KB
        __syncwarp();                                            // the barrier is armed before any copy is issued
        const size_t tok0 = row0 + (size_t)g0 * 32, gb = ((size_t)kvh * (A.max_ctx / 32) + g0) * HD;
        switch (lane) {                                          // one copy per lane: seven issue slots in parallel
          case 0: if (tail) bulk_1d(st + L::OFF_K, kvl.kshadow + tok0 * HD, L::SHADOW, bar);
                  else tma_2d(st + L::OFF_K, mk, 0, (int)tok0, bar); break;
          case 1: tma_2d(st + L::OFF_V, mv, 0, (int)tok0, bar); break;   // always the swizzled tile; rows past the unit are unused
          case 2: if (!tail) bulk_1d(st + L::OFF_KS, kvl.kscale + gb, ngr * L::SCB, bar); break;
          case 3: if (!tail) bulk_1d(st + L::OFF_KZ, kvl.kzero + gb, ngr * L::SCB, bar); break;
          case 4: bulk_1d(st + L::OFF_VS, kvl.vscale + tok0, ngr * 64, bar); break;
          case 5: bulk_1d(st + L::OFF_VZ, kvl.vzero + tok0, ngr * 64, bar); break;
          case 6: if (RD > 0) tma_2d(st + L::OFF_ROPE, &mapR, 0, g0 + P.sh.start / 32, bar); break;   // rows 32*(g0..g0+3) of the table
          default: break;
        }
        issued = k + 1;
      }
      if (!waited) { asm volatile("griddepcontrol.wait;" ::: "memory"); asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
      // After an abort nobody may have consumed the last copies: wait (bounded) until they have landed before the CTA ends.
      if (lane == 0 && *s_abort)
        for (int k = max(0, issued - NSTAGE); k < issued; ++k) mbar_wait(bar_full + 8 * (k % NSTAGE), (k / NSTAGE) & 1);
    } else if (early) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
  } else {
    // =========================================================== consumer warps
    if (early) {                                                // q16 and the partial buffers belong to the predecessor until here
      asm volatile("griddepcontrol.wait;" ::: "memory");
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    // ---- one-time set-up, spread over the consumer threads
    const int ct = threadIdx.x;                                 // 0..NCW*32-1
    {
      // Q as B fragments, pre-scaled by qscale*log2(e): entry [i][lane'] = 4 regs x, reg x = (q[g'][8w+x], q[g'][8w+x+4]), w = 4i+j'
      const float qs = A.qscale * LOG2E;
      for (int e = ct; e < NW * 32 * 4; e += NCW * 32) {
        const int x = e & 3, ln = (e >> 2) & 31, i = e >> 7, gg = ln >> 2, jj = ln & 3, c = 8 * (4 * i + jj) + x;
        float lo = 0.f, hi = 0.f;
        if (gg < G) {
          const size_t qb = ((size_t)r * A.nh + kvh * G + gg) * HD;
          lo = act_load<DT>(A.q16, qb + c) * qs; hi = act_load<DT>(A.q16, qb + c + 4) * qs;
        }
        reinterpret_cast<uint32_t*>(smem + L::OFF_QFRAG)[e] = pack_h2(lo, hi);
      }
      // relative rotation by dt = 0..31 tokens, from the table's rows 0..31: entry [tile][half][i][xp][lane'] =
      // {cd_{2xp}, sd_{2xp}, cd_{2xp+1}, sd_{2xp+1}}, each a half2 over frequencies (8w+x, 8w+x+4), w = 4i+j'
      if (RD > 0) {
        constexpr int NPd = NP > 0 ? NP : 1;
        for (int e = ct; e < 4 * NP * 2 * 32; e += NCW * 32) {
          const int ln = e & 31, xp = (e >> 5) & 1, i = (e >> 6) % NPd, th = (e >> 6) / NPd;   // th = tile*2 + half
          const int gg = ln >> 2, jj = ln & 3, dt = 8 * th + gg, w = 4 * i + jj;
          uint32_t o[4];
          #pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int f = 8 * w + 2 * xp + q;
            const float2 a = *reinterpret_cast<const float2*>(A.rope + ((size_t)dt * (RD / 2) + f) * 2);
            const float2 b = *reinterpret_cast<const float2*>(A.rope + ((size_t)dt * (RD / 2) + f + 4) * 2);
            o[2 * q] = pack_h2(a.x, b.x); o[2 * q + 1] = pack_h2(a.y, b.y);
          }
          *reinterpret_cast<uint4*>(smem + L::OFF_RELT + (size_t)e * 16) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");

    float acc[HD / 16][4];                                      // O^T: [m-tile][(even | odd channel) x (head 2j | 2j+1)]
    #pragma unroll
    for (int mt = 0; mt < HD / 16; ++mt) { acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f; }
    float m[2] = {-1e30f, -1e30f}, l[2] = {0.f, 0.f}, zacc[2] = {0.f, 0.f};   // heads 2j, 2j+1 (log2 domain); zacc = sum p*vzero
    float zs[4] = {0.f, 0.f, 0.f, 0.f};                         // [0], [1]: sum over ALL tokens of the rounded p*vscale, formed by an MMA against ones

    // per-lane constant offsets: K word i of row g (swizzled chunk), V chunk of rows 2j and 2j+1
    const int swz = HD == 256 ? (g & 7) : ((g >> 1) & 3);
    uint32_t koff[NW];
    #pragma unroll
    for (int i = 0; i < NW; ++i) koff[i] = g * L::ROWB + 16 * (i ^ swz) + 4 * j;
    // V through ldmatrix.trans: lane supplies the row address of matrix lane/8, row lane%8: token (mat&1)*8 + row, 16-byte
    // chunk 2q + (mat>>1) (q = which of the HD/64 loads), XOR-swizzled as the TMA tile is.
    const int vtok = ((lane >> 3) & 1) * 8 + (lane & 7), vch = lane >> 4;
    const uint32_t vrow = vtok * L::ROWB, vsw = HD == 256 ? (vtok & 7) : ((vtok >> 1) & 3);
    const uint32_t ONE2 = 0x3C003C00u;
    const uint32_t qfrag = sbase + L::OFF_QFRAG + lane * 16;
    const uint32_t relt = sbase + L::OFF_RELT + lane * 16;
    const NibK nk = nib_consts();

    // One 32-token group.  TAIL: the open group (fp16 shadow rows, `nvalid` visible tokens); else an int4 group.
    // `st` = stage base, `sub` = which of the unit's four groups (0 for the open group).
    auto group = [&](auto tail_c, const uint32_t st, const int sub, const int nvalid) {
      constexpr bool TAIL = decltype(tail_c)::value;
      const uint32_t s_k = st + L::OFF_K + sub * L::KB, s_v = st + L::OFF_V + sub * L::KB, s_ks = st + L::OFF_KS + sub * L::SCB,
                     s_kz = st + L::OFF_KZ + sub * L::SCB, s_vs = st + L::OFF_VS + sub * 64, s_rope = st + L::OFF_ROPE + sub * L::ROPEB;
      // ---- per-group fold: q' = q*scale (plain channels); Q rotated back by the group's first position (rotary
      //      channels); bias[h] = sum_c q[h][c]*zero[c] - sum_c off[c]*q'[h][c], both sums as MMA rows, so the operand
      //      offsets cancel exactly against the fp16-rounded q' the tiles really use.  Every A row carries the same
      //      vector, so every lane ends up with the bias of its own two heads.
      uint32_t qf[NW][4], rs[NRd][4], rz[NRd][4];
      float bz[4] = {0.f, 0.f, 0.f, 0.f}, bo[4] = {0.f, 0.f, 0.f, 0.f};
      #pragma unroll
      for (int i = 0; i < NW; ++i) {
        const uint4 q4 = lds128(qfrag + i * 512);
        const uint32_t qv[4] = {q4.x, q4.y, q4.z, q4.w};
        if (TAIL) {
          #pragma unroll
          for (int x = 0; x < 4; ++x) qf[i][x] = qv[x];
        } else {
          uint32_t sc[4], zz[4];
          pair_regs(lds128(s_ks + 16 * (4 * i + j)), sc);
          pair_regs(lds128(s_kz + 16 * (4 * i + j)), zz);
          if (i < NR) {
            #pragma unroll
            for (int x = 0; x < 4; ++x) { qf[i][x] = qv[x]; rs[i][x] = sc[x]; rz[i][x] = zz[x]; }
          } else {
            #pragma unroll
            for (int x = 0; x < 4; ++x) qf[i][x] = hmul2(qv[x], sc[x]);
            mma16816(bz, zz[0], 0u, zz[1], 0u, qv[0], qv[1]);
            mma16816(bz, zz[2], 0u, zz[3], 0u, qv[2], qv[3]);
            mma16816(bo, OFF_E, 0u, OFF_O, 0u, qf[i][0], qf[i][1]);
            mma16816(bo, OFF_E, 0u, OFF_O, 0u, qf[i][2], qf[i][3]);
          }
        }
      }
      if (RD > 0) {
        #pragma unroll
        for (int i = 0; i < NP; ++i) {
          const uint32_t rp = s_rope + 64 * (4 * i + j);     // 8 frequencies x (cos, sin) fp32
          const uint4 r0 = lds128(rp), r1 = lds128(rp + 16), r2 = lds128(rp + 32), r3 = lds128(rp + 48);
          const uint32_t C[4] = {pack_h2(__uint_as_float(r0.x), __uint_as_float(r2.x)), pack_h2(__uint_as_float(r0.z), __uint_as_float(r2.z)),
                                 pack_h2(__uint_as_float(r1.x), __uint_as_float(r3.x)), pack_h2(__uint_as_float(r1.z), __uint_as_float(r3.z))};
          const uint32_t S[4] = {pack_h2(__uint_as_float(r0.y), __uint_as_float(r2.y)), pack_h2(__uint_as_float(r0.w), __uint_as_float(r2.w)),
                                 pack_h2(__uint_as_float(r1.y), __uint_as_float(r3.y)), pack_h2(__uint_as_float(r1.w), __uint_as_float(r3.w))};
          #pragma unroll
          for (int x = 0; x < 4; ++x) {
            const uint32_t qa = qf[i][x], qb = qf[i + NP][x];
            qf[i][x] = hfma2(qa, C[x], hmul2(qb, S[x]));                 // u = qa*C + qb*S
            qf[i + NP][x] = hfma2(qb, C[x], hneg2(hmul2(qa, S[x])));     // w = qb*C - qa*S
          }
        }
      }
      const float bias0 = bz[0] - bo[0], bias1 = bz[1] - bo[1];

      uint32_t ka[NW];                                           // address of this lane's word i in row g of the current tile
      #pragma unroll
      for (int i = 0; i < NW; ++i) ka[i] = TAIL ? s_k + g * (HD * 2) + 16 * (4 * i + j) : s_k + koff[i];
      uint32_t va = s_v + vrow, vsa = s_vs + 2 * g, rta = relt;
      constexpr uint32_t KROW8 = TAIL ? 8 * HD * 2 : 8 * L::ROWB;      // eight rows further down

      #pragma unroll 1
      for (int tile = 0; tile < 2; ++tile) {
        if (TAIL && tile * 16 >= nvalid) break;
        // The tile's packed words and V rows are requested up front, so their shared-memory latency overlaps the arithmetic
        // that follows (the loads are ordered asm statements: the compiler will not hoist them by itself).
        uint32_t kw[2][NW];
        if (!TAIL) {
          #pragma unroll
          for (int h = 0; h < 2; ++h)
            #pragma unroll
            for (int i = 0; i < NW; ++i) kw[h][i] = lds32(ka[i] + h * KROW8);
        }
        uint32_t vx[HD / 64][4];                                 // [load q][tokens 0-7 | 8-15 of chunk 2q, the same of chunk 2q+1]
        #pragma unroll
        for (int q = 0; q < HD / 64; ++q) ldmatrix_x4_t(va + 16 * ((2 * q + vch) ^ vsw), vx[q]);
        auto load_k = [&](int h, int i, uint32_t (&o)[4]) {     // A regs of word w = 4i+j, row g + 8h of the tile
          if (TAIL) pair_regs(lds128(ka[i] + h * KROW8), o); else nib_regs(kw[h][i], o, nk);
        };
        // ---- S^T[16 tok x 8 heads] = K . Q^T, two independent accumulation chains
        float sa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        uint32_t kr[2][NRd][4];                                  // rotary words: true value, rotated by dt
        if (RD > 0) {
          #pragma unroll
          for (int h = 0; h < 2; ++h)
            #pragma unroll
            for (int i = 0; i < NP; ++i) {
              uint32_t a4[4], b4[4];
              load_k(h, i, a4); load_k(h, i + NP, b4);
              const uint4 t0 = lds128(rta + ((h * NP + i) * 2) * 512), t1 = lds128(rta + ((h * NP + i) * 2 + 1) * 512);
              const uint32_t cd[4] = {t0.x, t0.z, t1.x, t1.z}, sd[4] = {t0.y, t0.w, t1.y, t1.w};
              #pragma unroll
              for (int x = 0; x < 4; ++x) {
                uint32_t a = a4[x], b = b4[x];
                if (!TAIL) {                                     // (off+n) - off is exact; n*scale + zero rounds once
                  const uint32_t ng = (x & 1) ? NEG_O : NEG_E;
                  a = hfma2(hadd2(a, ng), rs[i][x], rz[i][x]); b = hfma2(hadd2(b, ng), rs[i + NP][x], rz[i + NP][x]);
                }
                kr[h][i][x] = hfma2(a, cd[x], hneg2(hmul2(b, sd[x])));        // a*cd - b*sd
                kr[h][i + NP][x] = hfma2(a, sd[x], hmul2(b, cd[x]));          // a*sd + b*cd
              }
            }
        }
        #pragma unroll
        for (int i = 0; i < NW; ++i) {
          uint32_t k0[4], k1[4];
          if (i < NR) {
            #pragma unroll
            for (int x = 0; x < 4; ++x) { k0[x] = kr[0][i][x]; k1[x] = kr[1][i][x]; }
          } else { load_k(0, i, k0); load_k(1, i, k1); }
          mma16816(sa[0], k0[0], k1[0], k0[1], k1[1], qf[i][0], qf[i][1]);
          mma16816(sa[1], k0[2], k1[2], k0[3], k1[3], qf[i][2], qf[i][3]);
        }
        // ---- softmax over the tile (log2 domain); rows rg, rg+8; heads 2j, 2j+1
        const int rg = tile * 16 + g;
        const bool v0 = !TAIL || rg < nvalid, v1 = !TAIL || rg + 8 < nvalid;
        const float s00 = v0 ? sa[0][0] + sa[1][0] + bias0 : -INFINITY, s01 = v0 ? sa[0][1] + sa[1][1] + bias1 : -INFINITY;
        const float s10 = v1 ? sa[0][2] + sa[1][2] + bias0 : -INFINITY, s11 = v1 ? sa[0][3] + sa[1][3] + bias1 : -INFINITY;
        float t0 = fmaxf(s00, s10), t1 = fmaxf(s01, s11);
        if (__any_sync(0xffffffffu, t0 > m[0] + 8.f || t1 > m[1] + 8.f)) {   // lazy rescale: the running max may lag by 2^8; no shuffle unless it must move
          #pragma unroll
          for (int o = 4; o <= 16; o <<= 1) { t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, o)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, o)); }
          const float n0 = fmaxf(m[0], t0), n1 = fmaxf(m[1], t1), a0 = ex2(m[0] - n0), a1 = ex2(m[1] - n1);
          m[0] = n0; m[1] = n1; l[0] *= a0; l[1] *= a1; zacc[0] *= a0; zacc[1] *= a1; zs[0] *= a0; zs[1] *= a1; zs[2] *= a0; zs[3] *= a1;
          #pragma unroll
          for (int mt = 0; mt < HD / 16; ++mt) { acc[mt][0] *= a0; acc[mt][1] *= a1; acc[mt][2] *= a0; acc[mt][3] *= a1; }
        }
        const float p00 = v0 ? ex2(s00 - m[0]) : 0.f, p01 = v0 ? ex2(s01 - m[1]) : 0.f;
        const float p10 = v1 ? ex2(s10 - m[0]) : 0.f, p11 = v1 ? ex2(s11 - m[1]) : 0.f;
        l[0] += p00 + p10; l[1] += p01 + p11;
        // V per-token scale folded into P (fp16), zero point into a per-head scalar: v = vs*(off+n) + (vz - off*vs), off = 0 for
        // even channels (1024 subtracted exactly before the MMA) and 64 for odd ones.  The -off*vs*p part uses the sum of the
        // ROUNDED p*vs the MMA consumes (an MMA row of ones), so the offset cancels exactly; it is subtracted once, after the loop.
        const float vs0 = v0 ? lds_h(vsa) : 0.f, vz0 = v0 ? lds_h(vsa + L::UG * 64) : 0.f;
        const float vs1 = v1 ? lds_h(vsa + 16) : 0.f, vz1 = v1 ? lds_h(vsa + L::UG * 64 + 16) : 0.f;
        const uint32_t pp0 = pack_h2(p00 * vs0, p01 * vs0), pp1 = pack_h2(p10 * vs1, p11 * vs1);
        zacc[0] += p00 * vz0 + p10 * vz1;
        zacc[1] += p01 * vz0 + p11 * vz1;
        const uint32_t pb0 = movmatrix_t(pp0);                   // B regs: (tokens 2j,2j+1 | head g)
        const uint32_t pb1 = movmatrix_t(pp1);                   //         (tokens 2j+8,2j+9 | head g)
        mma16816(zs, ONE2, ONE2, ONE2, ONE2, pb0, pb1);          // every row: sum over the tile's tokens of the rounded p*vscale
        // ---- O^T += V^T P^T.  A transposed 8x8 load hands lane (g, j) the 16-bit element g of token rows 2j and 2j+1 of a
        //      16-byte chunk: four channels (4g .. 4g+3 of the chunk's 32) of two consecutive tokens, which is the pairing along
        //      the contraction that an A register wants.  Nibbles are read in place: channel 4g+0 / 4g+2 (after >> 8) as 1024 + n,
        //      made n by an exact subtraction; 4g+1 / 4g+3 as 64 + n.  MMA row g = the even channel, row g+8 = the odd one.
        #pragma unroll
        for (int q = 0; q < HD / 64; ++q)
          #pragma unroll
          for (int p = 0; p < 2; ++p) {
            const uint32_t lo = vx[q][2 * p], hi = vx[q][2 * p + 1], lo8 = lo >> 8, hi8 = hi >> 8;
            mma16816(acc[(2 * q + p) * 2], hadd2(and_or(lo, nk.m0, nk.e), NEG_E), and_or(lo, nk.m1, nk.o),
                     hadd2(and_or(hi, nk.m0, nk.e), NEG_E), and_or(hi, nk.m1, nk.o), pb0, pb1);
            mma16816(acc[(2 * q + p) * 2 + 1], hadd2(and_or(lo8, nk.m0, nk.e), NEG_E), and_or(lo8, nk.m1, nk.o),
                     hadd2(and_or(hi8, nk.m0, nk.e), NEG_E), and_or(hi8, nk.m1, nk.o), pb0, pb1);
          }
        // next tile: sixteen rows further down
        #pragma unroll
        for (int i = 0; i < NW; ++i) ka[i] += 2 * KROW8;
        va += 16 * L::ROWB; vsa += 32; rta += 2 * NP * 2 * 512;
      }
    };

    bool ok = true;
    // Slot kk = (unit kk/4 of this CTA, group kk%4 of the unit), round-robin over the consumer warps: a fixed assignment, so
    // the summation order and with it every bit of the result is the same from run to run (handing slots out from a shared
    // counter was measured: no faster with two warps per scheduler, and not reproducible).
    for (int kk = warp; kk < nu * L::UG && ok; kk += NCW) {
      const int k = kk / L::UG, sub = kk % L::UG, u = u0 + k, s = k % NSTAGE;
      const bool tail = has_tail && u == nu4;
      if (tail ? sub != 0 : u * L::UG + sub >= nq) continue;     // the unit holds fewer than four groups
      const uint32_t st = sbase + L::OFF_STAGES + s * L::STAGE;
      if (!mbar_wait(bar_full + 8 * s, (k / NSTAGE) & 1)) { atomicExch(&g_decode_status, 1); *s_abort = 1; ok = false; break; }
      if (tail) group(std::true_type{}, st, 0, len - nq * 32);
      else group(std::false_type{}, st, sub, 32);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_empty + 8 * s);             // one of the four arrivals that free the stage
    }

    // ---- all consumers done with the ring: publish per-warp (m, l, O) into the merge buffer
    #pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
      l[0] += __shfl_xor_sync(0xffffffffu, l[0], o); l[1] += __shfl_xor_sync(0xffffffffu, l[1], o);
      zacc[0] += __shfl_xor_sync(0xffffffffu, zacc[0], o); zacc[1] += __shfl_xor_sync(0xffffffffu, zacc[1], o);
    }
    const float ze[2] = {zacc[0], zacc[1]}, zo[2] = {zacc[0] - 64.f * zs[0], zacc[1] - 64.f * zs[1]};
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");  // nobody still reads a stage
    if (!*s_abort) {
      float* wb = mbuf + (size_t)warp * 8 * (HD + 2);
      if (g == 0) { wb[(2 * j) * (HD + 2)] = m[0]; wb[(2 * j) * (HD + 2) + 1] = l[0]; wb[(2 * j + 1) * (HD + 2)] = m[1]; wb[(2 * j + 1) * (HD + 2) + 1] = l[1]; }
      #pragma unroll
      for (int mt = 0; mt < HD / 16; ++mt) {
        const int c = 32 * (mt >> 1) + 4 * g + 2 * (mt & 1);           // even channel of the m-tile; the odd one is c + 1
        wb[(2 * j) * (HD + 2) + 2 + c] = acc[mt][0] + ze[0]; wb[(2 * j + 1) * (HD + 2) + 2 + c] = acc[mt][1] + ze[1];
        wb[(2 * j) * (HD + 2) + 2 + c + 1] = acc[mt][2] + zo[0]; wb[(2 * j + 1) * (HD + 2) + 2 + c + 1] = acc[mt][3] + zo[1];
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory");
    // ---- merge the consumer warps and store this split's partial (natural-log m, as the merge kernel expects)
    if (!*s_abort) {
      for (int e = ct; e < G * HD; e += NCW * 32) {
        const int h = e / HD, c = e % HD;
        float M2 = -1e30f;
        #pragma unroll
        for (int w = 0; w < NCW; ++w) M2 = fmaxf(M2, mbuf[((size_t)w * 8 + h) * (HD + 2)]);
        float L2 = 0.f, o = 0.f;
        #pragma unroll
        for (int w = 0; w < NCW; ++w) {
          const float* wb = mbuf + ((size_t)w * 8 + h) * (HD + 2);
          const float sc = wb[0] > -1e29f ? ex2(wb[0] - M2) : 0.f;
          L2 += sc * wb[1]; o += sc * wb[2 + c];
        }
        const size_t p = ((size_t)r * A.splits + split) * A.nh + kvh * G + h;
        if (c == 0) { A.pm[p] = M2 > -1e29f ? M2 * LN2 : -1e30f; A.pl[p] = L2; }
        A.pacc[p * HD + c] = o;
      }
    }
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map over a packed array viewed as [rows][rowbytes] bytes, box = 128 rows (one unit), swizzle = row width.
bool make_map(CUtensorMap* out, const void* base, uint64_t rows, int rowbytes) {
  struct Key { const void* p; uint64_t rows; int rb; bool operator==(const Key& o) const { return p == o.p && rows == o.rows && rb == o.rb; } };
  struct Hash { size_t operator()(const Key& k) const { return std::hash<const void*>()(k.p) ^ (k.rows * 1315423911u) ^ (size_t)k.rb; } };
  static std::mutex mu; static std::unordered_map<Key, CUtensorMap, Hash> cache;
  std::lock_guard<std::mutex> lk(mu);
  const Key key{base, rows, rowbytes};
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)rowbytes, rows}, strides[1] = {(cuuint64_t)rowbytes};
  const cuuint32_t box[2] = {(cuuint32_t)rowbytes, 128}, estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = rowbytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// Tensor map over the rope table viewed as one row of RD floats per 32-token group (row stride = 32 table rows), box = 4 rows.
bool make_rope_map(CUtensorMap* out, const float* rope, int rd, uint64_t groups) {
  struct Key { const void* p; uint64_t n; int rd; bool operator==(const Key& o) const { return p == o.p && n == o.n && rd == o.rd; } };
  struct Hash { size_t operator()(const Key& k) const { return std::hash<const void*>()(k.p) ^ (k.n * 2654435761u) ^ (size_t)k.rd; } };
  static std::mutex mu; static std::unordered_map<Key, CUtensorMap, Hash> cache;
  std::lock_guard<std::mutex> lk(mu);
  const Key key{rope, groups, rd};
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)rd, groups}, strides[1] = {(cuuint64_t)32 * rd * 4};
  const cuuint32_t box[2] = {(cuuint32_t)rd, 4}, estr[2] = {1, 1};
  if (fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(rope), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

template <int HD, int RD, int DT>
int launch_t(const yskn_attn_g_args& a, int g, Shard sh, int early, const yskn_kv4_ms_rows& ms, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mr, cudaStream_t st) {
  using L = Lay<HD, RD>;
  auto kern = kv4_decode_mma_kernel<HD, RD, DT>;
  static std::atomic<unsigned long long> attr{0};               // once per device, like the reference's launchers once per process
  if (first_use_on_device(attr)) {
    KV4_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    KV4_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  }
  DecodeP P{a, sh, g, early, ms};
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(a.splits, a.kvh, a.M); cfg.blockDim = dim3(NTHREADS); cfg.dynamicSmemBytes = L::TOTAL; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  KV4_CUDA(cudaLaunchKernelEx(&cfg, kern, mk, mv, mr, P));
  return launch_status("kv4_decode_mma_kernel");
}

template <int HD, int RD>
int launch_dt(const yskn_attn_g_args& a, int g, int dt, Shard sh, int early, const yskn_kv4_ms_rows& ms, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mr, cudaStream_t st) {
  if (dt == YSKN_KV4_BF16) return launch_t<HD, RD, YSKN_KV4_BF16>(a, g, sh, early, ms, mk, mv, mr, st);
  return launch_t<HD, RD, YSKN_KV4_F16>(a, g, sh, early, ms, mk, mv, mr, st);
}

}  // namespace

bool decode_mma_supports(int g, int hd, int rd, int M) {
  if (g < 1 || g > 8 || M < 1 || M > 8) return false;
  return (hd == 256 && (rd == 64 || rd == 0)) || (hd == 128 && (rd == 128 || rd == 0));
}

// Uploads the table of per-sequence cache arrays and their K / V tensor maps for yskn_kv4_attention_ms (set-up: it copies from host memory).
int ms_prepare(const yskn_kv_layer* h_layers, int n_slots, int kvh, int hd, int max_ctx, yskn_kv_layer* d_layers, void* d_maps, cudaStream_t st) {
  if (!h_layers || !d_layers || !d_maps || n_slots <= 0 || n_slots > 64) KV4_REJECT("yskn_kv4_ms_prepare: bad arguments (n_slots %d)", n_slots);
  if (kvh <= 0 || (hd != 128 && hd != 256) || max_ctx <= 0 || max_ctx % 64) KV4_REJECT("yskn_kv4_ms_prepare: bad shape (kvh %d, hd %d, max_ctx %d)", kvh, hd, max_ctx);
  if ((uintptr_t)d_maps & 127) KV4_REJECT("yskn_kv4_ms_prepare: the map table must be 128-byte aligned");
  std::vector<CUtensorMap> maps(2 * (size_t)n_slots);
  const uint64_t rows = (uint64_t)kvh * max_ctx;
  for (int s = 0; s < n_slots; ++s) {
    const yskn_kv_layer& l = h_layers[s];
    const uintptr_t al = (uintptr_t)l.kq | (uintptr_t)l.vq | (uintptr_t)l.kscale | (uintptr_t)l.kzero | (uintptr_t)l.kshadow | (uintptr_t)l.vscale | (uintptr_t)l.vzero;
    if (!l.kq || !l.vq || !l.kscale || !l.kzero || !l.kshadow || !l.vscale || !l.vzero || (al & 15))
      KV4_REJECT("yskn_kv4_ms_prepare: cache arrays of slot %d missing or not 16-byte aligned", s);
    if (!make_map(&maps[2 * s], l.kq, rows, hd / 2) || !make_map(&maps[2 * s + 1], l.vq, rows, hd / 2))
      KV4_REJECT("yskn_kv4_ms_prepare: cuTensorMapEncodeTiled failed or is unavailable");
  }
  KV4_CUDA(cudaMemcpyAsync(d_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, st));
  KV4_CUDA(cudaMemcpyAsync(d_layers, h_layers, (size_t)n_slots * sizeof(yskn_kv_layer), cudaMemcpyHostToDevice, st));
  KV4_CUDA(cudaStreamSynchronize(st));                            // the host vectors go out of scope
  return 0;
}

int launch_decode_mma(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, Shard sh, int early, cudaStream_t st,
                      const yskn_kv4_ms_rows* ms) {
  const bool multi = ms != nullptr;
  if (multi ? !decode_mma_supports(g, hd, rd, 1) || a.M < 1 || a.M > 64 : !decode_mma_supports(g, hd, rd, a.M))
    KV4_REJECT("yskn_kv4_attention: tensor-core decode does not cover (g %d, hd %d, rd %d, M %d)", g, hd, rd, a.M);
  const uintptr_t al = multi ? (uintptr_t)a.rope
                             : (uintptr_t)a.kv.kq | (uintptr_t)a.kv.vq | (uintptr_t)a.kv.kscale | (uintptr_t)a.kv.kzero | (uintptr_t)a.kv.kshadow |
                               (uintptr_t)a.kv.vscale | (uintptr_t)a.kv.vzero | (uintptr_t)a.rope;
  if (al & 15) KV4_REJECT("yskn_kv4_attention: cache arrays and rope table must be 16-byte aligned");
  CUtensorMap mk, mv, mr;
  const uint64_t rows = (uint64_t)a.kvh * a.max_ctx;
  if (multi) { memset(&mk, 0, sizeof(mk)); memset(&mv, 0, sizeof(mv)); }      // the kernel takes the maps of the row's sequence from ms->maps
  else if (!make_map(&mk, a.kv.kq, rows, hd / 2) || !make_map(&mv, a.kv.vq, rows, hd / 2))
    KV4_REJECT("yskn_kv4_attention: cuTensorMapEncodeTiled failed or is unavailable");
  const yskn_kv4_ms_rows msv = multi ? *ms : yskn_kv4_ms_rows{nullptr, nullptr, nullptr, nullptr, 0};
  if (multi) early = 0;                                           // rows of one sequence in the same pass are appended by the predecessor
  // The rope table must cover positions [0, shard start + shard length); groups past that read as zero and are never used.
  if (rd == 0) mr = mk;
  else if (!make_rope_map(&mr, a.rope, rd, ((uint64_t)sh.start + (uint64_t)sh.len) / 32))
    KV4_REJECT("yskn_kv4_attention: cuTensorMapEncodeTiled failed for the rope table");
  if (hd == 256) return rd ? launch_dt<256, 64>(a, g, act_dtype, sh, early, msv, mk, mv, mr, st) : launch_dt<256, 0>(a, g, act_dtype, sh, early, msv, mk, mv, mr, st);
  return rd ? launch_dt<128, 128>(a, g, act_dtype, sh, early, msv, mk, mv, mr, st) : launch_dt<128, 0>(a, g, act_dtype, sh, early, msv, mk, mv, mr, st);
}

int decode_status_fetch(int* out) {
  int v = 0;
  KV4_CUDA(cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)));
  const int zero = 0;
  KV4_CUDA(cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int)));
  *out = v; return 0;
}

}  // namespace kv4
