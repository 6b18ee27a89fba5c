// Log-sum-exp merge of split-K partials (sm_100a).
//
// Restates the merge half of the reference's attn_combine_gqa_xform_kernel (src/attention_gqa.cu:123-134):
//   M2 = max_s pm;  w_s = pm > -1e29 ? exp(pm - M2) : 0;  L = sum w_s*pl;  o = sum w_s*pacc;
//   y = round_f16(o / L);  y += bv[kvh][d];  y *= sigmoid(gate);  store 16-bit.
// The same kernel, with other index maps, folds one shard's partials into an un-normalised (m, l, O) triple and
// merges the triples gathered from all shards of a sequence-sharded decode.
//
// The kernel is pure latency: a few hundred KB read once.  One block per (head, row) with 4*HD threads: thread
// (q, d) owns channel d and a quarter of the splits, issues its pacc loads before anything else so that they and the
// pm/pl loads are one round trip to L2, then the quarters are added in fixed order (0,1,2,3).  The sum over splits is
// therefore grouped in four runs rather than strictly sequential as in the reference; the result is deterministic.
// The launch carries the programmatic-stream-serialization attribute (the reference's PDL launches,
// src/pdl.cuh:23-30): the grid may be scheduled while the attention kernel drains and waits in griddepcontrol.wait.
#include "kv4_common.cuh"

namespace kv4 {
namespace {

struct CombineP {
  const float* pm; const float* pl; const float* pacc;   // partial layout  [M][S][nh] / [M][S][nh][HD]
  const float* triples;                                  // triple layout   [S][M][nh][HD+2]
  int S, M, nh, g;
  const void* bv; const void* gate; uint16_t* o16; float* triple_out;
  yskn_kv4_peer_exchange x;                              // PEER modes only
  unsigned wait_polls;                                   // PEER modes: polls (about 100 ns each) before a wait gives up
};

__device__ int g_merge_status = 0;                       // 7 = the wait for the other shards' triples ran out

// Exchange buffer of one rank (yskn_kv4_peer_exchange): uint2 slot[2][world][M*nh*(HD+2)], then int step, unsigned merge
// ticket.  A slot is one float of a triple together with the number of the step that wrote it, stored with ONE 8-byte
// store (delivered whole over NVLink), so a reader that finds the step's tag has the value: no fence, no arrival counter,
// one network latency.  Half `step & 1` is the one in use; a rank is never more than one step ahead of another, so a
// half is rewritten only after every rank has read it.
__device__ __forceinline__ size_t xch_data_floats(int world, int M, int nh, int hd) { return (size_t)2 * world * M * nh * (hd + 2) * 2; }
__device__ __forceinline__ void st_slot(float* base, size_t i, float v, unsigned tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(reinterpret_cast<uint2*>(base) + i), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_slot(const float* base, size_t i) {
  uint2 v; asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(reinterpret_cast<const uint2*>(base) + i) : "memory");
  return v;
}
constexpr unsigned PEER_WAIT_POLLS = 1u << 20;           // default limit, x ~0.5 us per poll round: about half a second
std::atomic<unsigned> g_peer_wait_polls{PEER_WAIT_POLLS}; // yskn_kv4_set_peer_wait_polls

constexpr int CB = 10;                                   // loads in flight per thread and batch: 4 runs x 10 cover 37-40 splits in one round trip

// PEER: with TRIPLE_OUT, the triple goes into every rank's exchange buffer (8-byte value+tag stores through NVLink peer
// mappings); with TRIPLE_IN, every thread polls (bounded) the slots it needs -- (m, l) of each rank and its own channel of
// each rank's O -- until they carry this step's tag, and the last block of the grid opens the next step.
// CQ = split runs per block: 4 when there are many splits to fetch and few blocks (decode: latency), 2 when the grid of
// 1,024-thread blocks would not fit the GPU at once (verify: hundreds of rows x heads), 1 for short sums (prefill).
template <int HD, int DT, bool TRIPLE_IN, bool TRIPLE_OUT, bool PEER, int CQ>
__global__ void __launch_bounds__(CQ * HD) kv4_combine_kernel(CombineP P) {
  // TRIPLE_IN && TRIPLE_OUT && PEER = the fused exchange: fold the splits, push the triple, wait for the other ranks' triples, merge.
  constexpr bool FUSED = TRIPLE_IN && TRIPLE_OUT && PEER, READ_TRIPLES = TRIPLE_IN && !FUSED;
  extern __shared__ float sm[];                          // [S] m, [S] l, [S] w, [CQ][HD] partial sums
  float* s_m = sm; float* s_l = sm + P.S; float* s_w = sm + 2 * P.S; float* s_part = sm + 3 * P.S;
  const int head = blockIdx.x, r = blockIdx.y, tid = threadIdx.x, q = tid / HD, d = tid % HD;
  const int per = (P.S + CQ - 1) / CQ, s0 = min(P.S, q * per), s1 = min(P.S, s0 + per);
  auto slot = [&](int s) -> size_t { return READ_TRIPLES ? (((size_t)s * P.M + r) * P.nh + head) * (HD + 2)
                                                      : ((size_t)r * P.S + s) * P.nh + head; };
  auto ld_acc = [&](int s) -> float { return READ_TRIPLES ? __ldcg(P.triples + slot(s) + 2 + d) : __ldcg(P.pacc + slot(s) * HD + d); };
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next step's attention grid may be scheduled; it waits for this one
  asm volatile("griddepcontrol.wait;" ::: "memory");     // the producer grid's writes are visible from here on
  __shared__ int s_bad;
  int par = 0;                                           // which half of the exchange buffers this step uses
  unsigned tag = 0;                                      // this step's number + 1 (a zero-filled buffer carries tag 0)
  const size_t xdata = PEER ? xch_data_floats(P.x.world, P.M, P.nh, HD) : 0;    // floats: two per slot
  const size_t xhalf = xdata / 4;                        // slots of one half
  if (PEER) {
    const int step = *reinterpret_cast<volatile int*>(P.x.buf[P.x.rank] + xdata);
    par = step & 1; tag = (unsigned)step + 1u;
  }
  // Polls (bounded) until this step's tag is on the slots this thread is responsible for: its channel of every rank's O,
  // and -- threads 0 .. 2*world-1 -- one rank's m or l, which go to shared memory for the whole block.  Call with the HD
  // threads of run 0 only; false = some thread of the block gave up (device status 7).
  __shared__ float s_tm[8], s_tl[8];
  auto poll_triples = [&](float (&tm)[8], float (&tl)[8], float (&to)[8]) -> bool {
    const float* mine = P.x.buf[P.x.rank];
    const size_t base = (size_t)par * xhalf + ((size_t)r * P.nh + head) * (HD + 2), rstride = (size_t)P.M * P.nh * (HD + 2);
    const unsigned all = (1u << P.x.world) - 1u;
    const bool ml = d < 2 * P.x.world;                   // this thread also fetches m (even d) or l (odd d) of rank d/2
    unsigned have = 0;                                   // bit src: O slot seen; bit 8: the m/l slot seen
    int ok = 1;
    for (unsigned polls = 0; ; ++polls) {
      uint2 c[8], e = make_uint2(0u, tag);
      #pragma unroll
      for (int src = 0; src < 8; ++src) c[src] = ld_slot(mine, base + (size_t)min(src, P.x.world - 1) * rstride + 2 + d);   // all loads in flight at once
      if (ml) e = ld_slot(mine, base + (size_t)(d >> 1) * rstride + (d & 1));
      #pragma unroll
      for (int src = 0; src < 8; ++src) if (src < P.x.world && c[src].y == tag) { have |= 1u << src; to[src] = __uint_as_float(c[src].x); }
      if (e.y == tag) { have |= 256u; if (ml) { if (d & 1) s_tl[d >> 1] = __uint_as_float(e.x); else s_tm[d >> 1] = __uint_as_float(e.x); } }
      if (have == (all | 256u)) break;
      if (polls > P.wait_polls) { atomicExch(&g_merge_status, 7); ok = 0; break; }
      __nanosleep(64);
    }
    if (d == 0) s_bad = 0;
    asm volatile("bar.sync 1, %0;" ::"n"(HD) : "memory");
    if (!ok) s_bad = 1;
    asm volatile("bar.sync 1, %0;" ::"n"(HD) : "memory");      // also: s_tm / s_tl are complete
    if (s_bad) return false;
    #pragma unroll
    for (int src = 0; src < 8; ++src) {
      if (src < P.x.world) { tm[src] = s_tm[src]; tl[src] = s_tl[src]; }
      else { tm[src] = -1e30f; tl[src] = 0.f; to[src] = 0.f; }
    }
    return true;
  };
  auto merge_triples = [&](const float (&tm)[8], const float (&tl)[8], const float (&to)[8], float& o_out, float& l_out) {
    float Mw = -1e30f;
    #pragma unroll
    for (int src = 0; src < 8; ++src) Mw = fmaxf(Mw, tm[src]);
    float Lw = 0.f, ow = 0.f;
    #pragma unroll
    for (int src = 0; src < 8; ++src) { const float wgt = tm[src] > -1e29f ? expf(tm[src] - Mw) : 0.f; Lw += wgt * tl[src]; ow += wgt * to[src]; }
    o_out = ow; l_out = Lw;
  };
  if (PEER && READ_TRIPLES) {                            // merge of pushed triples: nothing to fold, only HD threads work
    if (q != 0) return;
    float tm[8], tl[8], to[8], o, L2;
    if (!poll_triples(tm, tl, to)) return;               // some thread of the block gave up: no row from incomplete triples
    merge_triples(tm, tl, to, o, L2);
    float y = round_f16(o / L2);
    const size_t e = ((size_t)r * P.nh + head) * HD + d;
    if (P.bv) y = __fadd_rn(y, act_load<DT>(P.bv, (size_t)(head / P.g) * HD + d));
    if (P.gate) { const float gt = act_load<DT>(P.gate, e); y = __fmul_rn(y, __fdiv_rn(1.f, __fadd_rn(1.f, expf(-gt)))); }
    P.o16[e] = act_store16<DT>(y);
    asm volatile("bar.sync 1, %0;" ::"n"(HD) : "memory");      // every thread of the block has read its slots
    if (d == 0) {
      unsigned* ticket = reinterpret_cast<unsigned*>(P.x.buf[P.x.rank] + xdata) + 1;
      if (atomicAdd(ticket, 1u) == gridDim.x * gridDim.y - 1) {
        *ticket = 0u;
        __threadfence();
        volatile int* step = reinterpret_cast<volatile int*>(P.x.buf[P.x.rank] + xdata);
        *step = *step + 1;                             // every block of this grid has read it already
      }
    }
    return;
  }

  float v[CB];                                           // first batch of this thread's values: in flight with pm/pl
  #pragma unroll
  for (int k = 0; k < CB; ++k) v[k] = s0 + k < s1 ? ld_acc(s0 + k) : 0.f;
  for (int s = tid; s < P.S; s += CQ * HD) {
    if (READ_TRIPLES) { s_m[s] = __ldcg(P.triples + slot(s)); s_l[s] = __ldcg(P.triples + slot(s) + 1); }
    else { s_m[s] = __ldcg(P.pm + slot(s)); s_l[s] = __ldcg(P.pl + slot(s)); }
  }
  __syncthreads();
  // One warp forms the maximum, the weights and the weighted sum of l (lane-strided, then a fixed shuffle tree: the same
  // bits on every run); the other threads only wait for their loads meanwhile.
  __shared__ float s_M2, s_L2;
  if (tid < 32) {
    float mx = -1e30f;
    for (int s = tid; s < P.S; s += 32) mx = fmaxf(mx, s_m[s]);
    #pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float ls = 0.f;
    for (int s = tid; s < P.S; s += 32) { const float w = (s_m[s] > -1e29f) ? expf(s_m[s] - mx) : 0.f; s_w[s] = w; ls += w * s_l[s]; }
    #pragma unroll
    for (int o = 16; o; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
    if (tid == 0) { s_M2 = mx; s_L2 = ls; }
  }
  __syncthreads();
  const float M2 = s_M2;
  float o = 0.f;
  #pragma unroll
  for (int k = 0; k < CB; ++k) if (s0 + k < s1) o += s_w[s0 + k] * v[k];
  for (int sb = s0 + CB; sb < s1; sb += CB) {            // more than 4*CB splits: further batches
    #pragma unroll
    for (int k = 0; k < CB; ++k) v[k] = sb + k < s1 ? ld_acc(sb + k) : 0.f;
    #pragma unroll
    for (int k = 0; k < CB; ++k) if (sb + k < s1) o += s_w[sb + k] * v[k];
  }
  s_part[q * HD + d] = o;
  __syncthreads();
  if (q != 0) return;
  if (CQ == 4) o = (s_part[d] + s_part[HD + d]) + (s_part[2 * HD + d] + s_part[3 * HD + d]);
  if (CQ == 2) o = s_part[d] + s_part[HD + d];
  float L2 = s_L2;
  if (TRIPLE_OUT && PEER) {
    const size_t off = (size_t)par * xhalf + (((size_t)P.x.rank * P.M + r) * P.nh + head) * (HD + 2);
    for (int w = 0; w < P.x.world; ++w) {
      float* t = P.x.buf[w];
      if (d == 0) { st_slot(t, off, M2, tag); st_slot(t, off + 1, L2, tag); }
      st_slot(t, off + 2 + d, o, tag);
    }
    if (!FUSED) return;
    // ---- fused: every thread waits for its slots of all ranks' triples (the grid is small enough to be resident as a
    //      whole, so blocks that wait cannot keep a block that still has to push off the GPU), then merges them
    float tm[8], tl[8], to[8];
    if (!poll_triples(tm, tl, to)) return;
    merge_triples(tm, tl, to, o, L2);
  }
  if (TRIPLE_OUT && !FUSED) {
    float* t = P.triple_out + ((size_t)r * P.nh + head) * (HD + 2);
    if (d == 0) { t[0] = M2; t[1] = L2; }
    t[2 + d] = o;
    return;
  }
  float y = round_f16(o / L2);
  const size_t e = ((size_t)r * P.nh + head) * HD + d;
  if (P.bv) y = __fadd_rn(y, act_load<DT>(P.bv, (size_t)(head / P.g) * HD + d));
  if (P.gate) { const float gt = act_load<DT>(P.gate, e); y = __fmul_rn(y, __fdiv_rn(1.f, __fadd_rn(1.f, expf(-gt)))); }
  P.o16[e] = act_store16<DT>(y);
  if (PEER && TRIPLE_IN) {                               // the last block of the grid closes this step
    asm volatile("bar.sync 1, %0;" ::"n"(HD) : "memory");      // every thread of the block has read its triples
    if (d == 0) {
      unsigned* ticket = reinterpret_cast<unsigned*>(P.x.buf[P.x.rank] + xdata) + 1;
      if (atomicAdd(ticket, 1u) == gridDim.x * gridDim.y - 1) {
        *ticket = 0u;
        __threadfence();
        volatile int* step = reinterpret_cast<volatile int*>(P.x.buf[P.x.rank] + xdata);
        *step = *step + 1;                             // every block of this grid has read it already
      }
    }
  }
}

template <int HD, int DT, bool TI, bool TO, bool PEER>
int launch_k(const CombineP& P, size_t smem, cudaStream_t st) {
  const long long blocks = (long long)P.nh * P.M;
  const int CQ = (P.S < 8 || (TI && !TO && PEER)) ? 1 : (blocks <= 296 ? 4 : 2);   // 296 = two 1,024-thread blocks on each of 148 SMs; the merge of pushed triples folds nothing
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(P.nh, P.M); cfg.blockDim = dim3(CQ * HD); cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  if (CQ == 4) KV4_CUDA(cudaLaunchKernelEx(&cfg, kv4_combine_kernel<HD, DT, TI, TO, PEER, 4>, P));
  else if (CQ == 2) KV4_CUDA(cudaLaunchKernelEx(&cfg, kv4_combine_kernel<HD, DT, TI, TO, PEER, 2>, P));
  else KV4_CUDA(cudaLaunchKernelEx(&cfg, kv4_combine_kernel<HD, DT, TI, TO, PEER, 1>, P));
  return 0;
}

template <bool TI, bool TO, bool PEER = false> int launch_p(const CombineP& P, int hd, int dt, cudaStream_t st, const char* who) {
  if (P.S <= 0 || P.M <= 0 || P.nh <= 0 || P.g <= 0) KV4_REJECT("%s: bad arguments (splits %d, M %d, nh %d, g %d)", who, P.S, P.M, P.nh, P.g);
  if (P.M > 65535) KV4_REJECT("%s: M %d exceeds the grid limit", who, P.M);
  const size_t smem = ((size_t)3 * P.S + (size_t)4 * hd) * sizeof(float);
  if (smem > 48 * 1024) KV4_REJECT("%s: too many partials per row (%d)", who, P.S);
  const bool bf = dt == YSKN_KV4_BF16;
  if (dt != YSKN_KV4_F16 && dt != YSKN_KV4_BF16) KV4_REJECT("%s: act_dtype must be F16 or BF16", who);
  int rc;
  if (hd == 256) rc = bf ? launch_k<256, YSKN_KV4_BF16, TI, TO, PEER>(P, smem, st) : launch_k<256, YSKN_KV4_F16, TI, TO, PEER>(P, smem, st);
  else if (hd == 128) rc = bf ? launch_k<128, YSKN_KV4_BF16, TI, TO, PEER>(P, smem, st) : launch_k<128, YSKN_KV4_F16, TI, TO, PEER>(P, smem, st);
  else if (hd == 64) rc = bf ? launch_k<64, YSKN_KV4_BF16, TI, TO, PEER>(P, smem, st) : launch_k<64, YSKN_KV4_F16, TI, TO, PEER>(P, smem, st);
  else KV4_REJECT("%s: unsupported head_dim %d (64, 128, 256)", who, hd);               // src/attention_gqa.cu:180
  if (rc) return rc;
  return launch_status(who);
}

}  // namespace

int launch_combine(const yskn_attn_g_combine_args& a, int hd, int act_dtype, cudaStream_t st) {
  if (!a.pm || !a.pl || !a.pacc || !a.o16) KV4_REJECT("yskn_kv4_combine: null buffer");
  CombineP P{a.pm, a.pl, a.pacc, nullptr, a.splits, a.M, a.nh, a.g, a.bv, a.gate, a.o16, nullptr, {}, 0u};
  return launch_p<false, false>(P, hd, act_dtype, st, "yskn_kv4_combine");
}

int launch_local_triple(const yskn_attn_g_combine_args& a, int hd, float* d_triple, cudaStream_t st) {
  if (!a.pm || !a.pl || !a.pacc || !d_triple) KV4_REJECT("yskn_kv4_local_triple: null buffer");
  CombineP P{a.pm, a.pl, a.pacc, nullptr, a.splits, a.M, a.nh, a.g > 0 ? a.g : 1, nullptr, nullptr, nullptr, d_triple, {}, 0u};
  return launch_p<false, true>(P, hd, YSKN_KV4_F16, st, "yskn_kv4_local_triple");
}

int launch_merge_triples(const float* d_triples, int ranks, int M, int nh, int g, int hd, const uint16_t* bv,
                         const uint16_t* gate, uint16_t* o16, int act_dtype, cudaStream_t st) {
  if (!d_triples || !o16) KV4_REJECT("yskn_kv4_merge_triples: null buffer");
  CombineP P{nullptr, nullptr, nullptr, d_triples, ranks, M, nh, g, bv, gate, o16, nullptr, {}, 0u};
  return launch_p<true, false>(P, hd, act_dtype, st, "yskn_kv4_merge_triples");
}

static int check_exchange(const yskn_kv4_peer_exchange* x, const char* who) {
  if (!x || x->world < 1 || x->world > 8 || x->rank < 0 || x->rank >= x->world) KV4_REJECT("%s: bad exchange descriptor", who);
  for (int w = 0; w < x->world; ++w) if (!x->buf[w] || ((uintptr_t)x->buf[w] & 15)) KV4_REJECT("%s: exchange buffer %d missing or misaligned", who, w);
  return 0;
}

size_t exchange_bytes(int world, int M, int nh, int hd) {
  return ((size_t)2 * world * M * nh * (hd + 2)) * 8 + 16;   // value+tag slots of both halves, then step, merge ticket, pad
}

int launch_push_triple(const yskn_attn_g_combine_args& a, int hd, const yskn_kv4_peer_exchange* x, cudaStream_t st) {
  if (int rc = check_exchange(x, "yskn_kv4_push_triple")) return rc;
  if (!a.pm || !a.pl || !a.pacc) KV4_REJECT("yskn_kv4_push_triple: null buffer");
  CombineP P{a.pm, a.pl, a.pacc, nullptr, a.splits, a.M, a.nh, a.g > 0 ? a.g : 1, nullptr, nullptr, nullptr, nullptr, *x, g_peer_wait_polls.load()};
  return launch_p<false, true, true>(P, hd, YSKN_KV4_F16, st, "yskn_kv4_push_triple");
}

int launch_merge_pushed(const yskn_kv4_peer_exchange* x, int M, int nh, int g, int hd, const uint16_t* bv, const uint16_t* gate,
                        uint16_t* o16, int act_dtype, cudaStream_t st) {
  if (int rc = check_exchange(x, "yskn_kv4_merge_pushed")) return rc;
  if (!o16) KV4_REJECT("yskn_kv4_merge_pushed: null output");
  CombineP P{nullptr, nullptr, nullptr, nullptr, x->world, M, nh, g, bv, gate, o16, nullptr, *x, g_peer_wait_polls.load()};
  return launch_p<true, false, true>(P, hd, act_dtype, st, "yskn_kv4_merge_pushed");
}

// One launch for the whole exchange: fold this shard's splits, push the triple to every rank, wait for theirs, merge.
// Every block waits inside the kernel, so the grid must be resident as a whole: nh * M blocks of up to 1,024 threads.
int launch_exchange_merge(const yskn_attn_g_combine_args& a, int hd, int act_dtype, const yskn_kv4_peer_exchange* x, cudaStream_t st) {
  if (int rc = check_exchange(x, "yskn_kv4_exchange_merge")) return rc;
  if (!a.pm || !a.pl || !a.pacc || !a.o16) KV4_REJECT("yskn_kv4_exchange_merge: null buffer");
  int dev = 0, sms = 0;
  KV4_CUDA(cudaGetDevice(&dev));
  KV4_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if ((long long)a.nh * a.M > sms)
    KV4_REJECT("yskn_kv4_exchange_merge: nh * M = %lld blocks may not all be resident on %d SMs; use yskn_kv4_push_triple + yskn_kv4_merge_pushed", (long long)a.nh * a.M, sms);
  CombineP P{a.pm, a.pl, a.pacc, nullptr, a.splits, a.M, a.nh, a.g > 0 ? a.g : 1, a.bv, a.gate, a.o16, nullptr, *x, g_peer_wait_polls.load()};
  return launch_p<true, true, true>(P, hd, act_dtype, st, "yskn_kv4_exchange_merge");
}

void set_peer_wait_polls(unsigned polls) { g_peer_wait_polls.store(polls ? polls : PEER_WAIT_POLLS); }

int merge_status_fetch(int* out) {
  int v = 0;
  KV4_CUDA(cudaMemcpyFromSymbol(&v, g_merge_status, sizeof(int)));
  const int zero = 0;
  KV4_CUDA(cudaMemcpyToSymbol(g_merge_status, &zero, sizeof(int)));
  *out = v; return 0;
}

}  // namespace kv4
