// Log-sum-exp merge of split-K partials (sm_100a).
//
// Restates the merge half of the reference's attn_combine_gqa_xform_kernel (src/attention_gqa.cu:123-134):
//   M2 = max_s pm;  w_s = pm > -1e29 ? exp(pm - M2) : 0;  L = sum w_s*pl;  o = sum w_s*pacc (in split order);
//   y = round_f16(o / L);  y += bv[kvh][d];  y *= sigmoid(gate);  store 16-bit.
// The same kernel, with other index maps, folds one shard's partials into an un-normalised (m, l, O) triple
// and merges the triples gathered from all shards of a sequence-sharded decode.
//
// One block per (head, row), one thread per channel: the pacc reads of a block are `splits` contiguous
// HD*4-byte rows, the weights are computed once per block into shared memory.
#include "kv4_common.cuh"

namespace kv4 {
namespace {

struct CombineP {
  const float* pm; const float* pl; const float* pacc;   // partial layout  [M][S][nh] / [M][S][nh][HD]
  const float* triples;                                  // triple layout   [S][M][nh][HD+2]
  int S, M, nh, g;
  const void* bv; const void* gate; uint16_t* o16; float* triple_out;
};

template <int HD, int DT, bool TRIPLE_IN, bool TRIPLE_OUT>
__global__ void __launch_bounds__(HD) kv4_combine_kernel(CombineP P) {
  extern __shared__ float sm[];                          // [S] m, [S] l, [S] w
  float* s_m = sm; float* s_l = sm + P.S; float* s_w = sm + 2 * P.S;
  const int head = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
  auto slot = [&](int s) -> size_t { return TRIPLE_IN ? (((size_t)s * P.M + r) * P.nh + head) * (HD + 2)
                                                      : ((size_t)r * P.S + s) * P.nh + head; };
  for (int s = d; s < P.S; s += HD) {
    if (TRIPLE_IN) { s_m[s] = P.triples[slot(s)]; s_l[s] = P.triples[slot(s) + 1]; }
    else { s_m[s] = P.pm[slot(s)]; s_l[s] = P.pl[slot(s)]; }
  }
  __syncthreads();
  float M2 = -1e30f;
  for (int s = 0; s < P.S; ++s) M2 = fmaxf(M2, s_m[s]);
  for (int s = d; s < P.S; s += HD) s_w[s] = (s_m[s] > -1e29f) ? expf(s_m[s] - M2) : 0.f;
  __syncthreads();
  float L2 = 0.f, o = 0.f;
  #pragma unroll 4
  for (int s = 0; s < P.S; ++s) {
    const float w = s_w[s];
    const float a = TRIPLE_IN ? P.triples[slot(s) + 2 + d] : P.pacc[slot(s) * HD + d];
    L2 += w * s_l[s]; o += w * a;
  }
  if (TRIPLE_OUT) {
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
}

template <bool TI, bool TO> int launch_p(const CombineP& P, int hd, int dt, cudaStream_t st, const char* who) {
  if (P.S <= 0 || P.M <= 0 || P.nh <= 0 || P.g <= 0) KV4_REJECT("%s: bad arguments (splits %d, M %d, nh %d, g %d)", who, P.S, P.M, P.nh, P.g);
  const dim3 grid(P.nh, P.M); const size_t smem = (size_t)3 * P.S * sizeof(float);
  if (smem > 48 * 1024) KV4_REJECT("%s: too many partials per row (%d)", who, P.S);
#define KV4_GO(HD_, DT_) kv4_combine_kernel<HD_, DT_, TI, TO><<<grid, HD_, smem, st>>>(P)
  const bool bf = dt == YSKN_KV4_BF16;
  if (dt != YSKN_KV4_F16 && dt != YSKN_KV4_BF16) KV4_REJECT("%s: act_dtype must be F16 or BF16", who);
  if (hd == 256) { if (bf) KV4_GO(256, YSKN_KV4_BF16); else KV4_GO(256, YSKN_KV4_F16); }
  else if (hd == 128) { if (bf) KV4_GO(128, YSKN_KV4_BF16); else KV4_GO(128, YSKN_KV4_F16); }
  else if (hd == 64) { if (bf) KV4_GO(64, YSKN_KV4_BF16); else KV4_GO(64, YSKN_KV4_F16); }
  else KV4_REJECT("%s: unsupported head_dim %d (64, 128, 256)", who, hd);               // src/attention_gqa.cu:180
#undef KV4_GO
  return launch_status(who);
}

}  // namespace

int launch_combine(const yskn_attn_g_combine_args& a, int hd, int act_dtype, cudaStream_t st) {
  if (!a.pm || !a.pl || !a.pacc || !a.o16) KV4_REJECT("yskn_kv4_combine: null buffer");
  CombineP P{a.pm, a.pl, a.pacc, nullptr, a.splits, a.M, a.nh, a.g, a.bv, a.gate, a.o16, nullptr};
  return launch_p<false, false>(P, hd, act_dtype, st, "yskn_kv4_combine");
}

int launch_local_triple(const yskn_attn_g_combine_args& a, int hd, float* d_triple, cudaStream_t st) {
  if (!a.pm || !a.pl || !a.pacc || !d_triple) KV4_REJECT("yskn_kv4_local_triple: null buffer");
  CombineP P{a.pm, a.pl, a.pacc, nullptr, a.splits, a.M, a.nh, a.g > 0 ? a.g : 1, nullptr, nullptr, nullptr, d_triple};
  return launch_p<false, true>(P, hd, YSKN_KV4_F16, st, "yskn_kv4_local_triple");
}

int launch_merge_triples(const float* d_triples, int ranks, int M, int nh, int g, int hd, const uint16_t* bv,
                         const uint16_t* gate, uint16_t* o16, int act_dtype, cudaStream_t st) {
  if (!d_triples || !o16) KV4_REJECT("yskn_kv4_merge_triples: null buffer");
  CombineP P{nullptr, nullptr, nullptr, d_triples, ranks, M, nh, g, bv, gate, o16, nullptr};
  return launch_p<true, false>(P, hd, act_dtype, st, "yskn_kv4_merge_triples");
}

}  // namespace kv4
