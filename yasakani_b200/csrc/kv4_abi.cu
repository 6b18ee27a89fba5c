// extern "C" surface of the KV4 attention library: argument checks, kernel selection, error text.
// Entry points mirror the reference's launcher set (see include/yskn_kv4_abi.h for file:line of each).
#include "kv4_common.cuh"
#include <cstdarg>
#include <cstring>
#include <vector>

#define KV4_STR2(x) #x
#define KV4_STR(x) KV4_STR2(x)

namespace kv4 {

static thread_local char g_err[512] = "";
static std::atomic<int> g_algo{ALGO_AUTO};
// Per-device workspace that lets the plain entries take the tcgen05 kernel for wide passes (yskn_kv4_set_tc_workspace).
static std::atomic<void*> g_tc_ws[64];
static std::atomic<size_t> g_tc_ws_bytes[64];
int current_algo() { return g_algo.load(std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap; va_start(ap, fmt); vsnprintf(g_err, sizeof(g_err), fmt, ap); va_end(ap);
}

static int check_attn(const yskn_attn_g_args* a, int g, int hd, const char* who) {
  if (!a) KV4_REJECT("%s: null argument struct", who);
  if (!a->q16 || !a->d_pos || !a->pm || !a->pl || !a->pacc) KV4_REJECT("%s: null buffer", who);
  if (!a->kv.kq || !a->kv.kscale || !a->kv.kzero || !a->kv.kshadow || !a->kv.vq || !a->kv.vscale || !a->kv.vzero)
    KV4_REJECT("%s: null cache array", who);
  if (a->M <= 0 || a->splits <= 0 || a->kvh <= 0 || g <= 0 || a->nh != a->kvh * g)
    KV4_REJECT("%s: bad shape (M %d, splits %d, kvh %d, nh %d, g %d)", who, a->M, a->splits, a->kvh, a->nh, g);
  if (a->max_ctx <= 0 || a->max_ctx % 64) KV4_REJECT("%s: max_ctx %d is not a positive multiple of 64", who, a->max_ctx);
  if (a->splits > 65535 || a->M > 65535) KV4_REJECT("%s: splits %d / M %d exceed the grid limit", who, a->splits, a->M);
  (void)hd; return 0;
}

static int attention_dispatch(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, Shard sh, cudaStream_t st,
                              const yskn_kv4_attn_ext* x = nullptr) {
  if (act_dtype != YSKN_KV4_F16 && act_dtype != YSKN_KV4_BF16) KV4_REJECT("yskn_kv4_attention: act_dtype must be F16 or BF16");
  const int early = x ? (x->early != 0) : 0;
  if (x && (x->splits_short < 0 || x->splits_short > a->splits || (x->splits_short > 0 && x->long_len <= 0)))
    KV4_REJECT("yskn_kv4_attention: splits_short %d / long_len %d do not fit splits %d", x->splits_short, x->long_len, a->splits);
  // A row -> depth table or per-row split counts: the CUDA-core kernel partitions keys per row and implements both; the
  // tensor-core kernels partition per pass and take the plain causal pass only.
  if (x && (x->wk || x->splits_short > 0)) {
    if (x->wk && (sh.start != 0 || sh.len != a->max_ctx)) KV4_REJECT("yskn_kv4_attention: a row->depth table is not supported on a sequence shard");
    if (current_algo() == ALGO_MMA) KV4_REJECT("yskn_kv4_attention: the tensor-core kernels do not take a row->depth table or per-row split counts");
    return launch_attention_scalar(*a, g, hd, rd, act_dtype, sh, st, x);
  }
  if (rd > 0 && !a->rope) KV4_REJECT("yskn_kv4_attention: rotary width %d needs a rope table", rd);
  const bool mma_ok = decode_mma_supports(g, hd, rd, a->M);
  const int algo = current_algo();
  // Wide passes (more rows than the warp-level decode kernel takes) go to the tcgen05 kernel.  Up to TC_FUSED_MAX_ROWS rows it
  // converts the packed cache inside the kernel (every CTA pair converts the tiles it reads; measured at 32,768 tokens: 61 / 65 / 111 us
  // for 16 / 32 / 64 rows against 105 / 109 / 136 us with a full dequantisation in front); longer
  // passes dequantise once into a workspace, if the caller has lent one (valid_tokens = 0: the whole workspace is brought
  // up to date on every call), and take the converting form otherwise.
  if (a->M > 8 && algo != ALGO_SCALAR && sh.start == 0 && sh.len == a->max_ctx && !(((uintptr_t)a->q16 | (uintptr_t)a->pacc) & 15)) {
    constexpr int TC_FUSED_MAX_ROWS = 64;
    int dev = 0;
    if (a->M > TC_FUSED_MAX_ROWS && attention_tc_supports(g, hd, rd, act_dtype) && cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
      void* ws = g_tc_ws[dev].load(); const size_t have = g_tc_ws_bytes[dev].load();
      if (ws && have >= attention_tc_workspace_bytes(a->kvh, hd, a->max_ctx, a->M))
        return launch_attention_tc(*a, g, hd, rd, act_dtype, ws, have, 0, nullptr, nullptr, st);
    }
    const uintptr_t al = (uintptr_t)a->kv.kq | (uintptr_t)a->kv.vq | (uintptr_t)a->kv.kscale | (uintptr_t)a->kv.kzero | (uintptr_t)a->kv.kshadow | (uintptr_t)a->rope;
    if (attention_tc_fused_supports(g, hd, rd, act_dtype) && !(al & 15)) return launch_attention_tc_fused(*a, g, hd, rd, act_dtype, nullptr, nullptr, st);
  }
  if (algo == ALGO_MMA && !mma_ok) KV4_REJECT("yskn_kv4_attention: tensor-core path does not cover (g %d, hd %d, rd %d, M %d)", g, hd, rd, a->M);
  if (mma_ok && algo != ALGO_SCALAR) return launch_decode_mma(*a, g, hd, rd, act_dtype, sh, early, st);
  return launch_attention_scalar(*a, g, hd, rd, act_dtype, sh, st);
}

}  // namespace kv4

using namespace kv4;

extern "C" {

const char* yskn_kv4_last_error(void) { return g_err; }

const char* yskn_kv4_build_info(void) {
  return "yskn-kv4 b200 (sm_100a) cudart " KV4_STR(CUDART_VERSION);
}

int yskn_kv4_set_algo(int algo) {
  if (algo < ALGO_AUTO || algo > ALGO_MMA) KV4_REJECT("yskn_kv4_set_algo: unknown algorithm %d", algo);
  g_algo.store(algo, std::memory_order_relaxed); return 0;
}

int yskn_kv4_set_tc_workspace(void* d_workspace, size_t bytes) {
  int dev = 0;
  KV4_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) KV4_REJECT("yskn_kv4_set_tc_workspace: device ordinal %d out of range", dev);
  if (d_workspace && ((uintptr_t)d_workspace & 15)) KV4_REJECT("yskn_kv4_set_tc_workspace: the workspace must be 16-byte aligned");
  g_tc_ws_bytes[dev].store(d_workspace ? bytes : 0); g_tc_ws[dev].store(d_workspace);
  return 0;
}

int yskn_kv4_device_status(int* status) {
  if (!status) KV4_REJECT("yskn_kv4_device_status: null output");
  int a = 0, b = 0;
  if (int rc = decode_status_fetch(&a)) return rc;
  if (int rc = tc_status_fetch(&b)) return rc;
  int c = 0;
  if (int rc = merge_status_fetch(&c)) return rc;
  *status = a ? a : (b ? b : c); return 0;
}

int yskn_kv4_set_peer_wait_polls(unsigned polls) { set_peer_wait_polls(polls); return 0; }

size_t yskn_kv4_exchange_bytes(int world, int M, int nh, int hd) {
  if (world < 1 || world > 8 || M <= 0 || nh <= 0 || hd <= 0) return 0;
  return exchange_bytes(world, M, nh, hd);
}

int yskn_kv4_push_triple(const yskn_attn_g_combine_args* a, int hd, const yskn_kv4_peer_exchange* x, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv4_push_triple: null argument struct");
  return launch_push_triple(*a, hd, x, (cudaStream_t)cuda_stream);
}

int yskn_kv4_merge_pushed(const yskn_kv4_peer_exchange* x, int M, int nh, int g, int hd, const uint16_t* bv, const uint16_t* gate,
                          uint16_t* o16, int act_dtype, void* cuda_stream) {
  return launch_merge_pushed(x, M, nh, g, hd, bv, gate, o16, act_dtype, (cudaStream_t)cuda_stream);
}

int yskn_kv4_exchange_merge(const yskn_attn_g_combine_args* a, int hd, int act_dtype, const yskn_kv4_peer_exchange* x, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv4_exchange_merge: null argument struct");
  return launch_exchange_merge(*a, hd, act_dtype, x, (cudaStream_t)cuda_stream);
}

size_t yskn_kv4_tc_workspace_bytes(int kvh, int hd, int max_ctx, int M) {
  if (kvh <= 0 || (hd != 128 && hd != 256) || max_ctx <= 0 || M <= 0) return 0;
  return attention_tc_workspace_bytes(kvh, hd, max_ctx, M);
}

int yskn_kv4_attention_tc(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, void* d_workspace, size_t workspace_bytes,
                          int valid_tokens, void* cuda_stream) {
  if (int rc = check_attn(a, g, hd, "yskn_kv4_attention_tc")) return rc;
  if (rd > 0 && !a->rope) KV4_REJECT("yskn_kv4_attention_tc: rotary width %d needs a rope table", rd);
  return launch_attention_tc(*a, g, hd, rd, act_dtype, d_workspace, workspace_bytes, valid_tokens, nullptr, nullptr, (cudaStream_t)cuda_stream);
}

int yskn_kv4_prefill_tc(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, const uint16_t* bv, uint16_t* o16,
                        void* d_workspace, size_t workspace_bytes, int valid_tokens, void* cuda_stream) {
  if (!o16) KV4_REJECT("yskn_kv4_prefill_tc: null output");
  if (a && a->splits == 1) {                                 // one split: the attention kernel finishes the rows itself
    if (int rc = check_attn(a, g, hd, "yskn_kv4_prefill_tc")) return rc;
    if (rd > 0 && !a->rope) KV4_REJECT("yskn_kv4_prefill_tc: rotary width %d needs a rope table", rd);
    return launch_attention_tc(*a, g, hd, rd, act_dtype, d_workspace, workspace_bytes, valid_tokens, o16, bv, (cudaStream_t)cuda_stream);
  }
  if (int rc = yskn_kv4_attention_tc(a, g, hd, rd, act_dtype, d_workspace, workspace_bytes, valid_tokens, cuda_stream)) return rc;
  yskn_attn_g_combine_args c{a->pm, a->pl, a->pacc, a->splits, a->M, bv, o16, nullptr, a->nh, g};
  return launch_combine(c, hd, act_dtype, (cudaStream_t)cuda_stream);
}

int yskn_kv4_copy(void* dst, const void* src, size_t bytes, void* cuda_stream) {
  return launch_copy16(dst, src, bytes, (cudaStream_t)cuda_stream);
}

int yskn_kv4_rope_table(float* d_out, int max_ctx, float theta, int rd, void* cuda_stream) {
  return launch_rope_table(d_out, max_ctx, theta, rd, (cudaStream_t)cuda_stream);
}

int yskn_kv4_append(const yskn_kv_append_args* a, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv4_append: null argument struct");
  if (!a->kv.kshadow || !a->kv.vq || !a->kv.vscale || !a->kv.vzero || !a->kv.kq || !a->kv.kscale || !a->kv.kzero)
    KV4_REJECT("yskn_kv4_append: null cache array");
  return launch_append(*a, (cudaStream_t)cuda_stream);
}

int yskn_kv4_group_quant(const yskn_kv_quant_args* a, int kvh, int hd, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv4_group_quant: null argument struct");
  if (!a->kv.kshadow || !a->kv.kq || !a->kv.kscale || !a->kv.kzero) KV4_REJECT("yskn_kv4_group_quant: null cache array");
  return launch_group_quant(*a, kvh, hd, (cudaStream_t)cuda_stream);
}

int yskn_kv4_attention(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, void* cuda_stream) {
  if (int rc = check_attn(a, g, hd, "yskn_kv4_attention")) return rc;
  return attention_dispatch(a, g, hd, rd, act_dtype, Shard{0, a->max_ctx}, (cudaStream_t)cuda_stream);
}

int yskn_kv4_attention_ex(const yskn_attn_g_args* a, const yskn_kv4_attn_ext* x, int g, int hd, int rd, int act_dtype, void* cuda_stream) {
  if (int rc = check_attn(a, g, hd, "yskn_kv4_attention_ex")) return rc;
  return attention_dispatch(a, g, hd, rd, act_dtype, Shard{0, a->max_ctx}, (cudaStream_t)cuda_stream, x);
}

size_t yskn_kv4_ms_maps_bytes(int n_slots) { return n_slots > 0 ? (size_t)n_slots * 2 * 128 : 0; }

int yskn_kv4_ms_prepare(const yskn_kv_layer* h_layers, int n_slots, int kvh, int hd, int max_ctx, yskn_kv_layer* d_layers, void* d_maps,
                        void* cuda_stream) {
  return ms_prepare(h_layers, n_slots, kvh, hd, max_ctx, d_layers, d_maps, (cudaStream_t)cuda_stream);
}

int yskn_kv4_attention_ms(const yskn_attn_g_args* a, const yskn_kv4_ms_rows* ms, int g, int hd, int rd, int act_dtype, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv4_attention_ms: null argument struct");
  if (!ms || !ms->pos || !ms->slot || !ms->layers || !ms->maps || ms->n_slots <= 0 || ms->n_slots > 64)
    KV4_REJECT("yskn_kv4_attention_ms: incomplete row tables");
  if (!a->q16 || !a->pm || !a->pl || !a->pacc) KV4_REJECT("yskn_kv4_attention_ms: null buffer");
  if (a->M <= 0 || a->M > 64 || a->splits <= 0 || a->splits > 65535 || a->kvh <= 0 || g <= 0 || a->nh != a->kvh * g)
    KV4_REJECT("yskn_kv4_attention_ms: bad shape (M %d, splits %d, kvh %d, nh %d, g %d)", a->M, a->splits, a->kvh, a->nh, g);
  if (a->max_ctx <= 0 || a->max_ctx % 64) KV4_REJECT("yskn_kv4_attention_ms: max_ctx %d is not a positive multiple of 64", a->max_ctx);
  if (act_dtype != YSKN_KV4_F16 && act_dtype != YSKN_KV4_BF16) KV4_REJECT("yskn_kv4_attention_ms: act_dtype must be F16 or BF16");
  if (rd > 0 && !a->rope) KV4_REJECT("yskn_kv4_attention_ms: rotary width %d needs a rope table", rd);
  if ((uintptr_t)ms->maps & 127) KV4_REJECT("yskn_kv4_attention_ms: the map table must be 128-byte aligned");
  return launch_decode_mma(*a, g, hd, rd, act_dtype, Shard{0, a->max_ctx}, 0, (cudaStream_t)cuda_stream, ms);
}

int yskn_kv4_attention_shard(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, int shard_start, int shard_len,
                             void* cuda_stream) {
  return yskn_kv4_attention_shard_ex(a, nullptr, g, hd, rd, act_dtype, shard_start, shard_len, cuda_stream);
}

int yskn_kv4_attention_shard_ex(const yskn_attn_g_args* a, const yskn_kv4_attn_ext* x, int g, int hd, int rd, int act_dtype, int shard_start,
                                int shard_len, void* cuda_stream) {
  if (int rc = check_attn(a, g, hd, "yskn_kv4_attention_shard")) return rc;
  if (shard_start < 0 || shard_start % 32 || shard_len < 0 || shard_len % 32 || shard_len > a->max_ctx)
    KV4_REJECT("yskn_kv4_attention_shard: shard [%d, +%d) must start and end on multiples of 32 and fit max_ctx %d", shard_start, shard_len, a->max_ctx);
  return attention_dispatch(a, g, hd, rd, act_dtype, Shard{shard_start, shard_len}, (cudaStream_t)cuda_stream, x);
}

int yskn_kv4_decode(const yskn_attn_g_args* a, const yskn_attn_g_combine_args* c, int g, int hd, int rd, int act_dtype, void* cuda_stream) {
  return yskn_kv4_decode_ex(a, c, nullptr, g, hd, rd, act_dtype, cuda_stream);
}

int yskn_kv4_decode_ex(const yskn_attn_g_args* a, const yskn_attn_g_combine_args* c, const yskn_kv4_attn_ext* x, int g, int hd, int rd,
                       int act_dtype, void* cuda_stream) {
  if (int rc = check_attn(a, g, hd, "yskn_kv4_decode")) return rc;
  if (!c || !c->o16 || c->pm != a->pm || c->pl != a->pl || c->pacc != a->pacc || c->splits != a->splits || c->M != a->M || c->nh != a->nh || c->g != g)
    KV4_REJECT("yskn_kv4_decode: the merge arguments must describe the attention call's scratch and shape");
  if (act_dtype != YSKN_KV4_F16 && act_dtype != YSKN_KV4_BF16) KV4_REJECT("yskn_kv4_decode: act_dtype must be F16 or BF16");
  if (rd > 0 && !a->rope) KV4_REJECT("yskn_kv4_decode: rotary width %d needs a rope table", rd);
  cudaStream_t st = (cudaStream_t)cuda_stream;
  if (int rc = attention_dispatch(a, g, hd, rd, act_dtype, Shard{0, a->max_ctx}, st, x)) return rc;
  return launch_combine(*c, hd, act_dtype, st);
}

int yskn_kv4_decode_shard_triple(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, int shard_start, int shard_len,
                                 float* d_triple, void* cuda_stream) {
  if (int rc = check_attn(a, g, hd, "yskn_kv4_decode_shard_triple")) return rc;
  if (!d_triple) KV4_REJECT("yskn_kv4_decode_shard_triple: null output");
  if (shard_start < 0 || shard_start % 32 || shard_len < 0 || shard_len % 32 || shard_len > a->max_ctx)
    KV4_REJECT("yskn_kv4_decode_shard_triple: shard [%d, +%d) must start and end on multiples of 32 and fit max_ctx %d", shard_start, shard_len, a->max_ctx);
  if (rd > 0 && !a->rope) KV4_REJECT("yskn_kv4_decode_shard_triple: rotary width %d needs a rope table", rd);
  cudaStream_t st = (cudaStream_t)cuda_stream;
  const Shard sh{shard_start, shard_len};
  if (int rc = attention_dispatch(a, g, hd, rd, act_dtype, sh, st)) return rc;
  yskn_attn_g_combine_args c{a->pm, a->pl, a->pacc, a->splits, a->M, nullptr, nullptr, nullptr, a->nh, g};
  return launch_local_triple(c, hd, d_triple, st);
}

int yskn_kv4_combine(const yskn_attn_g_combine_args* a, int hd, int act_dtype, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv4_combine: null argument struct");
  return launch_combine(*a, hd, act_dtype, (cudaStream_t)cuda_stream);
}

int yskn_kv4_xform_a8(const uint16_t* d_o16, const int8_t* d_signs, int8_t* d_qx, float* d_alpha, int M, int n, void* cuda_stream) {
  return launch_xform_a8(d_o16, d_signs, d_qx, d_alpha, M, n, (cudaStream_t)cuda_stream);
}

int yskn_kv4_prefill(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, const uint16_t* bv, uint16_t* o16,
                     void* cuda_stream) {
  if (int rc = check_attn(a, g, hd, "yskn_kv4_prefill")) return rc;
  if (!o16) KV4_REJECT("yskn_kv4_prefill: null output");
  if (int rc = attention_dispatch(a, g, hd, rd, act_dtype, Shard{0, a->max_ctx}, (cudaStream_t)cuda_stream)) return rc;
  yskn_attn_g_combine_args c{a->pm, a->pl, a->pacc, a->splits, a->M, bv, o16, nullptr, a->nh, g};
  return launch_combine(c, hd, act_dtype, (cudaStream_t)cuda_stream);
}

int yskn_kv4_local_triple(const yskn_attn_g_combine_args* a, int hd, float* d_triple, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv4_local_triple: null argument struct");
  return launch_local_triple(*a, hd, d_triple, (cudaStream_t)cuda_stream);
}

int yskn_kv4_merge_triples(const float* d_triples, int ranks, int M, int nh, int g, int hd, const uint16_t* bv,
                           const uint16_t* gate, uint16_t* o16, int act_dtype, void* cuda_stream) {
  return launch_merge_triples(d_triples, ranks, M, nh, g, hd, bv, gate, o16, act_dtype, (cudaStream_t)cuda_stream);
}

int yskn_kv4_decode_noalloc(const uint16_t* q16, const yskn_kv_layer* kv, int max_ctx, const int* d_pos, int splits, const float* rope,
                            int kvh, int nh, int hd, int rd, float qscale, int act_dtype, uint16_t* o16, void* cuda_stream) {
  return decode_noalloc(q16, kv, max_ctx, d_pos, splits, rope, kvh, nh, hd, rd, qscale, act_dtype, o16, (cudaStream_t)cuda_stream);
}

int yskn_kv4_attention_host(const uint16_t* h_q16, const yskn_kv_layer* h_kv, int max_ctx, int M, int pos0, int splits,
                            const float* h_rope, int kvh, int nh, int hd, int rd, float qscale, int act_dtype,
                            uint16_t* h_o16, int reps, float* ms_out) {
  if (!h_q16 || !h_kv || !h_o16) KV4_REJECT("yskn_kv4_attention_host: null buffer");
  if (max_ctx <= 0 || max_ctx % 64 || M <= 0 || pos0 < 0 || pos0 + M > max_ctx || kvh <= 0 || nh % kvh || hd % 32 || reps <= 0 || splits <= 0)
    KV4_REJECT("yskn_kv4_attention_host: bad shape");
  if (rd > 0 && !h_rope) KV4_REJECT("yskn_kv4_attention_host: rotary width %d needs a rope table", rd);
  const int g = nh / kvh; const size_t ng = (size_t)max_ctx / 32;
  const size_t bytes[7] = {(size_t)kvh * ng * 32 * (hd / 2), (size_t)kvh * ng * hd * 2, (size_t)kvh * ng * hd * 2,
                           (size_t)kvh * max_ctx * hd * 2, (size_t)kvh * max_ctx * (hd / 2), (size_t)kvh * max_ctx * 2,
                           (size_t)kvh * max_ctx * 2};
  const void* src[7] = {h_kv->kq, h_kv->kscale, h_kv->kzero, h_kv->kshadow, h_kv->vq, h_kv->vscale, h_kv->vzero};
  std::vector<void*> dev;
  auto cleanup = [&]() { for (void* p : dev) cudaFree(p); };
  auto dalloc = [&](size_t n, const void* h) -> void* {
    void* p = nullptr; if (cudaMalloc(&p, n ? n : 16) != cudaSuccess) return nullptr; dev.push_back(p);
    if (h && cudaMemcpy(p, h, n, cudaMemcpyHostToDevice) != cudaSuccess) return nullptr; return p; };
  void* d[7];
  for (int i = 0; i < 7; ++i) { d[i] = dalloc(bytes[i], src[i]); if (!d[i]) { int e = (int)cudaGetLastError(); cleanup(); set_error("yskn_kv4_attention_host: device allocation or upload failed"); return e ? e : (int)cudaErrorMemoryAllocation; } }
  const size_t nq = (size_t)M * nh * hd, np = (size_t)M * splits * nh;
  void* dq = dalloc(nq * 2, h_q16); void* dpos = dalloc(4, &pos0);
  void* drope = rd > 0 ? dalloc((size_t)max_ctx * (rd / 2) * 8, h_rope) : nullptr;
  void* dpm = dalloc(np * 4, nullptr); void* dpl = dalloc(np * 4, nullptr); void* dpa = dalloc(np * hd * 4, nullptr);
  void* dout = dalloc(nq * 2, nullptr);
  if (!dq || !dpos || (rd > 0 && !drope) || !dpm || !dpl || !dpa || !dout) { cleanup(); set_error("yskn_kv4_attention_host: device allocation or upload failed"); return (int)cudaErrorMemoryAllocation; }
  yskn_attn_g_args A{(const uint16_t*)dq, {(uint8_t*)d[0], (uint16_t*)d[1], (uint16_t*)d[2], (uint16_t*)d[3], (uint8_t*)d[4], (uint16_t*)d[5], (uint16_t*)d[6]},
                     max_ctx, M, (const int*)dpos, splits, (float*)dpm, (float*)dpl, (float*)dpa, (const float*)drope, kvh, nh, qscale};
  yskn_attn_g_combine_args Cb{(float*)dpm, (float*)dpl, (float*)dpa, splits, M, nullptr, (uint16_t*)dout, nullptr, nh, g};
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  int rc = 0;
  for (int i = 0; i < reps && !rc; ++i) {
    cudaEventRecord(e0, 0);
    rc = yskn_kv4_attention(&A, g, hd, rd, act_dtype, nullptr);
    if (!rc) rc = yskn_kv4_combine(&Cb, hd, act_dtype, nullptr);
    cudaEventRecord(e1, 0);
    cudaError_t se = cudaEventSynchronize(e1);
    if (!rc && se != cudaSuccess) { set_error("yskn_kv4_attention_host: %s", cudaGetErrorString(se)); rc = (int)se; }
    if (!rc && ms_out) cudaEventElapsedTime(&ms_out[i], e0, e1);
  }
  if (!rc) { cudaError_t ce = cudaMemcpy(h_o16, dout, nq * 2, cudaMemcpyDeviceToHost); if (ce != cudaSuccess) { set_error("yskn_kv4_attention_host: download: %s", cudaGetErrorString(ce)); rc = (int)ce; } }
  cudaEventDestroy(e0); cudaEventDestroy(e1); cleanup();
  return rc;
}

int yskn_kvx_rotate(const float* d_x, float* d_y, long long rows, int inverse, void* cuda_stream) {
  return launch_kvx_rotate(d_x, d_y, rows, inverse, (cudaStream_t)cuda_stream);
}
int yskn_kvx_encode(const void* d_x, int x_dtype, int8_t* d_q8, float* d_scales, long long rows, void* cuda_stream) {
  return launch_kvx_encode(d_x, x_dtype, d_q8, d_scales, rows, (cudaStream_t)cuda_stream);
}
int yskn_kvx_decode(const int8_t* d_q8, const float* d_scales, void* d_y, int y_dtype, long long rows, void* cuda_stream) {
  return launch_kvx_decode(d_q8, d_scales, d_y, y_dtype, rows, (cudaStream_t)cuda_stream);
}
int yskn_tb_attention(const yskn_tb_attn_args* a, int act_dtype, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_tb_attention: null argument struct");
  return launch_tb_attention(*a, act_dtype, (cudaStream_t)cuda_stream);
}
int yskn_kvx_attn_post(const yskn_kvx_attn_post_args* a, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kvx_attn_post: null argument struct");
  return launch_kvx_attn_post(*a, (cudaStream_t)cuda_stream);
}

int yskn_tb_blob_info(const uint8_t* h_blob, size_t blob_len, int* nm) { return tb_blob_info(h_blob, blob_len, nm); }
size_t yskn_tb_scratch_bytes(int rows, int nm) { return tb_scratch_bytes(rows, nm); }
int yskn_tb_encode(const uint8_t* d_blob, int nm, const float* d_x, const int* d_grp, const int* d_pos, int rows, float* d_y, uint8_t* d_pay,
                   int pay_stride, uint32_t* d_side, void* d_scratch, size_t scratch_bytes, void* cuda_stream) {
  return launch_tb_encode(d_blob, nm, d_x, d_grp, d_pos, rows, d_y, d_pay, pay_stride, d_side, d_scratch, scratch_bytes, (cudaStream_t)cuda_stream);
}

int yskn_tb_decode(const uint8_t* d_blob, const int* d_grp, const int* d_pos, const uint8_t* d_pay, int pay_stride, const uint32_t* d_side,
                   const float* d_yin, float* d_y, int rows, void* cuda_stream) {
  return launch_tb_decode(d_blob, d_grp, d_pos, d_pay, pay_stride, d_side, d_yin, d_y, rows, (cudaStream_t)cuda_stream);
}

int yskn_kv8_attention(const yskn_kv8_attn_args* a, int act_dtype, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv8_attention: null argument struct");
  // passes of more than 8 rows: the tcgen05 kernel over the INT8 rows, when the arrays are aligned for it
  if (a->M > 8 && current_algo() != ALGO_SCALAR && a->q16 && a->pacc && !(((uintptr_t)a->q16 | (uintptr_t)a->pacc) & 15))
    return launch_kv8_attention_tc(*a, act_dtype, (cudaStream_t)cuda_stream);
  return launch_kv8_attention(*a, act_dtype, (cudaStream_t)cuda_stream);
}
int yskn_kv8_attention_tc(const yskn_kv8_attn_args* a, int act_dtype, void* cuda_stream) {
  if (!a) KV4_REJECT("yskn_kv8_attention_tc: null argument struct");
  return launch_kv8_attention_tc(*a, act_dtype, (cudaStream_t)cuda_stream);
}
int yskn_kv8_combine(const float* d_pm, const float* d_pl, const float* d_pacc, int splits, int M, int nh, const void* d_gate,
                     void* d_o16, int act_dtype, int inverse_rotate, void* cuda_stream) {
  return launch_kv8_combine(d_pm, d_pl, d_pacc, splits, M, nh, d_gate, d_o16, act_dtype, inverse_rotate, (cudaStream_t)cuda_stream);
}

int yskn_kvx_probe(const float* x, int8_t* q, float* scales, float* y, int rows) {
  if (rows <= 0 || rows % 2) return -1;                  // the reference's probe takes row pairs
  if (!x || !q || !scales || !y) KV4_REJECT("yskn_kvx_probe: null buffer");
  const size_t n = (size_t)rows * 256;
  float *dx = nullptr, *ds = nullptr, *dy = nullptr; int8_t* dq = nullptr;
  cudaError_t rc = cudaMalloc(&dx, n * 4);
  if (rc == cudaSuccess) rc = cudaMalloc(&dy, n * 4);
  if (rc == cudaSuccess) rc = cudaMalloc(&dq, n);
  if (rc == cudaSuccess) rc = cudaMalloc(&ds, (size_t)rows * 4);
  if (rc == cudaSuccess) rc = cudaMemcpy(dx, x, n * 4, cudaMemcpyHostToDevice);
  int lrc = 0;
  if (rc == cudaSuccess) lrc = launch_kvx_encode(dx, YSKN_KV4_F32, dq, ds, rows, nullptr);
  if (rc == cudaSuccess && !lrc) lrc = launch_kvx_decode(dq, ds, dy, YSKN_KV4_F32, rows, nullptr);
  if (rc == cudaSuccess && !lrc) rc = cudaDeviceSynchronize();
  if (rc == cudaSuccess && !lrc) rc = cudaMemcpy(y, dy, n * 4, cudaMemcpyDeviceToHost);
  if (rc == cudaSuccess && !lrc) rc = cudaMemcpy(q, dq, n, cudaMemcpyDeviceToHost);
  if (rc == cudaSuccess && !lrc) rc = cudaMemcpy(scales, ds, (size_t)rows * 4, cudaMemcpyDeviceToHost);
  cudaFree(dx); cudaFree(dy); cudaFree(dq); cudaFree(ds);
  if (rc != cudaSuccess) { set_error("yskn_kvx_probe: %s", cudaGetErrorString(rc)); return (int)rc; }
  return lrc;
}

}  // extern "C"
