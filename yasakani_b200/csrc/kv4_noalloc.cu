// One decode step (split-K attention + merge) that needs no scratch buffer from the caller.
//
// Who this is for: callers that reach the library from a place where they cannot obtain device memory -- a
// plugin host that owns no allocator, a serving loop that must not call cudaMalloc because it synchronises the
// whole device, a thin C client that only holds the cache and the query.  The regular entries
// (yskn_kv4_attention + yskn_kv4_combine) want pm/pl/pacc scratch sized by the caller; here that scratch is a
// fixed array inside the library image, so every GPU that loads the library carries it until the process exits.
//
// Limits: one query row (M = 1) and splits * nh * (hd + 2) <= KV4_NOALLOC_FLOATS floats (2,113,536 bytes; e.g.
// 64 splits x 32 heads x head_dim 256).  Larger requests are rejected with an error text, never truncated.
//
// Sharing: every call on a device uses the same array.  Nothing in it has to start at zero -- the attention kernel
// writes every partial slot it later reads -- but two calls that overlap on the GPU (different streams, or the same
// graph launched twice concurrently) race on it.  Serialise them.
#include "kv4_common.cuh"
#include <mutex>

namespace kv4 {
namespace {

constexpr size_t KV4_NOALLOC_FLOATS = (size_t)64 * 32 * (256 + 2);
constexpr size_t KV4_NOALLOC_PAD = 8;                // two planes rounded up to a multiple of four floats

// Scratch for the split-K partials: [splits][nh] m, [splits][nh] l, [splits][nh][hd] O, packed back to back.
// In host code this name is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[KV4_NOALLOC_FLOATS + KV4_NOALLOC_PAD];

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
float* g_scratch_ptr[MAX_DEVICES] = {};

// Device address of the scratch array on the current device; looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = -1;
  KV4_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) KV4_REJECT("yskn_kv4_decode_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_scratch_ptr[dev]) {
    float* p = nullptr;
    KV4_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

int decode_noalloc(const uint16_t* q16, const yskn_kv_layer* kv, int max_ctx, const int* d_pos, int splits, const float* rope,
                   int kvh, int nh, int hd, int rd, float qscale, int act_dtype, uint16_t* o16, cudaStream_t st) {
  if (!q16 || !kv || !d_pos || !o16) KV4_REJECT("yskn_kv4_decode_noalloc: null buffer");
  if (!kv->kq || !kv->kscale || !kv->kzero || !kv->kshadow || !kv->vq || !kv->vscale || !kv->vzero)
    KV4_REJECT("yskn_kv4_decode_noalloc: null cache array");
  if (act_dtype != YSKN_KV4_F16 && act_dtype != YSKN_KV4_BF16) KV4_REJECT("yskn_kv4_decode_noalloc: act_dtype must be F16 or BF16");
  if (kvh <= 0 || nh <= 0 || nh % kvh || nh / kvh > 8 || splits <= 0 || splits > 65535 || (hd != 64 && hd != 128 && hd != 256) || max_ctx <= 0 || max_ctx % 64)
    KV4_REJECT("yskn_kv4_decode_noalloc: bad shape (kvh %d, nh %d, hd %d, splits %d, max_ctx %d)", kvh, nh, hd, splits, max_ctx);
  if (rd < 0 || rd > hd || rd % 2) KV4_REJECT("yskn_kv4_decode_noalloc: rotary width %d does not fit head_dim %d", rd, hd);
  const size_t need = (size_t)splits * nh * (hd + 2);
  if (need > KV4_NOALLOC_FLOATS)
    KV4_REJECT("yskn_kv4_decode_noalloc: splits*nh*(hd+2) = %zu floats exceeds the built-in scratch of %zu floats; "
               "use fewer splits or the entries that take caller scratch", need, KV4_NOALLOC_FLOATS);
  if (rd > 0 && !rope) KV4_REJECT("yskn_kv4_decode_noalloc: rotary width %d needs a rope table", rd);
  float* s = nullptr;
  if (int rc = scratch_for_current_device(&s)) return rc;
  const size_t n = ((size_t)splits * nh + 3) / 4 * 4;      // the m and l planes, padded so that the O plane starts 16-byte aligned
  yskn_attn_g_args a{q16, *kv, max_ctx, 1, d_pos, splits, s, s + n, s + 2 * n, rope, kvh, nh, qscale};
  const int g = nh / kvh;
  const bool mma_ok = decode_mma_supports(g, hd, rd, 1);
  const int algo = current_algo();                       // yskn_kv4_set_algo applies here as in yskn_kv4_attention
  if (algo == ALGO_MMA && !mma_ok) KV4_REJECT("yskn_kv4_decode_noalloc: tensor-core path does not cover (g %d, hd %d, rd %d)", g, hd, rd);
  int rc = mma_ok && algo != ALGO_SCALAR
               ? launch_decode_mma(a, g, hd, rd, act_dtype, Shard{0, max_ctx}, 0, st)
               : launch_attention_scalar(a, g, hd, rd, act_dtype, Shard{0, max_ctx}, st);
  if (rc) return rc;
  yskn_attn_g_combine_args c{a.pm, a.pl, a.pacc, splits, 1, nullptr, o16, nullptr, nh, g};
  return launch_combine(c, hd, act_dtype, st);
}

}  // namespace kv4
