/*
 * C ABI of the B200 (sm_100a) KV4 attention path: quantize-and-append codec, split-K GQA
 * flash-decode, split merge, multi-row verify, causal prefill, shard-triple merge.
 *
 * Conventions follow the reference's ABI (include/yskn_abi.h:19-20,31 and src/c_api.cpp:17-49):
 * every entry returns int, 0 on success, -1 for a rejected argument (message via
 * yskn_kv4_last_error(), thread-local), or a positive cudaError_t.  No C++ exception and no
 * torch type crosses this boundary.  Entries taking `void* cuda_stream` only enqueue work:
 * they never synchronise, allocate or read device memory on the host, so a caller may capture
 * them into a CUDA graph exactly as the reference engine captures its passes
 * (src/engine35.cpp:1973-1989).  All buffers are caller-owned device memory unless the entry
 * name ends in `_host`.
 *
 * Argument structs are member-for-member the reference's launcher structs, so the engine can
 * pass its own objects through a reinterpret_cast (file:line given at each struct).
 */
#ifndef YSKN_KV4_ABI_H
#define YSKN_KV4_ABI_H
#include <stddef.h>
#include <stdint.h>
#if defined(_WIN32)
#  define YSKN_KV4_API __declspec(dllexport)
#else
#  define YSKN_KV4_API __attribute__((visibility("default")))
#endif
#ifdef __cplusplus
extern "C" {
#endif

/* yskn::KvLayer, src/post_kernels.hpp:7-15.  One layer's packed cache:
 *   kq      u8  [Hkv][max_ctx/32][32][HD/2]   byte = channel 2j (low nibble) | channel 2j+1 (high)
 *   kscale  f16 [Hkv][max_ctx/32][HD]          per channel, per 32-token group
 *   kzero   f16 [Hkv][max_ctx/32][HD]
 *   kshadow f16 [Hkv][max_ctx][HD]             every K row, un-rotated
 *   vq      u8  [Hkv][max_ctx][HD/2]
 *   vscale  f16 [Hkv][max_ctx]                 per token
 *   vzero   f16 [Hkv][max_ctx]
 * max_ctx is a multiple of 64 (src/loader.cpp:79).  Every array must be 16-byte aligned. */
typedef struct yskn_kv_layer {
  uint8_t*  kq;
  uint16_t* kscale;
  uint16_t* kzero;
  uint16_t* kshadow;
  uint8_t*  vq;
  uint16_t* vscale;
  uint16_t* vzero;
} yskn_kv_layer;

/* yskn::KvQuantArgs, src/post_kernels.hpp:26 */
typedef struct yskn_kv_quant_args { yskn_kv_layer kv; const int* d_pos; int M; int max_ctx; } yskn_kv_quant_args;

/* yskn::AttnGArgs, src/args.hpp:14-15.  q16 [M][nh][HD] already rotated; pm, pl [M][splits][nh];
 * pacc [M][splits][nh][HD]; rope = (cos,sin) float pairs [max_ctx][rd/2]; *d_pos = position of
 * row 0 (device scalar, so the launch does not depend on it). */
typedef struct yskn_attn_g_args {
  const uint16_t* q16; yskn_kv_layer kv; int max_ctx; int M; const int* d_pos; int splits;
  float* pm; float* pl; float* pacc; const float* rope; int kvh; int nh; float qscale;
} yskn_attn_g_args;

/* yskn::AttnGCombineArgs, src/args.hpp:16-17.  bv [Hkv][HD] and gate [M][nh][HD] may be NULL. */
typedef struct yskn_attn_g_combine_args {
  const float* pm; const float* pl; const float* pacc; int splits; int M; const uint16_t* bv; uint16_t* o16;
  const uint16_t* gate; int nh; int g;
} yskn_attn_g_combine_args;

/* Element type of activations handed in or out (q16, gate, o16, append rows). */
enum { YSKN_KV4_F16 = 0, YSKN_KV4_BF16 = 1, YSKN_KV4_F32 = 2 };

/* Input of the append step: the K and V branches of the reference's QKV epilogue
 * (qkv_post_kernel, src/post_kernels.cu:48-82) with the GEMV un-mixing left to the caller.
 * k_in, v_in: [M][kvh][hd] rows of `in_dtype`; K must be post-norm, PRE-RoPE. */
typedef struct yskn_kv_append_args {
  const void* k_in; const void* v_in; int in_dtype;
  yskn_kv_layer kv; const int* d_pos; int M; int max_ctx; int kvh; int hd;
} yskn_kv_append_args;

YSKN_KV4_API const char* yskn_kv4_last_error(void);   /* yskn_last_error, include/yskn_abi.h:31 */
YSKN_KV4_API const char* yskn_kv4_build_info(void);   /* yskn_build_info, src/c_api.cpp:55 */

/* Kernel choice of yskn_kv4_attention / yskn_kv4_prefill: 0 = automatic (tensor-core kernels where they cover the
 * shape, else the CUDA-core kernel), 1 = CUDA-core kernel only, 2 = tensor-core kernels only (unsupported shapes are
 * rejected).  Process-wide; the counterpart of the reference's YSKN_ATTN_GENERIC switch (src/engine.cpp:189-193). */
YSKN_KV4_API int yskn_kv4_set_algo(int algo);

/* Reads and clears the device status word of the tensor-core decode kernel on the current device (synchronises):
 * 0 = ok, 1/2 = a bounded wait on the decode staging ring ran out (consumer/producer), 3 = misaligned shared memory,
 * 4/5/6 = a bounded wait ran out in the tcgen05 kernel (softmax warps / MMA issuer / producer),
 * 7 = the wait for another shard's triple ran out (yskn_kv4_merge_pushed, yskn_kv4_exchange_merge).
 * A non-zero status means the partials of that launch are invalid.  The kernels never trap; compare the reference's
 * device-side __trap() on bad input (src/kvq_gpu.cuh:91). */
YSKN_KV4_API int yskn_kv4_device_status(int* status);

/* launch_rope_table_g, src/attention_gqa.cu:158-167. */
YSKN_KV4_API int yskn_kv4_rope_table(float* d_out, int max_ctx, float theta, int rd, void* cuda_stream);

/* No counterpart in the reference (its engine keeps activations on the device).  A copy by a kernel for the few kilobytes a
 * decode step exchanges with the host -- the query and the new token's K / V rows in, the attention rows out: dst and src
 * are device pointers or pinned host memory (cudaHostAlloc / cudaHostRegister: device-accessible under unified addressing);
 * bytes and both addresses multiples of 16, at most 64 MiB.  Enqueue-only and graph-capturable like every launcher; in a
 * captured pass it replaces a memcpy node of about 6 us by a kernel node of about 2.  Host memory is read past the caches. */
YSKN_KV4_API int yskn_kv4_copy(void* dst, const void* src, size_t bytes, void* cuda_stream);

/* K shadow store + per-token V int4 (src/post_kernels.cu:48-82) followed by the group quant of every
 * 32-token K group completed by rows [*d_pos, *d_pos+M) (launch_kv_group_quant_g, src/attention_gqa.cu:182-187). */
YSKN_KV4_API int yskn_kv4_append(const yskn_kv_append_args* a, void* cuda_stream);

/* launch_kv_group_quant_g, src/attention_gqa.cu:182-187 (and launch_kv_group_quant, src/post_kernels.cu:86-96). */
YSKN_KV4_API int yskn_kv4_group_quant(const yskn_kv_quant_args* a, int kvh, int hd, void* cuda_stream);

/* launch_attention_gqa, src/attention_gqa.cu:168-175 (and launch_attention, src/attention_kv4q.cu:461-468):
 * split-K partials (pm, pl, pacc) for rows 0..M-1, row r at position *d_pos + r seeing keys 0..*d_pos+r.
 * act_dtype = element type of q16 (YSKN_KV4_F16 as in the reference, or YSKN_KV4_BF16).
 * Every one of the `splits` partial slots of every (row, head) is written; unused ones carry pm = -1e30. */
YSKN_KV4_API int yskn_kv4_attention(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, void* cuda_stream);

/* Extras of an attention call that yskn::AttnGArgs has no member for: the fields the 27B engine's argument set adds
 * (Q35AttnArgs, src/q35.hpp:126-130, and the `wk` argument of launch_q35_atx, src/q35.hpp:136).  A NULL pointer or an
 * all-zero struct is the plain call.
 *   early         the reference's `early` (src/q35.hpp:127, use at src/q35_kernels.cu:1195-1206): the caller promises that
 *                 *d_pos and every cache row below it were final before the kernel that precedes this launch in the stream
 *                 started, so a kernel launched with programmatic stream serialization may read them ahead of
 *                 griddepcontrol.wait and fill its staging ring while the predecessor drains.  Rows at or above *d_pos,
 *                 q16 and the partial buffers are touched only after the wait.
 *   splits_short, long_len   rows that see fewer than long_len keys use splits_short splits instead of `splits`
 *                 (src/q35_atx.cu:113; defaults 31 below 4,096, src/engine35.hpp:434-438); 0 = off.  The partial slots
 *                 beyond a row's split count are written as empty (pm = -1e30).
 *   wk            row -> depth table of a tree-shaped verify pass (src/q35_atx.cu:111-119), M bytes on the device or NULL:
 *                 row r sits at position *d_pos + wk[r], sees the cached keys 0 .. *d_pos + wk[r] - 1 and its own key, which
 *                 is stored in cache slot *d_pos + r.  NULL means wk[r] = r, the plain causal pass. */
typedef struct yskn_kv4_attn_ext { int early; int splits_short; int long_len; const uint8_t* wk; } yskn_kv4_attn_ext;

/* yskn_kv4_attention / yskn_kv4_decode / yskn_kv4_attention_shard with the extras above. */
YSKN_KV4_API int yskn_kv4_attention_ex(const yskn_attn_g_args* a, const yskn_kv4_attn_ext* x, int g, int hd, int rd, int act_dtype,
                                       void* cuda_stream);

/* Rows of several sequences in one pass: the multi-request rows of the reference (Q35MsRows, src/q35.hpp:27-35, kernels in
 * src/q35_atxpk_ms.cu), each row with its own position and its own cache, so that a batch of independent decodes is ONE
 * launch.  All tables live in device memory:
 *   pos[r]   absolute position of row r in its sequence; the row sees keys 0 .. pos[r] of that sequence
 *   slot[r]  index of row r's sequence in `layers` / `maps`
 *   layers   [n_slots] cache arrays of each sequence (same kvh, head_dim and max_ctx for all)
 *   maps     [n_slots][2] the K and V tensor maps of each sequence, 128 bytes each, 128-byte aligned
 * yskn_kv4_ms_prepare fills `layers` and `maps` (yskn_kv4_ms_maps_bytes(n_slots) bytes) from a HOST array of cache
 * descriptors; it is the set-up step made when sequences are bound to slots (it copies from host memory and synchronises
 * the stream, so it is not for graph capture).  yskn_kv4_attention_ms then only enqueues: partials as
 * yskn_kv4_attention writes them ([M][splits][nh]; a->kv and a->d_pos are ignored, a->max_ctx is the common capacity),
 * to be merged by yskn_kv4_combine.  Covers the shapes of the tensor-core decode kernel (g <= 8, head_dim 128 / 256),
 * M <= 64 rows, n_slots <= 64. */
typedef struct yskn_kv4_ms_rows { const int* pos; const int* slot; const yskn_kv_layer* layers; const void* maps; int n_slots; } yskn_kv4_ms_rows;
YSKN_KV4_API size_t yskn_kv4_ms_maps_bytes(int n_slots);
YSKN_KV4_API int yskn_kv4_ms_prepare(const yskn_kv_layer* h_layers, int n_slots, int kvh, int hd, int max_ctx, yskn_kv_layer* d_layers,
                                     void* d_maps, void* cuda_stream);
YSKN_KV4_API int yskn_kv4_attention_ms(const yskn_attn_g_args* a, const yskn_kv4_ms_rows* ms, int g, int hd, int rd, int act_dtype,
                                       void* cuda_stream);

/* launch_attn_combine_gqa_xform, src/attention_gqa.cu:123-134,176-181, up to and including the o16 store
 * (the sign/FWHT/int8 preparation of the next GEMV input is the caller's). act_dtype applies to o16 and gate. */
YSKN_KV4_API int yskn_kv4_combine(const yskn_attn_g_combine_args* a, int hd, int act_dtype, void* cuda_stream);

/* The rest of launch_attn_combine_gqa_xform (src/attention_gqa.cu:135-139 through a8_group512_tail,
 * src/a8_prologue.cuh:86-98,122-133): the int8 input of the projection that follows attention.  Per 512 values of a merged
 * fp16 row o16 [M][n] (n = nh * head_dim, a multiple of 512): x = o16 * signs[i]; Walsh-Hadamard transform of length 512;
 * * 1/sqrt(512); fp16 rounding; alpha = max|x| / 127; qx = rne(x / alpha) clamped to +-127 (0 when alpha is 0).
 * signs [n] are +-1, qx [M][n] int8, alpha [M][n/512] fp32.  Bit-exact with the reference's kernel on the same o16.
 * Launched with programmatic stream serialization right behind the merge. */
YSKN_KV4_API int yskn_kv4_xform_a8(const uint16_t* d_o16, const int8_t* d_signs, int8_t* d_qx, float* d_alpha, int M, int n,
                                   void* cuda_stream);

/* yskn_kv4_attention followed by yskn_kv4_combine in one call: the merge kernel is launched with programmatic stream
 * serialization (the reference's PDL launches, src/pdl.cuh:23-30), so its launch latency hides behind the attention
 * kernel.  `c->pm/pl/pacc/splits/M/nh/g` must describe the same scratch as `a`. */
YSKN_KV4_API int yskn_kv4_decode(const yskn_attn_g_args* a, const yskn_attn_g_combine_args* c, int g, int hd, int rd, int act_dtype,
                                 void* cuda_stream);
YSKN_KV4_API int yskn_kv4_decode_ex(const yskn_attn_g_args* a, const yskn_attn_g_combine_args* c, const yskn_kv4_attn_ext* x, int g, int hd,
                                    int rd, int act_dtype, void* cuda_stream);

/* launch_attention_prefill, src/attention_kv4q.cu:381-453: attention of M new rows whose K/V are already
 * appended, merged in one call to o16 (+ optional bias bv).  `a->pm/pl/pacc` must hold `splits` slots per
 * (row, head) as for yskn_kv4_attention. */
YSKN_KV4_API int yskn_kv4_prefill(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype,
                                  const uint16_t* bv, uint16_t* o16, void* cuda_stream);

/* Tensor-core (tcgen05) attention for many rows: the verify pass and causal prefill.  The counterpart of the reference's
 * dequantise-once path for wide passes, launch_kv_dequant + launch_attention_f32 / launch_attention_prefill_f32
 * (src/attention_kv4q.cu:198-323, src/args.hpp:37-40), whose caller-owned KvF32 arrays become one caller-owned fp16
 * workspace of yskn_kv4_tc_workspace_bytes(kvh, hd, max_ctx, M) bytes (16-byte aligned).  Each call first brings the
 * workspace up to date for tokens [valid_tokens, *d_pos + M): pass 0 unless the same workspace already holds the
 * dequantised tokens [0, valid_tokens) of this cache from an earlier call (valid_tokens <= *d_pos; nothing below the
 * 128-token tile of valid_tokens is touched).  q16 is fp16 or bf16 (act_dtype; bv and o16 have the same type: bf16
 * queries are converted to fp16 operand rows inside the kernel, which is exact for values within the fp16 range); q16,
 * pacc and o16 must be 16-byte aligned (vector stores).  Semantics, partial layout and `splits` are those of yskn_kv4_attention; yskn_kv4_prefill_tc also merges to
 * o16 (+ optional bias).
 * d_workspace = NULL with workspace_bytes = 0 selects the form that needs no workspace: converter warps inside the attention
 * kernel read the packed rows of each key tile (int4 words, scale / zero rows, rope rows, shadow rows of the open groups)
 * and write the fp16 operand tiles themselves.  One launch, nothing dequantised to memory; valid_tokens is ignored.  This
 * form needs the rotary width to be a multiple of 16 channels. */
YSKN_KV4_API size_t yskn_kv4_tc_workspace_bytes(int kvh, int hd, int max_ctx, int M);
/* The plain entries -- yskn_kv4_attention, yskn_kv4_decode, yskn_kv4_prefill, the reference's launcher set unchanged -- run
 * passes of more than 8 rows on the tcgen05 kernel whenever the shape is covered (head_dim 128 / 256, full cache, 16-byte
 * aligned arrays): without a workspace (the converting form above) by default.  This call lends the library a workspace on
 * the CURRENT device (NULL takes it back); passes of more than 64 rows then use the workspace form
 * when it holds yskn_kv4_tc_workspace_bytes(...) for the call, which is faster for long passes (a prefill converts each
 * tile once instead of once per query tile).  Through this route the whole workspace is rewritten on every call (as with
 * valid_tokens = 0); callers that keep it across passes use the _tc entries.  The library only stores the pointer: the
 * caller owns the memory and must not run two such passes on one device at the same time. */
YSKN_KV4_API int yskn_kv4_set_tc_workspace(void* d_workspace, size_t bytes);
YSKN_KV4_API int yskn_kv4_attention_tc(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, void* d_workspace,
                                       size_t workspace_bytes, int valid_tokens, void* cuda_stream);
YSKN_KV4_API int yskn_kv4_prefill_tc(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, const uint16_t* bv,
                                     uint16_t* o16, void* d_workspace, size_t workspace_bytes, int valid_tokens,
                                     void* cuda_stream);

/* Sequence-sharded decode (no reference counterpart: the reference is single-GPU, README.md:37).
 * yskn_kv4_attention_shard is yskn_kv4_attention over a cache that holds only the global tokens
 * [shard_start, shard_start + shard_len) (both multiples of 32, so that no K group and no rope-table row of a
 * group straddles a shard; local token t = global t - shard_start):
 * *d_pos stays the GLOBAL position of row 0, `a->rope` the full table, `a->max_ctx` the local capacity.  Keys outside
 * the shard contribute nothing; a shard with no visible key writes pm = -1e30 in every slot.
 * yskn_kv4_local_triple folds the `splits` partials of each (row, head) into one un-normalised
 * (m, l, O[HD]) triple, float [M][nh][HD+2]; yskn_kv4_merge_triples merges `ranks` gathered triples
 * [ranks][M][nh][HD+2] into o16 with the same arithmetic as yskn_kv4_combine. */
YSKN_KV4_API int yskn_kv4_attention_shard(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype,
                                          int shard_start, int shard_len, void* cuda_stream);
YSKN_KV4_API int yskn_kv4_attention_shard_ex(const yskn_attn_g_args* a, const yskn_kv4_attn_ext* x, int g, int hd, int rd, int act_dtype,
                                             int shard_start, int shard_len, void* cuda_stream);
/* yskn_kv4_attention_shard + yskn_kv4_local_triple in one call (same launch form as yskn_kv4_decode). */
YSKN_KV4_API int yskn_kv4_decode_shard_triple(const yskn_attn_g_args* a, int g, int hd, int rd, int act_dtype, int shard_start,
                                              int shard_len, float* d_triple, void* cuda_stream);
/* The same exchange without a library collective: every rank stores its triple straight into every rank's exchange
 * buffer through NVLink peer mappings, each float together with the step's number in one 8-byte store, so that a reader
 * that finds the number has the value (no fence, no arrival counter: one network latency); the merge kernel polls
 * (bounded, about half a second, then device status 7) until all sources carry this step's number and merges.  buf[w] is rank w's exchange buffer as mapped
 * into THIS process (buf[rank] is the local one), each of yskn_kv4_exchange_bytes(world, M, nh, hd) bytes, 16-byte
 * aligned and zero-filled once before the first step.  Two halves are used alternately, so the ranks need no other
 * synchronisation between steps; every rank must run push and merge exactly once per step, in this order.
 * After a wait ran out (device status 7) the step is abandoned half way: the arrival counters and the step word of
 * that rank no longer agree with its peers'.  Recover by stopping all ranks between steps, zero-filling every rank's
 * exchange buffer again and resuming; the library does not repair it on its own. */
typedef struct yskn_kv4_peer_exchange { float* buf[8]; int world; int rank; } yskn_kv4_peer_exchange;
/* Limit of the wait above in poll rounds of about half a microsecond (process-wide, read at launch; 0 restores the
 * default of 2^20, about half a second).  A short limit lets a host-made failure -- a rank that never pushed -- be observed quickly. */
YSKN_KV4_API int yskn_kv4_set_peer_wait_polls(unsigned polls);
YSKN_KV4_API size_t yskn_kv4_exchange_bytes(int world, int M, int nh, int hd);
YSKN_KV4_API int yskn_kv4_push_triple(const yskn_attn_g_combine_args* a, int hd, const yskn_kv4_peer_exchange* x, void* cuda_stream);
YSKN_KV4_API int yskn_kv4_merge_pushed(const yskn_kv4_peer_exchange* x, int M, int nh, int g, int hd, const uint16_t* bv,
                                       const uint16_t* gate, uint16_t* o16, int act_dtype, void* cuda_stream);
/* Push and merge in ONE launch: every block folds its splits, stores the triple to all ranks, waits (bounded, status 7) for
 * theirs and merges into a->o16 (bias and gate as yskn_kv4_combine).  The blocks wait inside the kernel, so the grid of
 * nh * M blocks must be resident as a whole: nh * M <= 148, larger requests are rejected (use push + merge).  Same buffer
 * protocol as above: in a step a rank calls either this or the pair push/merge. */
YSKN_KV4_API int yskn_kv4_exchange_merge(const yskn_attn_g_combine_args* a, int hd, int act_dtype, const yskn_kv4_peer_exchange* x,
                                         void* cuda_stream);
YSKN_KV4_API int yskn_kv4_local_triple(const yskn_attn_g_combine_args* a, int hd, float* d_triple, void* cuda_stream);
YSKN_KV4_API int yskn_kv4_merge_triples(const float* d_triples, int ranks, int M, int nh, int g, int hd,
                                        const uint16_t* bv, const uint16_t* gate, uint16_t* o16, int act_dtype,
                                        void* cuda_stream);

/* No counterpart in the reference (its launchers always take caller scratch, src/engine.cpp:560-561).
 * One decode step -- split-K attention of ONE query row plus the merge to o16 -- for callers that cannot get device
 * memory for the pm/pl/pacc partials: a plugin host without an allocator, or a serving loop where cudaMalloc is off
 * limits because it stalls the whole GPU.  The partials live in a fixed array inside the library (2,113,536 bytes per
 * GPU that loads it, held until exit), so the call allocates nothing, on the host side of CUDA or through any library.
 * Limit: splits * nh * (hd + 2) <= 528,384 floats (for instance 64 splits x 32 heads x head_dim 256); anything
 * larger is rejected with -1 and a message.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and should therefore be made before any stream capture; later
 * calls only enqueue.  All calls on a device share the array: calls that overlap on the GPU race, run them in order.
 * Nothing needs clearing between calls, every partial slot is rewritten before it is read.  Arguments as for
 * yskn_kv4_attention / yskn_kv4_combine with M = 1, no bias, no gate. */
YSKN_KV4_API int yskn_kv4_decode_noalloc(const uint16_t* q16, const yskn_kv_layer* kv, int max_ctx, const int* d_pos, int splits,
                                         const float* rope, int kvh, int nh, int hd, int rd, float qscale, int act_dtype,
                                         uint16_t* o16, void* cuda_stream);

/* Host-pointer probe in the style of the reference's kernel probes (yskn_atxpk_bench, src/kvx_probe.cu:190-330):
 * uploads a packed cache and M query rows, runs attention + combine `reps` times on the current device,
 * downloads o16 and, if ms_out != NULL, the per-repetition device times in milliseconds (ms_out[reps]).
 * Returns 0, -1 (bad argument) or a cudaError_t.  Allocates and frees its own device memory. */
YSKN_KV4_API int yskn_kv4_attention_host(const uint16_t* h_q16, const yskn_kv_layer* h_kv, int max_ctx, int M, int pos0,
                                         int splits, const float* h_rope, int kvh, int nh, int hd, int rd, float qscale,
                                         int act_dtype, uint16_t* h_o16, int reps, float* ms_out);

/* ---------------------------------------------------------------------------------------------------------------
 * Family-B row codec, step 1: sign-Hadamard-256 rotation + INT8 rows (reference src/kvx_codec.cuh, built with
 * YSKN_KVX_MODE 3, CMakeLists.txt:56).  Rows are 256 values; q8 is [rows][256] int8, scales [rows] fp32.
 * Bit-exact with the reference's kvx_sign / kvx_rotate / kvx_store and with the round trip of its probe.
 * Device pointers, enqueue-only, nothing allocated; rows = 0 is a no-op. */

/* kvx_rotate, src/kvx_codec.cuh:35-49: y = H(sign . x) / 16, or with inverse != 0: y = sign . H(x) / 16.  fp32 rows,
 * 16-byte aligned; x == y is allowed.  This is what the reference applies to Q rows and, inverted, to the merged output
 * (src/q35_kernels.cu:1420-1422). */
YSKN_KV4_API int yskn_kvx_rotate(const float* d_x, float* d_y, long long rows, int inverse, void* cuda_stream);

/* kvx_rotate (forward) + kvx_store, src/kvx_codec.cuh:35-70: scale = max|r| / 127, q = rne(r / scale) clamped to +-127
 * (0 for an all-zero row).  x_dtype = YSKN_KV4_F32 / F16 / BF16 (values are widened to fp32 exactly first). */
YSKN_KV4_API int yskn_kvx_encode(const void* d_x, int x_dtype, int8_t* d_q8, float* d_scales, long long rows, void* cuda_stream);

/* (float)q * scale, then the inverse rotation (src/kvx_probe.cu:15-19); y_dtype F16/BF16 rounds the fp32 result once. */
YSKN_KV4_API int yskn_kvx_decode(const int8_t* d_q8, const float* d_scales, void* d_y, int y_dtype, long long rows, void* cuda_stream);

/* The attention block's row epilogue for INT8 rows: the reference's launch_q35_attn_post / q35_attn_post_kernel
 * (src/q35_kernels.cu:1013-1069, argument struct Q35AttnPostArgs, src/q35.hpp:97-104) from the point where a thread holds
 * its bf16-rounded projection value (:1029).  What precedes that point in the reference's kernel -- the combine of the
 * GEMV's partial sums, tau, and the inverse Hadamard-512 (part_*, tau_*, nw_*, sg_*, xsm) -- belongs to the weight path
 * and stays with the caller, which hands over the rows instead:
 *   q_rows bf16 [M][nh][512]   per head 256 query channels, then the 256 gate channels (the projection's output order)
 *   k_rows, v_rows bf16 [M][kvh][256]
 * Per query / key head: RMS norm over the 256 channels with weight (1 + w), partial RoPE (rotate-half over the first rd
 * channels, table row of *d_pos + token), sign-Hadamard-256 rotation; q16 bf16 [M][nh][256]; keys and (rotated) values go
 * to the INT8 row caches k8 / v8 [kvh][max_ctx][256] with ks / vs [kvh][max_ctx] at the token's position; gate16 bf16
 * [M][nh][256] is the gate half as it is.  Bit-exact with the reference's kernel: pm != 0 computes 1 / sqrt with IEEE
 * operations (its portable-math mode, src/pm_math.cuh:16, q35_set_pm), pm = 0 uses rsqrtf like its default.  rd is a
 * multiple of 64 up to 256 (the reference: 64); rope is the float2 table [max_ctx][rd/2] (yskn_kv4_rope_table), 16-byte
 * aligned; row arrays 8-byte aligned.  A token whose position lies outside [0, max_ctx) stores no cache row. */
typedef struct {
  const uint16_t* q_rows; const uint16_t* k_rows; const uint16_t* v_rows;
  const uint16_t* qn_w; const uint16_t* kn_w;   /* bf16 [256] each */
  float eps; int M; const int* d_pos; const float* rope; int rd;
  uint16_t* q16; uint16_t* gate16;
  int8_t* k8; int8_t* v8; float* ks; float* vs;
  int max_ctx; int nh; int kvh; int pm;
} yskn_kvx_attn_post_args;
YSKN_KV4_API int yskn_kvx_attn_post(const yskn_kvx_attn_post_args* a, void* cuda_stream);

/* Host-pointer probe with the contract of the reference's yskn_kvx_probe (src/kvx_probe.cu:22-36): rows even and > 0,
 * x[rows*256] in; q[rows*256], scales[rows], y[rows*256] (decoded) out.  Returns 0, -1 (bad rows) or a cudaError_t.
 * Allocates and frees its own device memory. */
YSKN_KV4_API int yskn_kvx_probe(const float* x, int8_t* q, float* scales, float* y, int rows);

/* ---------------------------------------------------------------------------------------------------------------
 * Family-B row codec, step 2: the trellis ("CDQ") re-quantisation of 256-value rows with 3 / 4 / 5 bits per value and
 * its packed payload (reference: tb_fakequant, src/kvq_gpu.cuh:54-148; the fast encoder and its packer,
 * src/kvq_fast.cuh:96-232; launch_tb_fast, :242-255).  The code tables, scale multipliers and per-group records come
 * from a "KVQP v1" profile blob (fields: src/kvq_gpu.cuh:57-68; loader checks: src/engine35.cpp:50-53), which the
 * caller uploads to the device as it is.  Bit-exact with the reference on the same blob and rows.
 *
 * yskn_tb_blob_info: HOST-side check of a blob with the reference loader's rules; *nm = its number of scale multipliers.
 * yskn_tb_encode: rows of 256 fp32 values d_x [rows][256]; d_grp[r] = group record of row r ((layer*4 + kv_head)*2 + kind,
 * kind 0 = K, 1 = V), d_pos[r] = its position (rows below the group's guard position are passed through and not
 * packed).  Outputs, each optional (NULL): d_y [rows][256] the re-quantised rows; d_pay [rows][pay_stride bytes] the
 * payload, 8*k 32-bit words per row, the k new bits of every value MSB first (pay_stride >= 160, a multiple of 4);
 * d_side [rows][2] = the row's scale (fp32 bits) and its two fp16 low-rank coefficients.  d_scratch:
 * yskn_tb_scratch_bytes(rows, nm) bytes.  Enqueue-only, nothing allocated. */
/* yskn_tb_decode: the packed rows back to fp32 values (tba_unpack_kernel, src/kvq_attn.cuh:39-72): every value's state is
 * the 8-bit window of the row's bit stream that ends with its field, so rows decode without the search; rows that were
 * not packed take d_yin (may be NULL: zeros).  Same d_grp / d_pos / pay_stride as the encoder's. */
YSKN_KV4_API int yskn_tb_decode(const uint8_t* d_blob, const int* d_grp, const int* d_pos, const uint8_t* d_pay, int pay_stride,
                                const uint32_t* d_side, const float* d_yin, float* d_y, int rows, void* cuda_stream);
YSKN_KV4_API int yskn_tb_blob_info(const uint8_t* h_blob, size_t blob_len, int* nm);
YSKN_KV4_API size_t yskn_tb_scratch_bytes(int rows, int nm);
YSKN_KV4_API int yskn_tb_encode(const uint8_t* d_blob, int nm, const float* d_x, const int* d_grp, const int* d_pos, int rows, float* d_y,
                                uint8_t* d_pay, int pay_stride, uint32_t* d_side, void* d_scratch, size_t scratch_bytes, void* cuda_stream);

/* Decode attention straight over packed trellis rows: the counterpart of the reference's attention over packed rows
 * (launch_q35_atxpk, src/q35_atxpk.hpp:14-24, src/q35_atxpk3.cuh / q35_atxpk4.cuh) for passes of a few rows.  Every key and
 * value row is unpacked inside the kernel by the rule of yskn_tb_decode (tba_unpack_kernel, src/kvq_attn.cuh:39-72; bit for
 * bit the same values) and consumed at once, so the result equals attention over the unpacked rows; nothing unpacked is
 * written to memory.  k_pay / v_pay [kvh][max_ctx][pay_stride] bytes and k_side / v_side [kvh][max_ctx][2] words as
 * yskn_tb_encode writes them with pos = the token's position; grp_k / grp_v [kvh] (device) name the profile's group record
 * of each head's rows; rows the profile leaves unpacked (position below the group's guard, or a group that is not a
 * packed one) are read from k_plain / v_plain fp32 [kvh][max_ctx][256] (NULL: zeros), the `yin` of yskn_tb_decode.
 * q16 [M][nh][256] bf16 or fp16; row r sits at *d_pos + r and sees keys 0 .. *d_pos + r; partials in the layout of
 * yskn_kv8_attention (merge with yskn_kv8_combine).  A CUDA-core kernel (32 keys per warp step, payload rows staged by asynchronous copies): a first path, far from the memory roofline (latency-bound). */
typedef struct {
  const uint16_t* q16; const uint8_t* blob;
  const uint8_t* k_pay; const uint8_t* v_pay; int pay_stride;
  const uint32_t* k_side; const uint32_t* v_side;
  const int* grp_k; const int* grp_v;
  const float* k_plain; const float* v_plain;
  int max_ctx; int M; const int* d_pos; int splits;
  float* pm; float* pl; float* pacc;
  int kvh; int nh; float qscale;
} yskn_tb_attn_args;
YSKN_KV4_API int yskn_tb_attention(const yskn_tb_attn_args* a, int act_dtype, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------------------------
 * Family-B decode attention over the INT8 rows above: the INT8 members of the reference's Q35AttnArgs
 * (src/q35.hpp:126-130), with the head counts the reference fixes at compile time (Q35_NH, Q35_KVH) as fields.
 * head_dim is 256.  q16 [M][nh][256] is bf16 (the reference's dtype) or fp16, already rotated (yskn_kvx_rotate);
 * k8, v8 [kvh][max_ctx][256] int8 with ks, vs [kvh][max_ctx] fp32 (yskn_kvx_encode); row r sits at *d_pos + r and sees
 * keys 0 .. *d_pos + r; partials in the reference's layout pm, pl [M][splits][nh], pacc [M][splits][nh][256]. */
typedef struct yskn_kv8_attn_args {
  const uint16_t* q16;
  const int8_t* k8; const int8_t* v8; const float* ks; const float* vs;
  int max_ctx; int M; const int* d_pos; int splits;
  float* pm; float* pl; float* pacc;
  int kvh; int nh; float qscale;            /* the reference multiplies q by 0.0625 = 1/sqrt(256) (src/q35_kernels.cu:1211) */
} yskn_kv8_attn_args;

/* launch_q35_attention, INT8 branch (q35_attention_kernel<true>, src/q35_kernels.cu:1176-1281).  nh / kvh <= 8,
 * max_ctx a multiple of 64, k8/v8 16-byte aligned.  Split boundaries are multiples of 16 keys (the merge does not depend on them). */
YSKN_KV4_API int yskn_kv8_attention(const yskn_kv8_attn_args* a, int act_dtype, void* cuda_stream);
/* The same partials for many rows (verify passes, prefill) on the tcgen05 kernel: the counterpart of the reference's
 * tensor-core verify kernels over INT8 rows (launch_q35_atx / q35_fa8_kernel, src/q35_atx.cu:92-793, src/q35_fa.cu:48-303;
 * same row semantics as q35_attention_kernel<KV8>, row by row).  Converter warps read the INT8 rows and scales and write
 * fp16 operand tiles (byte times scale, rounded once to fp16); q16 fp16 or bf16; q16 and pacc 16-byte aligned; `splits`
 * partitions the 128-key tiles below *d_pos.  yskn_kv8_attention takes this route by itself for M > 8. */
YSKN_KV4_API int yskn_kv8_attention_tc(const yskn_kv8_attn_args* a, int act_dtype, void* cuda_stream);

/* Merge of the splits as launch_q35_combine does up to the gated row (src/q35_kernels.cu:1400-1424): y = o / L, inverse
 * rotation if inverse_rotate != 0, rounding to the activation dtype, then y * sigmoid(gate) with the reference's roundings
 * if d_gate != NULL ([M][nh][256], activation dtype).  splits <= 64.  The int8 requantisation for the next GEMV is not part of this. */
YSKN_KV4_API int yskn_kv8_combine(const float* d_pm, const float* d_pl, const float* d_pacc, int splits, int M, int nh, const void* d_gate,
                                  void* d_o16, int act_dtype, int inverse_rotate, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
