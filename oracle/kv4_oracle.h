/*
 * CPU oracle for the KV4 attention path -- TEST INFRASTRUCTURE, NOT PRODUCT.
 *
 * A scalar C restatement of the reference's Family-A ("KV4") algorithm: the
 * quantize-and-append codec, the packed-cache layout, the dequantisation rule,
 * RoPE-on-read, split-K online softmax and the split merge.  Only tests, the
 * smoke check and the bench's CPU-baseline leg may call into this library; the
 * product library never links or loads it.
 *
 * Pinning: the reference ships no golden vectors or known-answer tests for this
 * path, so the restatement is pinned against the reference's own CUDA kernels
 * compiled from its sources (oracle/_ref, run on a GPU box) and against the
 * committed known-answer files under tests/golden/ that this oracle produced.
 *
 * Citations are file:line inside the reference project.
 */
#ifndef YSKN_KV4_ORACLE_H
#define YSKN_KV4_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Packed cache of one layer; same member order as the reference's KvLayer
 * (src/post_kernels.hpp:7-15).  Shapes (src/attention_gqa.cu:40-49,153):
 *   kq      u8   [Hkv][max_ctx/32][32][HD/2]  byte = ch 2j low nibble, 2j+1 high
 *   kscale  f16  [Hkv][max_ctx/32][HD]
 *   kzero   f16  [Hkv][max_ctx/32][HD]
 *   kshadow f16  [Hkv][max_ctx][HD]           every token, un-rotated
 *   vq      u8   [Hkv][max_ctx][HD/2]
 *   vscale  f16  [Hkv][max_ctx]
 *   vzero   f16  [Hkv][max_ctx]                                              */
typedef struct ysko_kv_layer {
  uint8_t* kq; uint16_t* kscale; uint16_t* kzero; uint16_t* kshadow;
  uint8_t* vq; uint16_t* vscale; uint16_t* vzero;
} ysko_kv_layer;

/* scalar conversions (IEEE, round-to-nearest-even) */
uint16_t ysko_f32_to_f16(float f);
float    ysko_f16_to_f32(uint16_t h);
uint16_t ysko_f32_to_bf16(float f);
float    ysko_bf16_to_f32(uint16_t h);
void     ysko_bf16_to_f16_array(const uint16_t* in, uint16_t* out, size_t n);

/* (cos,sin) table [max_ctx][rd/2][2], angle = float(t) * theta^(-2i/rd)
 * (src/attention_gqa.cu:158-162). */
void ysko_rope_table(float* out, int max_ctx, float theta, int rd);

/* Append M rows at positions [pos0, pos0+M): K row -> fp16 shadow
 * (src/post_kernels.cu:52-54), V row -> per-token int4 (src/post_kernels.cu:64-82),
 * then quantise every 32-token K group whose last token lies in the pass
 * (src/attention_gqa.cu:143-154).  k16/v16 are fp16 [M][Hkv][HD]. */
void ysko_append(const ysko_kv_layer* kv, int hkv, int hd, int max_ctx, int pos0, int M,
                 const uint16_t* k16, const uint16_t* v16);
/* Only the group-quant step (src/attention_gqa.cu:143-154). */
void ysko_group_quant(const ysko_kv_layer* kv, int hkv, int hd, int max_ctx, int pos0, int M);

/* Reference-literal split-K partials (src/attention_gqa.cu:17-118): row r has
 * pos = pos0 + r, len = pos + 1, per = ceil(len/S), keys [s*per, min(len,(s+1)*per)).
 * pm, pl: [M][S][Hq]; pacc: [M][S][Hq][HD].  rope may be NULL when rd == 0. */
void ysko_attention_partials(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                             int S, float* pm, float* pl, float* pacc, const float* rope,
                             int hkv, int hq, int hd, int rd, float qscale, int threads);
void ysko_attention_partials_shard(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                                   int S, float* pm, float* pl, float* pacc, const float* rope,
                                   int hkv, int hq, int hd, int rd, float qscale, int threads,
                                   int shard_start, int shard_len);
/* Split merge -> fp16 (src/attention_gqa.cu:127-134): optional V bias bv [Hkv][HD]
 * and sigmoid gate [M][Hq][HD], both fp16. */
void ysko_combine(const float* pm, const float* pl, const float* pacc, int S, int M, int hq, int g, int hd,
                  const uint16_t* bv, const uint16_t* gate, uint16_t* o16);

/* Tolerance oracle: softmax over the dequantised cache with double accumulators,
 * no splits; row r sees keys 0..pos0+r with the own-group-from-shadow rule
 * (src/attention_gqa.cu:24,38-43,55-70).  out: float [M][Hq][HD] (no bias/gate).
 * row_begin/row_end select a subset of rows (others left untouched). */
/* Family-B step 2: trellis re-quantisation of 256-value rows and its packed payload (tb_oracle.c) */
int ysko_tb_check_blob(const uint8_t* blob, size_t n);
void ysko_tb_encode(const uint8_t* blob, const float* x, const int* grp, const int* pos, int rows,
                    float* y_fq, uint8_t* fields, uint32_t* pay, uint32_t* side, int* kb);
void ysko_tb_unpack(const uint8_t* blob, const int* grp, const int* pos, const uint32_t* pay, int stride_words, const uint32_t* side,
                    const float* yin, float* y, int rows);
void ysko_tb_decode_fields(const uint8_t* blob, int g, const uint32_t* pay, float scale, float* xq);
void ysko_xform_a8(const uint16_t* o16, const int8_t* signs, int8_t* qx, float* alpha, int M, int n);
void ysko_attention_exact_wk(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                             const float* rope, int hkv, int hq, int hd, int rd, float qscale,
                             float* out, int row_begin, int row_end, int threads, const uint8_t* wk);
void ysko_attention_exact(const uint16_t* q16, const ysko_kv_layer* kv, int max_ctx, int M, int pos0,
                          const float* rope, int hkv, int hq, int hd, int rd, float qscale,
                          float* out, int row_begin, int row_end, int threads);

/* Merge of R (m, l, O) triples per head, as exchanged between sequence shards:
 * parts [R][Hq][HD+2] = {m, l, O[HD]} un-normalised; out float [Hq][HD]. */
void ysko_merge_triples(const float* parts, int R, int hq, int hd, float* out);

int ysko_max_threads(void);

/* ---- Family-B row codec, step 1 (kvx_oracle.c): rows of 256 fp32 values */
float ysko_kvx_sign(int d);
void ysko_kvx_rotate(const float* x, float* y, long rows, int inverse);
void ysko_kvx_encode(const float* x, int8_t* q8, float* scales, long rows);
void ysko_kvx_decode(const int8_t* q8, const float* scales, float* y, long rows);
void ysko_kvx_attn_post(const uint16_t* q_rows, const uint16_t* k_rows, const uint16_t* v_rows, const uint16_t* qn_w, const uint16_t* kn_w,
                        float eps, int M, int pos0, const float* rope, int rd, int nh, int kvh, int max_ctx,
                        uint16_t* q16, uint16_t* gate16, int8_t* k8, float* ks, int8_t* v8, float* vs);
void ysko_rows_attention_exact(const float* q, const float* k, const float* v, int max_ctx, int M, int pos0, int kvh, int nh,
                               float qscale, float* out);
void ysko_kv8_attention_exact(const float* q, const int8_t* k8, const int8_t* v8, const float* ks, const float* vs, int max_ctx,
                              int M, int pos0, int kvh, int nh, float qscale, float* out);
#ifdef __cplusplus
}
#endif
#endif
