// Shared declarations of the KV4 attention library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <atomic>
#include <cstdint>
#include <cstdio>
#include "../../include/yskn_kv4_abi.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "this library is written for sm_100a (B200) only"
#endif

namespace kv4 {

// ---- host-side error plumbing (thread-local message, like src/c_api.cpp:17) ----
void set_error(const char* fmt, ...);
#define KV4_REJECT(...) do { ::kv4::set_error(__VA_ARGS__); return -1; } while (0)
#define KV4_CUDA(expr) do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) { \
    ::kv4::set_error("%s: %s", #expr, cudaGetErrorString(e__)); return (int)e__; } } while (0)
inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("%s: %s", what, cudaGetErrorString(e)); return (int)e; }
  return 0;
}

// Function attributes are per device: true the first time a launcher runs on the current device (flags = one word per
// launcher, bit d = done on device d).  The reference sets them once per process (src/q35_fa.cu:305-307) because an engine
// owns one GPU; a process that drives several GPUs through this library gets them on each.
inline bool first_use_on_device(std::atomic<unsigned long long>& flags) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
  const unsigned long long bit = 1ull << dev;
  return (flags.fetch_or(bit) & bit) == 0;
}

// ---- device scalar helpers ----
__device__ __forceinline__ float h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t f2h(float f) { return __half_as_ushort(__float2half_rn(f)); }
__device__ __forceinline__ float bf2f(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t f2bf(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float round_f16(float f) { return __half2float(__float2half_rn(f)); }

// activation element (q16, gate, o16, append rows) -> float and back
template <int DT> __device__ __forceinline__ float act_load(const void* p, size_t i) {
  if (DT == YSKN_KV4_F16) return h2f(static_cast<const uint16_t*>(p)[i]);
  if (DT == YSKN_KV4_BF16) return bf2f(static_cast<const uint16_t*>(p)[i]);
  return static_cast<const float*>(p)[i];
}
template <int DT> __device__ __forceinline__ uint16_t act_store16(float v) {
  return DT == YSKN_KV4_BF16 ? f2bf(v) : f2h(v);
}

// A sequence shard: the local cache arrays hold global tokens [start, start+len); start is a multiple of 32.
// One GPU: {0, max_ctx}.
struct Shard { int start; int len; };

// ---- launchers implemented in the .cu files (all enqueue-only) ----
int launch_rope_table(float* d_out, int max_ctx, float theta, int rd, cudaStream_t st);
int launch_append(const yskn_kv_append_args& a, cudaStream_t st);
int launch_group_quant(const yskn_kv_quant_args& a, int kvh, int hd, cudaStream_t st);
int launch_attention_scalar(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, Shard sh, cudaStream_t st,
                            const yskn_kv4_attn_ext* ext = nullptr);
int launch_decode_mma(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, Shard sh, int early, cudaStream_t st,
                      const yskn_kv4_ms_rows* ms = nullptr);
int ms_prepare(const yskn_kv_layer* h_layers, int n_slots, int kvh, int hd, int max_ctx, yskn_kv_layer* d_layers, void* d_maps, cudaStream_t st);
bool decode_mma_supports(int g, int hd, int rd, int M);
int decode_status_fetch(int* out);
int tc_status_fetch(int* out);       // same for the tcgen05 multi-row kernel
bool attention_tc_supports(int g, int hd, int rd, int act_dtype);
size_t attention_tc_workspace_bytes(int kvh, int hd, int max_ctx, int M);
bool attention_tc_fused_supports(int g, int hd, int rd, int act_dtype);
int launch_attention_tc_fused(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, uint16_t* o16_direct, const uint16_t* bv, cudaStream_t st);
// o16_direct != nullptr and splits == 1: rows are finished in the kernel (o/l, + bv) and no partials are written
int launch_attention_tc(const yskn_attn_g_args& a, int g, int hd, int rd, int act_dtype, void* workspace, size_t workspace_bytes,
                        int valid_tokens, uint16_t* o16_direct, const uint16_t* bv, cudaStream_t st);   // reads and clears the device status word of the tensor-core decode kernel
int launch_combine(const yskn_attn_g_combine_args& a, int hd, int act_dtype, cudaStream_t st);
int launch_xform_a8(const uint16_t* o16, const int8_t* signs, int8_t* qx, float* alpha, int M, int n, cudaStream_t st);
int launch_local_triple(const yskn_attn_g_combine_args& a, int hd, float* d_triple, cudaStream_t st);
int launch_merge_triples(const float* d_triples, int ranks, int M, int nh, int g, int hd, const uint16_t* bv,
                         const uint16_t* gate, uint16_t* o16, int act_dtype, cudaStream_t st);

int decode_noalloc(const uint16_t* q16, const yskn_kv_layer* kv, int max_ctx, const int* d_pos, int splits, const float* rope,
                   int kvh, int nh, int hd, int rd, float qscale, int act_dtype, uint16_t* o16, cudaStream_t st);

size_t exchange_bytes(int world, int M, int nh, int hd);
int launch_push_triple(const yskn_attn_g_combine_args& a, int hd, const yskn_kv4_peer_exchange* x, cudaStream_t st);
int launch_merge_pushed(const yskn_kv4_peer_exchange* x, int M, int nh, int g, int hd, const uint16_t* bv, const uint16_t* gate,
                        uint16_t* o16, int act_dtype, cudaStream_t st);
int launch_exchange_merge(const yskn_attn_g_combine_args& a, int hd, int act_dtype, const yskn_kv4_peer_exchange* x, cudaStream_t st);
int merge_status_fetch(int* out);
void set_peer_wait_polls(unsigned polls);

// Family-B row codec, step 1 (kvx_codec.cu)
int launch_copy16(void* dst, const void* src, size_t bytes, cudaStream_t st);
int launch_kvx_rotate(const float* x, float* y, long long rows, int inverse, cudaStream_t st);
int launch_kvx_encode(const void* x, int x_dtype, int8_t* q8, float* scales, long long rows, cudaStream_t st);
int launch_kvx_decode(const int8_t* q8, const float* scales, void* y, int y_dtype, long long rows, cudaStream_t st);
int launch_kvx_attn_post(const yskn_kvx_attn_post_args& a, cudaStream_t st);

// Family-B row codec, step 2: trellis re-quantisation and payload (kvq_trellis.cu)
size_t tb_scratch_bytes(int rows, int nm);
int tb_blob_info(const uint8_t* h_blob, size_t n, int* nm);
int launch_tb_attention(const yskn_tb_attn_args& a, int act_dtype, cudaStream_t st);
int launch_tb_encode(const uint8_t* blob, int nm, const float* x, const int* grp, const int* pos, int rows, float* y, uint8_t* pay, int pay_stride,
                     uint32_t* side, void* scratch, size_t scratch_bytes, cudaStream_t st);

int launch_tb_decode(const uint8_t* blob, const int* grp, const int* pos, const uint8_t* pay, int pay_stride, const uint32_t* side, const float* yin,
                     float* y, int rows, cudaStream_t st);

// Family-B decode attention over INT8 rows (kv8_decode.cu)
int launch_kv8_attention(const yskn_kv8_attn_args& a, int act_dtype, cudaStream_t st);
int launch_kv8_attention_tc(const yskn_kv8_attn_args& a, int act_dtype, cudaStream_t st);   // kv4_tc.cu, many rows
int launch_kv8_combine(const float* pm, const float* pl, const float* pacc, int splits, int M, int nh, const void* gate, void* o16,
                       int act_dtype, int inverse_rotate, cudaStream_t st);

// Which attention kernel yskn_kv4_attention picks; set through yskn_kv4_set_algo (tests compare paths).
enum Algo { ALGO_AUTO = 0, ALGO_SCALAR = 1, ALGO_MMA = 2 };
int current_algo();

}  // namespace kv4
