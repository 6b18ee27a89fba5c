// Input quantisation of the projection that follows attention (sm_100a): per 512 values of a merged attention row, sign
// flip, Walsh-Hadamard transform of length 512, fp16 rounding, int8 codes with one fp32 scale.
//
// Restates the tail of the reference's merge kernels (attn_combine_gqa_xform_kernel, src/attention_gqa.cu:135-139, through
// a8_group512_tail, src/a8_prologue.cuh:122-133, and fwht512_v, :86-98), which the reference runs inside the merge kernel.
// Here it is a launch of its own right behind the merge (programmatic stream serialization, like the reference's PDL
// launches): the merge kernel's blocks own one head of 64-256 channels each, a 512-group spans two or more of them.
// Bit-exact: every butterfly adds or subtracts the same two fp32 values in the same stage order h = 1 .. 256 (the upper
// element of a pair gets lower - upper), the scaling, rounding and division are the reference's explicit RN operations.
#include "kv4_common.cuh"

namespace kv4 {
namespace {

__global__ void __launch_bounds__(512) kv4_xform_a8_kernel(const uint16_t* __restrict__ o16, const int8_t* __restrict__ signs,
                                                           int8_t* __restrict__ qx, float* __restrict__ alpha, int n) {
  __shared__ float b0[512], b1[512];
  __shared__ unsigned s_amax;
  const int blk = blockIdx.x, tok = blockIdx.y, p = threadIdx.x, lane = p & 31, ng = n / 512;
  asm volatile("griddepcontrol.wait;" ::: "memory");                 // o16 comes from the merge kernel just before
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (p == 0) s_amax = 0u;
  const size_t e = (size_t)tok * n + (size_t)blk * 512 + p;
  float v = __fmul_rn(h2f(o16[e]), (float)signs[blk * 512 + p]);
  #pragma unroll
  for (int h = 1; h < 32; h <<= 1) { const float q = __shfl_xor_sync(0xffffffffu, v, h); v = (lane & h) ? __fsub_rn(q, v) : __fadd_rn(v, q); }
  #pragma unroll
  for (int h = 32; h < 512; h <<= 1) {
    float* const b = (h == 32 || h == 128) ? b0 : b1;               // two buffers: a stage may overwrite what the stage before last read
    b[p] = v; __syncthreads();
    const float q = b[p ^ h]; v = (p & h) ? __fsub_rn(q, v) : __fadd_rn(v, q);
  }
  v = round_f16(__fmul_rn(v, 0.044194173824159216f));               // 1 / sqrt(512)
  unsigned mx = __float_as_uint(fabsf(v));
  #pragma unroll
  for (int o = 16; o; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) atomicMax(&s_amax, mx);
  __syncthreads();
  const float al = __fdiv_rn(__uint_as_float(s_amax), 127.f);
  if (p == 0) alpha[(size_t)tok * ng + blk] = al;
  const float r = al > 0.f ? __fdiv_rn(v, al) : 0.f;
  int q = __float2int_rn(r); q = q < -127 ? -127 : (q > 127 ? 127 : q);
  qx[e] = (int8_t)q;
}

}  // namespace

int launch_xform_a8(const uint16_t* o16, const int8_t* signs, int8_t* qx, float* alpha, int M, int n, cudaStream_t st) {
  if (!o16 || !signs || !qx || !alpha) KV4_REJECT("yskn_kv4_xform_a8: null buffer");
  if (M <= 0 || M > 65535 || n <= 0 || n % 512) KV4_REJECT("yskn_kv4_xform_a8: bad shape (M %d, row length %d must be a multiple of 512)", M, n);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(n / 512, M); cfg.blockDim = dim3(512); cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  KV4_CUDA(cudaLaunchKernelEx(&cfg, kv4_xform_a8_kernel, o16, signs, qx, alpha, n));
  return launch_status("kv4_xform_a8_kernel");
}

}  // namespace kv4
