// TEST INFRASTRUCTURE, NOT PRODUCT.
// C entry point around the reference's Family-B decode launcher (launch_q35_attention, INT8 branch), compiled together
// with the reference's src/q35_kernels.cu where it lies (oracle/Makefile, target `ref`).  Pins the CPU oracle of the
// INT8-row attention and this library's kernel against the reference's own kernel on a GPU.  No product code.
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include "q35.hpp"           // reference: src/q35.hpp (Q35AttnArgs, Q35_NH = 24, Q35_KVH = 4, Q35_HD = 256)

namespace yskn {
bool pdl_enabled() { return false; }   // defined in the reference's engine.cpp, which is not compiled here
}

extern "C" int yref_q35_shape(int* nh, int* kvh, int* hd) { *nh = yskn::Q35_NH; *kvh = yskn::Q35_KVH; *hd = yskn::Q35_HD; return 0; }

// src/q35_kernels.cu:1279-1281; q16 bf16 [M][24][256], k8/v8 int8 [4][max_ctx][256], ks/vs f32 [4][max_ctx]
extern "C" int yref_q35_attention_kv8(const uint16_t* q16, const int8_t* k8, const int8_t* v8, const float* ks, const float* vs,
                                      int max_ctx, int M, const int* d_pos, int splits, float* pm, float* pl, float* pacc, void* st) {
  yskn::Q35AttnArgs A{};
  A.q16 = q16; A.kc = nullptr; A.vc = nullptr; A.max_ctx = max_ctx; A.M = M; A.d_pos = d_pos; A.splits = splits;
  A.pm = pm; A.pl = pl; A.pacc = pacc; A.early = 0; A.k8 = k8; A.v8 = v8; A.ks = ks; A.vs = vs;
  try { yskn::launch_q35_attention(A, (cudaStream_t)st); } catch (const std::exception&) { return -1; }
  return (int)cudaGetLastError();
}

// src/q35_kernels.cu:1013-1069 (launch_q35_attn_post, the plain kernel: no xsm, no prefetch, INT8 row caches).  One GEMV
// slice (nw = 1) and tau = 1 (`ones`, at least 24 * 512 floats), signs all +1 (`signs`, at least 24 * 512 bytes), so that a
// block's 512 projection values are bf16(H512(part) / sqrt(512)).  part_q [M][24 * 512], part_k / part_v [M][4 * 256].
// pm selects the kernel's portable-math mode (q35_set_pm, src/q35_kernels.cu:1139).
extern "C" int yref_q35_attn_post(const float* part_q, const float* part_k, const float* part_v, const float* ones, const int8_t* signs,
                                  const uint16_t* qn_w, const uint16_t* kn_w, float eps, int M, const int* d_pos, const float* rope,
                                  uint16_t* q16, uint16_t* gate16, int8_t* k8, int8_t* v8, float* ks, float* vs, int max_ctx, int pm, void* st) {
  yskn::Q35AttnPostArgs A{};
  A.part_q = part_q; A.part_k = part_k; A.part_v = part_v; A.tau_q = ones; A.tau_k = ones; A.tau_v = ones;
  A.nw_q = 1; A.nw_k = 1; A.nw_v = 1; A.sg_q = signs; A.sg_k = signs; A.sg_v = signs; A.qn_w = qn_w; A.kn_w = kn_w;
  A.eps = eps; A.M = M; A.d_pos = d_pos; A.rope = reinterpret_cast<const float2*>(rope); A.q16 = q16; A.gate16 = gate16;
  A.kc = nullptr; A.vc = nullptr; A.max_ctx = max_ctx; A.k8 = k8; A.v8 = v8; A.ks = ks; A.vs = vs;
  try { yskn::q35_set_pm(pm, (cudaStream_t)st); yskn::launch_q35_attn_post(A, (cudaStream_t)st); } catch (const std::exception&) { return -1; }
  return (int)cudaGetLastError();
}
