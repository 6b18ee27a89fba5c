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
