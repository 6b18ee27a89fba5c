// TEST INFRASTRUCTURE, NOT PRODUCT.
// Link glue for the reference's trellis probes (yskn_tb_probe, yskn_tb_probe2, yskn_tbp_pack_unpack in src/kvx_probe.cu,
// built with YSKN_KVX_MODE=3) compiled together with the reference's src/q35_kernels.cu where they lie (oracle/Makefile,
// target `ref`).  The probe file also holds attention benches that call launchers from translation units which take minutes
// to compile and are not needed here; they are given definitions that refuse to run.  No product code.
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include "q35.hpp"
#include "q35_atxpk.hpp"

namespace yskn {
bool pdl_enabled() { return false; }   // defined in the reference's engine.cpp, which is not compiled here
void launch_q35_atx(const Q35AttnArgs&, const uint8_t*, cudaStream_t) { throw std::runtime_error("launch_q35_atx: not built into this test library"); }
void launch_q35_atx_pk(const Q35AttnArgs&, const uint8_t*, const Q35PkArgs&, cudaStream_t) { throw std::runtime_error("launch_q35_atx_pk: not built into this test library"); }
}
