#include "kv4_common.cuh"
namespace kv4 {
bool decode_mma_supports(int, int, int, int) { return false; }
int launch_decode_mma(const yskn_attn_g_args&, int, int, int, int, Shard, cudaStream_t) { KV4_REJECT("decode mma: not built"); }
}
