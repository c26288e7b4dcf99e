// placeholder: streaming kernel not built yet
#include "carry_gdn_common.cuh"
namespace carry {
bool tile128_eligible(const KParams&) { return false; }
int launch_tile128(const KParams&, cudaStream_t) { return CARRY_GDN_ERR_UNSUPPORTED; }
}
