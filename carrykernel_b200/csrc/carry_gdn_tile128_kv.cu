// Streaming kernel, statequant layout [K][V] (every residual format, scale mode
// and activation type): see carry_gdn_tile128.cuh.
#include "carry_gdn_tile128.cuh"

namespace carry {
int launch_tile128_kv(const KParams& p, cudaStream_t stream, int sms) {
  return launch_layout<LAYOUT_KV>(p, stream, sms);
}
}  // namespace carry
