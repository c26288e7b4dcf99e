// Streaming kernel, slot layout [V][K] (every residual format, scale mode and
// activation type): see carry_gdn_tile128.cuh.
#include "carry_gdn_tile128.cuh"

namespace carry {
int launch_tile128_vk(const KParams& p, cudaStream_t stream, int sms) {
  return launch_layout<LAYOUT_VK>(p, stream, sms);
}
}  // namespace carry

#ifdef CARRY_TEST_WAIT_EXPIRY
// Test-only (twin library): a kernel that lets the launch behind it in the stream start at once, idles for
// `delay_ns` (at most 0.2 ms), and only then copies `bytes` (a multiple of 16) from src to dst -- a
// predecessor that is still writing the streaming kernel's inputs while that kernel takes its first look
// at them ahead of its dependency wait.
namespace carry {
namespace {
__global__ void late_writer_kernel(uint4* dst, const uint4* src, long long n16, unsigned delay_ns) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (unsigned waited = 0; waited < delay_ns; waited += 1000) __nanosleep(1000);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i];
}
}  // namespace
}  // namespace carry
extern "C" int carry_gdn_test_late_writer(void* dst, const void* src, long long bytes, unsigned delay_ns, void* stream) {
  if (bytes < 0 || bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) % 16 != 0)
    return CARRY_GDN_ERR_SHAPE;
  if (delay_ns > 200000u) delay_ns = 200000u;
  carry::late_writer_kernel<<<8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(dst), static_cast<const uint4*>(src), bytes / 16, delay_ns);
  return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
}
#endif
