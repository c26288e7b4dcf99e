// Eligibility test and layout dispatch of the 128x128 streaming kernel; the
// kernels themselves are instantiated in carry_gdn_tile128_vk.cu / _kv.cu.
#include "carry_gdn_common.cuh"

namespace carry {

int launch_tile128_vk(const KParams& p, cudaStream_t stream, int sms);
int launch_tile128_kv(const KParams& p, cudaStream_t stream, int sms);

namespace {
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
}  // namespace

// The streaming kernel needs K = V = 128, an integer residual (any residual format in the statequant
// layout), a per-V state
// scale, qmax = 2^(bits-1) - 1 for 3..8 bits, and 16-byte aligned, dense rows for every bulk copy.
bool tile128_eligible(const KParams& p) {
  if (p.K != 128 || p.V != 128) return false;
  const bool int_resid = p.res_fmt == CARRY_RES_INT8 || p.res_fmt == CARRY_RES_INT4;
  const bool float_resid = p.res_fmt == CARRY_RES_FP32 || p.res_fmt == CARRY_RES_FP16 || p.res_fmt == CARRY_RES_FP8;
  if (!int_resid && !(float_resid && !p.packed)) return false;   // float residuals: statequant layout only
  if (p.sscale_mode != CARRY_SCALE_PER_V) return false;
  // the kernel divides by qmax with a multiply and a correcting fused multiply-add, which equals the
  // IEEE quotient for these values (the quantisation widths 3..8 bits) and has not been checked for others
  if (p.qmax != 3.f && p.qmax != 7.f && p.qmax != 15.f && p.qmax != 31.f && p.qmax != 63.f && p.qmax != 127.f)
    return false;
  if (p.HV > 128 || (long long)p.B * p.HV > 0x7fffffffLL) return false;
  const int qes = p.qkv_dtype == CARRY_F32 ? 4 : 2;
  if (!aligned16(p.codes_in) || !aligned16(p.codes_out) || !aligned16(p.resid_in) || !aligned16(p.resid_out) ||
      !aligned16(p.sscale_in) || !aligned16(p.sscale_out) ||
      (int_resid && (!aligned16(p.rscale_in) || !aligned16(p.rscale_out))) ||
      !aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.out))
    return false;
  if (p.packed) {
    if ((p.stride_mixed_tok * qes) % 16) return false;
    if (p.stride_state_slot % 16 || p.stride_resid_slot % 16 || p.stride_sscale_slot % 4) return false;
    if (p.rscale_mode == CARRY_SCALE_PER_V ? (p.stride_rscale_slot % 4) : (p.stride_rscale_slot % 4 || p.HV % 4))
      return false;
  } else {
    if (int_resid && p.rscale_mode == CARRY_SCALE_PER_HEAD && p.HV % 4) return false;
  }
  return true;
}

int launch_tile128(const KParams& p, cudaStream_t stream) {
  static thread_local int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return CARRY_GDN_ERR_NO_DEVICE;
  if (dev >= 64) return CARRY_GDN_ERR_NO_DEVICE;
  if (sms[dev] == 0) {
    if (cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms[dev] <= 0) {
      cudaGetLastError();
      sms[dev] = 0;
      return CARRY_GDN_ERR_NO_DEVICE;
    }
  }
  KParams q = p;
  auto log2_or_minus1 = [](int x) { int s = 0; while ((1 << s) < x) ++s; return (1 << s) == x ? s : -1; };
  q.hv_shift = log2_or_minus1(p.HV);
  q.group = p.HV / p.H;
  q.group_shift = log2_or_minus1(q.group);
  return q.packed ? launch_tile128_vk(q, stream, sms[dev]) : launch_tile128_kv(q, stream, sms[dev]);
}

}  // namespace carry
