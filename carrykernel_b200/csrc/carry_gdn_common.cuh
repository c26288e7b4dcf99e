// Shared device helpers and the kernel-side parameter block for the fused
// Gated-DeltaNet decode step (INT8 state + error-feedback residual), sm_100a.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/carry_gdn.h"

namespace carry {

constexpr float kEps = 1e-12f;
constexpr float kSoftplusThreshold = 20.0f;

// Everything a kernel needs, for both front ends.  `packed == 0`: statequant
// layout [B,HV,K,V], alpha/beta given.  `packed == 1`: slot pool [slots,HV,V,K],
// gates derived in the kernel from a, b, A_log, dt_bias.
struct KParams {
  int packed;
  int B, H, HV, K, V;
  int hv_shift;      // log2(HV) when HV is a power of two, else -1       (filled by tile128's launcher;
  int group;         // value heads per key head, HV / H                    the streaming kernel splits tile
  int group_shift;   // log2(group) when that is a power of two, else -1    indices without dividing)
  float qmax;
  float inv_qmax;    // 1 / qmax rounded to nearest, worked out on the host (the streaming kernels multiply by it)
  int res_fmt, rscale_mode, sscale_mode, eps_mode;
  int qkv_dtype, o_dtype;
  int* status;
  // state (for the statequant layout `*_out` may differ from `*_in`)
  const int8_t* codes_in;
  int8_t* codes_out;
  const float* sscale_in;
  float* sscale_out;
  const void* resid_in;
  void* resid_out;
  const float* rscale_in;
  float* rscale_out;
  long long stride_state_slot, stride_resid_slot, stride_sscale_slot, stride_rscale_slot;
  // activations
  const void* q;
  const void* k;
  const void* v;
  long long stride_mixed_tok;
  const float* alpha;
  const float* beta;
  const void* a;
  const void* b;
  long long stride_a_tok, stride_b_tok;
  int ab_dtype;
  const void* A_log;
  const void* dt_bias;
  int A_log_dtype, dt_bias_dtype;
  float qscale;
  int l2norm;
  const int* slot_idx;
  long long stride_idx;
  int num_slots;
  void* out;
};

__device__ __forceinline__ float load_as_float(const void* p, long long i, int dtype) {
  if (dtype == CARRY_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == CARRY_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, long long i, int dtype, float x) {
  if (dtype == CARRY_F32) reinterpret_cast<float*>(p)[i] = x;
  else if (dtype == CARRY_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(x);
}

// scale from an absolute maximum, with the floor applied where the front end's
// reference applies it
__device__ __forceinline__ float scale_from_amax(float amax, float qmax, int eps_mode) {
  if (eps_mode == CARRY_EPS_ON_AMAX) return __fdiv_rn(fmaxf(amax, kEps), qmax);
  return fmaxf(__fdiv_rn(amax, qmax), kEps);
}

// round(x / s) with torch.round semantics (half to even), then the symmetric clamp
__device__ __forceinline__ float quantize_div(float x, float s, float qmax) {
  return fminf(fmaxf(rintf(__fdiv_rn(x, s)), -qmax), qmax);
}

// in-kernel gates of the slot path: decay = exp(-exp(A_log) * softplus(a + dt_bias)),
// write strength = sigmoid(b)
__device__ __forceinline__ void slot_gates(float a, float b, float A_log, float dt_bias,
                                           float& alpha, float& beta) {
  const float x = a + dt_bias;
  const float sp = (x <= kSoftplusThreshold) ? logf(1.0f + expf(x)) : x;
  const float g = -expf(A_log) * sp;
  alpha = expf(g);
  beta = __fdiv_rn(1.0f, 1.0f + expf(-b));
}

// Resolved addresses of one (request, head) tile.
struct Tile {
  bool skip;            // padding slot: write zeros to out, touch nothing else
  const int8_t* codes_in;
  int8_t* codes_out;
  const float* sscale_in;
  float* sscale_out;
  const uint8_t* resid_in;
  uint8_t* resid_out;
  const float* rscale_in;
  float* rscale_out;
  const void* q;        // already offset to this head (element index 0)
  const void* k;
  const void* v;
  long long q_off, k_off, v_off;   // element offsets into q/k/v base pointers
  long long out_off;    // element offset into out
  float alpha, beta;
};

__device__ __forceinline__ int resid_bytes_per_elem_x2(int res_fmt) {
  // twice the bytes per element, so INT4 is representable
  switch (res_fmt) {
    case CARRY_RES_FP32: return 8;
    case CARRY_RES_FP16: return 4;
    case CARRY_RES_FP8: return 2;
    case CARRY_RES_INT8: return 2;
    case CARRY_RES_INT4: return 1;
    default: return 0;
  }
}

__device__ __forceinline__ Tile resolve_tile(const KParams& p, int n, int hv) {
  Tile t;
  t.skip = false;
  const long long KV = (long long)p.K * p.V;
  const int rb2 = resid_bytes_per_elem_x2(p.res_fmt);
  if (!p.packed) {
    const long long nh = (long long)n * p.HV + hv;
    t.codes_in = p.codes_in + nh * KV;
    t.codes_out = p.codes_out + nh * KV;
    const long long ss = (p.sscale_mode == CARRY_SCALE_PER_V) ? nh * p.V : nh;
    t.sscale_in = p.sscale_in + ss;
    t.sscale_out = p.sscale_out + ss;
    t.resid_in = reinterpret_cast<const uint8_t*>(p.resid_in) + nh * KV * rb2 / 2;
    t.resid_out = reinterpret_cast<uint8_t*>(p.resid_out) + nh * KV * rb2 / 2;
    const long long rs = (p.rscale_mode == CARRY_SCALE_PER_V) ? nh * p.V : nh;
    t.rscale_in = p.rscale_in ? p.rscale_in + rs : nullptr;
    t.rscale_out = p.rscale_out ? p.rscale_out + rs : nullptr;
    t.q_off = nh * p.K;
    t.k_off = nh * p.K;
    t.v_off = nh * p.V;
    t.out_off = nh * p.V;
    t.alpha = p.alpha[nh];
    t.beta = p.beta[nh];
    return t;
  }
  const long long slot = p.slot_idx[(long long)n * p.stride_idx];
  t.out_off = ((long long)n * p.HV + hv) * p.V;
  if (slot <= 0 || slot >= p.num_slots) {
    if (slot >= p.num_slots && p.status) atomicOr(p.status, CARRY_GDN_STATUS_BAD_SLOT);
    t.skip = true;
    return t;
  }
  t.codes_in = p.codes_in + slot * p.stride_state_slot + (long long)hv * KV;
  t.codes_out = const_cast<int8_t*>(t.codes_in);
  t.sscale_in = p.sscale_in + slot * p.stride_sscale_slot + (long long)hv * p.V;
  t.sscale_out = const_cast<float*>(t.sscale_in);
  t.resid_in = reinterpret_cast<const uint8_t*>(p.resid_in) + slot * p.stride_resid_slot +
               (long long)hv * KV * rb2 / 2;
  t.resid_out = const_cast<uint8_t*>(t.resid_in);
  t.rscale_in = p.rscale_in + slot * p.stride_rscale_slot +
                ((p.rscale_mode == CARRY_SCALE_PER_V) ? (long long)hv * p.V : (long long)hv);
  t.rscale_out = const_cast<float*>(t.rscale_in);
  const int h = hv / (p.HV / p.H);
  const long long row = (long long)n * p.stride_mixed_tok;
  t.q_off = row + (long long)h * p.K;
  t.k_off = row + (long long)p.H * p.K + (long long)h * p.K;
  t.v_off = row + 2LL * p.H * p.K + (long long)hv * p.V;
  const float a = load_as_float(p.a, (long long)n * p.stride_a_tok + hv, p.ab_dtype);
  const float b = load_as_float(p.b, (long long)n * p.stride_b_tok + hv, p.ab_dtype);
  slot_gates(a, b, load_as_float(p.A_log, hv, p.A_log_dtype),
             load_as_float(p.dt_bias, hv, p.dt_bias_dtype), t.alpha, t.beta);
  return t;
}

// kernels / launchers implemented in the other translation units
int launch_generic(const KParams& p, cudaStream_t stream);
int launch_fp32(const CarryGdnFp32Args& a, cudaStream_t stream);
bool tile128_eligible(const KParams& p);
int launch_tile128(const KParams& p, cudaStream_t stream);
int launch_multi(const KParams& p, int T, long long stride_mixed_t, long long stride_a_t, long long stride_b_t,
                 cudaStream_t stream);
bool noef128_eligible(const KParams& p);
int launch_noef128(const KParams& p, cudaStream_t stream);
int launch_pool_store(const CarryGdnPoolStoreArgs& a, cudaStream_t stream);
int launch_pool_load(const CarryGdnPoolLoadArgs& a, cudaStream_t stream);
int launch_pool_copy(const CarryGdnPoolCopyArgs& a, cudaStream_t stream);

}  // namespace carry
