// Generic tile kernels: any K, V that fits one SM's shared memory, every
// residual format, both memory layouts, both scale granularities.  One CTA owns
// one (request, head) tile, stages it in shared memory as fp32 and keeps the
// reference's operation order: (code*scale)*alpha, h + (k*dv) with the product
// rounded first, true division before round-half-to-even.
//
// These are the correctness-first kernels.  The 128x128 streaming kernel in
// carry_gdn_tile128.cu is the fast path for the serving shapes; both are CUDA,
// there is no CPU fallback behind either.
#include "carry_gdn_common.cuh"

namespace carry {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_max(float x, float* red) {
  // red: kThreads/32 floats of shared memory
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, red[i]);
  return m;
}

__device__ __forceinline__ float block_sum(float x, float* red) {
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) m += red[i];
  return m;
}

__device__ __forceinline__ float decode_resid(const uint8_t* base, long long idx, int fmt) {
  switch (fmt) {
    case CARRY_RES_FP32: return reinterpret_cast<const float*>(base)[idx];
    case CARRY_RES_FP16: return __half2float(reinterpret_cast<const __half*>(base)[idx]);
    case CARRY_RES_FP8: return static_cast<float>(reinterpret_cast<const __nv_fp8_e5m2*>(base)[idx]);
    case CARRY_RES_INT8: return static_cast<float>(reinterpret_cast<const int8_t*>(base)[idx]);
    case CARRY_RES_INT4: {
      const int byte = base[idx >> 1];
      int nib = (idx & 1) ? (byte >> 4) : (byte & 0xF);
      if (nib > 7) nib -= 16;
      return static_cast<float>(nib);
    }
    default: return 0.f;
  }
}

// Tile element (kk, vv) sits at kk*V + vv in the statequant layout and at
// vv*K + kk in the slot layout.  In shared memory it always sits at
// kk*(V+1) + vv: the column walks below are conflict-free and both memory
// orders load and store without bank conflicts.
__global__ void __launch_bounds__(kThreads) gdn_generic_kernel(const __grid_constant__ KParams p) {
  extern __shared__ float smem[];
  const int K = p.K, V = p.V, LD = V + 1;
  float* T = smem;                     // [K][LD] state -> target -> codes
  float* E = T + (size_t)K * LD;       // [K][LD] residual -> new residual -> residual codes
  float* sk = E + (size_t)K * LD;      // [K]
  float* sq = sk + K;                  // [K]
  float* sv = sq + K;                  // [V]
  float* red = sv + V;                 // [8]

  const int tid = threadIdx.x;
  const int n = blockIdx.x / p.HV, hv = blockIdx.x % p.HV;
  const Tile t = resolve_tile(p, n, hv);
  if (t.skip) {
    for (int i = tid; i < V; i += kThreads) store_from_float(p.out, t.out_off + i, p.o_dtype, 0.f);
    return;
  }
  const int KV = K * V;
  const bool has_resid = p.res_fmt != CARRY_RES_NONE;
  const bool int_resid = p.res_fmt == CARRY_RES_INT8 || p.res_fmt == CARRY_RES_INT4;
  const float head_sscale = (p.sscale_mode == CARRY_SCALE_PER_HEAD) ? t.sscale_in[0] : 0.f;
  const float head_rscale =
      (int_resid && p.rscale_mode == CARRY_SCALE_PER_HEAD) ? t.rscale_in[0] : 0.f;

  // ---- vectors --------------------------------------------------------------
  float qss = 0.f, kss = 0.f;
  for (int i = tid; i < K; i += kThreads) {
    const float qv = load_as_float(p.q, t.q_off + i, p.qkv_dtype);
    const float kv = load_as_float(p.k, t.k_off + i, p.qkv_dtype);
    sq[i] = qv;
    sk[i] = kv;
    qss += qv * qv;
    kss += kv * kv;
  }
  for (int i = tid; i < V; i += kThreads) sv[i] = load_as_float(p.v, t.v_off + i, p.qkv_dtype);
  if (p.packed) {
    if (p.l2norm) {
      const float qn = sqrtf(block_sum(qss, red) + 1e-6f);
      const float kn = sqrtf(block_sum(kss, red) + 1e-6f);
      for (int i = tid; i < K; i += kThreads) {
        sq[i] = __fdiv_rn(sq[i], qn) * p.qscale;
        sk[i] = __fdiv_rn(sk[i], kn);
      }
    } else {
      __syncthreads();
      for (int i = tid; i < K; i += kThreads) sq[i] = sq[i] * p.qscale;
    }
  }

  // ---- load: dequantise + decay, residual to fp32 ---------------------------
  for (int idx = tid; idx < KV; idx += kThreads) {
    int kk, vv;
    if (p.packed) { vv = idx / K; kk = idx - vv * K; } else { kk = idx / V; vv = idx - kk * V; }
    const float s = (p.sscale_mode == CARRY_SCALE_PER_V) ? t.sscale_in[vv] : head_sscale;
    const float c = static_cast<float>(t.codes_in[idx]);
    T[kk * LD + vv] = __fmul_rn(__fmul_rn(c, s), t.alpha);
    float e = 0.f;
    if (has_resid) {
      e = decode_resid(t.resid_in, idx, p.res_fmt);
      if (int_resid)
        e = __fmul_rn(e, (p.rscale_mode == CARRY_SCALE_PER_V) ? t.rscale_in[vv] : head_rscale);
    }
    E[kk * LD + vv] = e;
  }
  __syncthreads();

  // ---- per-column recurrence; target = h' + e -------------------------------
  float amax_local = 0.f;
  for (int vv = tid; vv < V; vv += kThreads) {
    float read = 0.f;
    for (int kk = 0; kk < K; ++kk) read = fmaf(T[kk * LD + vv], sk[kk], read);
    const float dv = __fmul_rn(t.beta, __fadd_rn(sv[vv], -read));
    float o = 0.f, amax = 0.f;
    for (int kk = 0; kk < K; ++kk) {
      const float hn = __fadd_rn(T[kk * LD + vv], __fmul_rn(sk[kk], dv));
      o = fmaf(hn, sq[kk], o);
      const float tg = has_resid ? __fadd_rn(hn, E[kk * LD + vv]) : hn;
      T[kk * LD + vv] = tg;
      amax = fmaxf(amax, fabsf(tg));
    }
    store_from_float(p.out, t.out_off + vv, p.o_dtype, o);
    sv[vv] = amax;                       // column amax, reused below
    amax_local = fmaxf(amax_local, amax);
  }
  float head_amax = 0.f;
  if (p.sscale_mode == CARRY_SCALE_PER_HEAD) head_amax = block_max(amax_local, red);

  // ---- quantise the state, form the new residual -----------------------------
  float eamax_local = 0.f;
  for (int vv = tid; vv < V; vv += kThreads) {
    const float s_new = scale_from_amax(
        (p.sscale_mode == CARRY_SCALE_PER_V) ? sv[vv] : head_amax, p.qmax, p.eps_mode);
    if (p.sscale_mode == CARRY_SCALE_PER_V) t.sscale_out[vv] = s_new;
    else if (vv == 0) t.sscale_out[0] = s_new;
    float eamax = 0.f;
    for (int kk = 0; kk < K; ++kk) {
      const float tg = T[kk * LD + vv];
      const float code = quantize_div(tg, s_new, p.qmax);
      T[kk * LD + vv] = code;
      const float en = __fadd_rn(tg, -__fmul_rn(code, s_new));
      E[kk * LD + vv] = en;
      eamax = fmaxf(eamax, fabsf(en));
    }
    sv[vv] = eamax;
    eamax_local = fmaxf(eamax_local, eamax);
  }
  if (int_resid) {
    const float rq = (p.res_fmt == CARRY_RES_INT4) ? 7.0f : 127.0f;
    float head_eamax = 0.f;
    if (p.rscale_mode == CARRY_SCALE_PER_HEAD) head_eamax = block_max(eamax_local, red);
    for (int vv = tid; vv < V; vv += kThreads) {
      const float es = scale_from_amax(
          (p.rscale_mode == CARRY_SCALE_PER_V) ? sv[vv] : head_eamax, rq, p.eps_mode);
      if (p.rscale_mode == CARRY_SCALE_PER_V) t.rscale_out[vv] = es;
      else if (vv == 0) t.rscale_out[0] = es;
      for (int kk = 0; kk < K; ++kk) E[kk * LD + vv] = quantize_div(E[kk * LD + vv], es, rq);
    }
  }
  __syncthreads();

  // ---- store in memory order -------------------------------------------------
  for (int idx = tid; idx < KV; idx += kThreads) {
    int kk, vv;
    if (p.packed) { vv = idx / K; kk = idx - vv * K; } else { kk = idx / V; vv = idx - kk * V; }
    t.codes_out[idx] = static_cast<int8_t>(T[kk * LD + vv]);
    const float e = E[kk * LD + vv];
    switch (p.res_fmt) {
      case CARRY_RES_FP32: reinterpret_cast<float*>(t.resid_out)[idx] = e; break;
      case CARRY_RES_FP16: reinterpret_cast<__half*>(t.resid_out)[idx] = __float2half_rn(e); break;
      case CARRY_RES_FP8: reinterpret_cast<__nv_fp8_e5m2*>(t.resid_out)[idx] = __nv_fp8_e5m2(e); break;
      case CARRY_RES_INT8: reinterpret_cast<int8_t*>(t.resid_out)[idx] = static_cast<int8_t>(e); break;
      default: break;
    }
  }
  if (p.res_fmt == CARRY_RES_INT4) {
    // consecutive memory-order indices (2j, 2j+1) share a byte: even index low nibble
    for (int j = tid; j < KV / 2; j += kThreads) {
      int kk0, vv0, kk1, vv1;
      const int i0 = 2 * j, i1 = 2 * j + 1;
      if (p.packed) { vv0 = i0 / K; kk0 = i0 - vv0 * K; vv1 = i1 / K; kk1 = i1 - vv1 * K; }
      else { kk0 = i0 / V; vv0 = i0 - kk0 * V; kk1 = i1 / V; vv1 = i1 - kk1 * V; }
      const int lo = static_cast<int>(E[kk0 * LD + vv0]) & 0xF;
      const int hi = static_cast<int>(E[kk1 * LD + vv1]) & 0xF;
      t.resid_out[j] = static_cast<uint8_t>(lo | (hi << 4));
    }
  }
}

// fp32 state, no quantisation: h' = alpha*h + k (beta (v - (alpha*h)^T k))^T, o = h'^T q
__global__ void __launch_bounds__(kThreads) gdn_fp32_kernel(const __grid_constant__ CarryGdnFp32Args a) {
  extern __shared__ float smem[];
  const int K = a.K, V = a.V;
  float* T = smem;          // [K][V]
  float* sk = T + (size_t)K * V;
  float* sq = sk + K;
  const int tid = threadIdx.x;
  const long long nh = blockIdx.x;
  const float alpha = a.alpha[nh], beta = a.beta[nh];
  const float* hin = a.h_in + nh * K * V;
  float* hout = a.h_out + nh * K * V;
  for (int i = tid; i < K; i += kThreads) {
    sk[i] = load_as_float(a.k, nh * K + i, a.qkv_dtype);
    sq[i] = load_as_float(a.q, nh * K + i, a.qkv_dtype);
  }
  for (int idx = tid; idx < K * V; idx += kThreads) T[idx] = __fmul_rn(alpha, hin[idx]);
  __syncthreads();
  for (int vv = tid; vv < V; vv += kThreads) {
    float read = 0.f;
    for (int kk = 0; kk < K; ++kk) read = fmaf(T[kk * V + vv], sk[kk], read);
    const float dv = __fmul_rn(beta, __fadd_rn(load_as_float(a.v, nh * V + vv, a.qkv_dtype), -read));
    float o = 0.f;
    for (int kk = 0; kk < K; ++kk) {
      const float hn = __fadd_rn(T[kk * V + vv], __fmul_rn(sk[kk], dv));
      T[kk * V + vv] = hn;
      o = fmaf(hn, sq[kk], o);
    }
    store_from_float(a.o, nh * V + vv, a.o_dtype, o);
  }
  __syncthreads();
  for (int idx = tid; idx < K * V; idx += kThreads) hout[idx] = T[idx];
}

// The same step for K = V = 128 as a streaming kernel: the tile never sits in shared memory.
// A CTA of 8 warps takes one (request, head) tile; a lane holds 4 consecutive columns of 16
// rows (rows warp, warp + 8, ...: 64 state values in registers, 16 independent 16-byte reads
// in flight per thread).  The two sums over K -- (alpha h)^T k and h'^T q -- are finished
// across the warps through 4 KB of shared memory.  Each state element is read once and
// written once; h_out may alias h_in (a thread reads its elements before it writes them).
constexpr int kF = 128;
__global__ void __launch_bounds__(kThreads, 2) gdn_fp32_tile128_kernel(const __grid_constant__ CarryGdnFp32Args a) {
  __shared__ __align__(16) float red[kThreads / 32][kF];
  __shared__ __align__(16) float sk[kF], sq[kF], sdv[kF];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, c0 = 4 * lane;
  const long long tiles = (long long)a.B * a.HV;
  for (long long nh = blockIdx.x; nh < tiles; nh += gridDim.x) {
    const float* hin = a.h_in + nh * kF * kF;
    float* hout = a.h_out + nh * kF * kF;
    float4 h[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) h[j] = *reinterpret_cast<const float4*>(hin + (warp + 8 * j) * kF + c0);
    if (tid < kF) {
      sk[tid] = load_as_float(a.k, nh * kF + tid, a.qkv_dtype);
      sq[tid] = load_as_float(a.q, nh * kF + tid, a.qkv_dtype);
    }
    const float alpha = a.alpha[nh], beta = a.beta[nh];
    __syncthreads();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float kk = sk[warp + 8 * j];
      h[j].x = __fmul_rn(alpha, h[j].x); h[j].y = __fmul_rn(alpha, h[j].y);
      h[j].z = __fmul_rn(alpha, h[j].z); h[j].w = __fmul_rn(alpha, h[j].w);
      acc.x = fmaf(h[j].x, kk, acc.x); acc.y = fmaf(h[j].y, kk, acc.y);
      acc.z = fmaf(h[j].z, kk, acc.z); acc.w = fmaf(h[j].w, kk, acc.w);
    }
    *reinterpret_cast<float4*>(&red[warp][c0]) = acc;
    __syncthreads();
    if (tid < kF) {
      float read = red[0][tid];
#pragma unroll
      for (int w = 1; w < kThreads / 32; ++w) read += red[w][tid];
      sdv[tid] = __fmul_rn(beta, __fadd_rn(load_as_float(a.v, nh * kF + tid, a.qkv_dtype), -read));
    }
    __syncthreads();
    const float4 dv = *reinterpret_cast<const float4*>(&sdv[c0]);
    acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int row = warp + 8 * j;
      const float kk = sk[row], qq = sq[row];
      h[j].x = __fadd_rn(h[j].x, __fmul_rn(kk, dv.x)); h[j].y = __fadd_rn(h[j].y, __fmul_rn(kk, dv.y));
      h[j].z = __fadd_rn(h[j].z, __fmul_rn(kk, dv.z)); h[j].w = __fadd_rn(h[j].w, __fmul_rn(kk, dv.w));
      acc.x = fmaf(h[j].x, qq, acc.x); acc.y = fmaf(h[j].y, qq, acc.y);
      acc.z = fmaf(h[j].z, qq, acc.z); acc.w = fmaf(h[j].w, qq, acc.w);
      *reinterpret_cast<float4*>(hout + row * kF + c0) = h[j];
    }
    __syncthreads();                                   // every warp has read the first sums
    *reinterpret_cast<float4*>(&red[warp][c0]) = acc;
    __syncthreads();
    if (tid < kF) {
      float o = red[0][tid];
#pragma unroll
      for (int w = 1; w < kThreads / 32; ++w) o += red[w][tid];
      store_from_float(a.o, nh * kF + tid, a.o_dtype, o);
    }
    __syncthreads();                                   // red, sk, sq are rewritten by the next tile
  }
}

constexpr size_t kMaxSmem = 227 * 1024;

}  // namespace

int launch_generic(const KParams& p, cudaStream_t stream) {
  const size_t smem =
      sizeof(float) * (2 * (size_t)p.K * (p.V + 1) + 2 * (size_t)p.K + p.V + 8);
  if (smem > kMaxSmem) return CARRY_GDN_ERR_UNSUPPORTED;
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return CARRY_GDN_ERR_NO_DEVICE;
  if (smem > configured[dev]) {
    if (cudaFuncSetAttribute(gdn_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kMaxSmem) != cudaSuccess) {
      cudaGetLastError();
      return CARRY_GDN_ERR_NO_DEVICE;
    }
    configured[dev] = kMaxSmem;
  }
  const long long tiles = (long long)p.B * p.HV;
  if (tiles == 0) return CARRY_GDN_OK;
  gdn_generic_kernel<<<(unsigned)tiles, kThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
}

int launch_fp32(const CarryGdnFp32Args& a, cudaStream_t stream) {
  const long long all_tiles = (long long)a.B * a.HV;
  if (all_tiles == 0) return CARRY_GDN_OK;
  if (a.K == kF && a.V == kF && ((uintptr_t)a.h_in % 16) == 0 && ((uintptr_t)a.h_out % 16) == 0) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long cap = (long long)sms * 2 * 8;      // 2 CTAs per SM, a few tiles each
    gdn_fp32_tile128_kernel<<<(unsigned)(all_tiles < cap ? all_tiles : cap), kThreads, 0, stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
  }
  const size_t smem = sizeof(float) * ((size_t)a.K * a.V + 2 * (size_t)a.K);
  if (smem > kMaxSmem) return CARRY_GDN_ERR_UNSUPPORTED;
  static thread_local size_t configured[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return CARRY_GDN_ERR_NO_DEVICE;
  if (smem > configured[dev]) {
    if (cudaFuncSetAttribute(gdn_fp32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)kMaxSmem) != cudaSuccess) {
      cudaGetLastError();
      return CARRY_GDN_ERR_NO_DEVICE;
    }
    configured[dev] = kMaxSmem;
  }
  const long long tiles = (long long)a.B * a.HV;
  if (tiles == 0) return CARRY_GDN_OK;
  gdn_fp32_kernel<<<(unsigned)tiles, kThreads, smem, stream>>>(a);
  return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
}

}  // namespace carry
