// The quantized step without error feedback (CARRY_RES_NONE) for K = V = 128 in the
// statequant layout [K][V]: the "uniform grid, no feedback" arm of the reference's
// granularity experiments (statequant/quant.py:23-34 with one scale per head, or one
// per V column).  A streaming kernel in the manner of the fp32 step: the tile lives in
// registers (a lane holds 16 consecutive columns of 4 rows: 64 state values, four
// 16-byte reads of codes in flight), sums and maxima over K cross the CTA through
// shared memory, every code is read once and written once.
#include "carry_gdn_common.cuh"

namespace carry {
namespace {

constexpr int kT = 128;
constexpr int kThreads = 256;
constexpr int kGroups = 32;                       // row groups of a tile: 8 warps x 4 rows per pass
constexpr float kMagic = 12582912.0f;             // 1.5 * 2^23: x + kMagic rounds x to an integer, half to even
constexpr float kTieGuard = 0.4999847412109375f;  // 0.5 - 2^-16

// 1/s to within 2^-24 relative; s is a scale (normal, >= 1e-12 / 127)
__device__ __forceinline__ float rcp_refined(float s) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(s));
  return fmaf(y, fmaf(-s, y, 1.0f), y);
}

__device__ __forceinline__ float s8_of(uint32_t w, int byte) { return (float)(int)(int8_t)(w >> (8 * byte)); }

__device__ __forceinline__ uint32_t pack4(float a, float b, float c, float d) {   // low bytes of code + kMagic
  const uint32_t lo = __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x0040);
  const uint32_t hi = __byte_perm(__float_as_uint(c), __float_as_uint(d), 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

__global__ void __launch_bounds__(kThreads, 2) gdn_noef128_kernel(const __grid_constant__ KParams p) {
  __shared__ __align__(16) float red[kGroups][kT];    // partial sums of a column, one row per row group
  __shared__ __align__(16) float redm[kGroups][kT];   // partial maxima
  __shared__ __align__(16) float sk[kT], sq[kT], sdv[kT], ss[kT], sinv[kT];
  __shared__ float wmax[kThreads / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c0 = 16 * (lane & 7), rsub = 4 * warp + (lane >> 3);      // my columns; my row within a pass
  const bool per_head = p.sscale_mode == CARRY_SCALE_PER_HEAD;
  const long long tiles = (long long)p.B * p.HV;

  for (long long nh = blockIdx.x; nh < tiles; nh += gridDim.x) {
    const int8_t* cin = p.codes_in + nh * kT * kT;
    int8_t* cout = p.codes_out + nh * kT * kT;
    uint4 w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = *reinterpret_cast<const uint4*>(cin + (32 * j + rsub) * kT + c0);
    if (tid < kT) {
      sk[tid] = load_as_float(p.k, nh * kT + tid, p.qkv_dtype);
      sq[tid] = load_as_float(p.q, nh * kT + tid, p.qkv_dtype);
      ss[tid] = per_head ? p.sscale_in[nh] : p.sscale_in[nh * kT + tid];
    }
    const float alpha = p.alpha[nh], beta = p.beta[nh];
    __syncthreads();

    // dequantise, decay, partial <column, k>
    float h[4][16], acc[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[c] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float kk = sk[32 * j + rsub];
      const uint32_t ww[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        h[j][c] = __fmul_rn(__fmul_rn(s8_of(ww[c >> 2], c & 3), ss[c0 + c]), alpha);
        acc[c] = fmaf(h[j][c], kk, acc[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < 16; c += 4)
      *reinterpret_cast<float4*>(&red[rsub][c0 + c]) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
    __syncthreads();
    if (tid < kT) {
      float read = red[0][tid];
#pragma unroll
      for (int g = 1; g < kGroups; ++g) read += red[g][tid];
      sdv[tid] = __fmul_rn(beta, __fadd_rn(load_as_float(p.v, nh * kT + tid, p.qkv_dtype), -read));
    }
    __syncthreads();

    // rank-1 write and partial <column, q>; then partial column maxima (two loops: fewer values live at once)
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[c] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float kk = sk[32 * j + rsub], qq = sq[32 * j + rsub];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        h[j][c] = __fadd_rn(h[j][c], __fmul_rn(kk, sdv[c0 + c]));
        acc[c] = fmaf(h[j][c], qq, acc[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < 16; c += 4)
      *reinterpret_cast<float4*>(&red[rsub][c0 + c]) = make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]);
#pragma unroll
    for (int c = 0; c < 16; c += 4) {
      float m[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        m[i] = fmaxf(fmaxf(fabsf(h[0][c + i]), fabsf(h[1][c + i])), fmaxf(fabsf(h[2][c + i]), fabsf(h[3][c + i])));
      *reinterpret_cast<float4*>(&redm[rsub][c0 + c]) = make_float4(m[0], m[1], m[2], m[3]);
    }
    __syncthreads();
    float colmax = 0.f;
    if (tid < kT) {
      float o = red[0][tid];
      colmax = redm[0][tid];
#pragma unroll
      for (int g = 1; g < kGroups; ++g) { o += red[g][tid]; colmax = fmaxf(colmax, redm[g][tid]); }
      store_from_float(p.out, nh * kT + tid, p.o_dtype, o);
    }
    if (per_head) {                                   // one scale for the whole matrix
      float m = colmax;
      for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
      if (lane == 0) wmax[warp] = m;
      __syncthreads();
      if (tid < kT) {
        float t = wmax[0];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) t = fmaxf(t, wmax[i]);
        const float s = scale_from_amax(t, p.qmax, p.eps_mode);
        ss[tid] = s;
        sinv[tid] = rcp_refined(s);
        if (tid == 0) p.sscale_out[nh] = s;
      }
    } else if (tid < kT) {
      const float s = scale_from_amax(colmax, p.qmax, p.eps_mode);
      ss[tid] = s;
      sinv[tid] = rcp_refined(s);
      p.sscale_out[nh * kT + tid] = s;
    }
    __syncthreads();

    // codes: rint(h / s) as fma(h, 1/s, 1.5 * 2^23), whose low byte is the code.  |h / s| <= qmax, so the
    // candidate can only be wrong within 127 * 2^-24 < 2^-16 of a tie; the exact remainder h - code * s
    // shows those, and a word that has one is redone with the true division.
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t word[4];
#pragma unroll
      for (int m = 0; m < 4; ++m) {                   // four columns = one word of codes at a time
        float y[4], worst = -1.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = 4 * m + i;
          const float s = ss[c0 + c];
          y[i] = fmaf(h[j][c], sinv[c0 + c], kMagic);
          worst = fmaxf(worst, fmaf(-kTieGuard, s, fabsf(fmaf(kMagic - y[i], s, h[j][c]))));
        }
        if (worst > 0.f) {
#pragma unroll
          for (int i = 0; i < 4; ++i) y[i] = quantize_div(h[j][4 * m + i], ss[c0 + 4 * m + i], p.qmax) + kMagic;
        }
        word[m] = pack4(y[0], y[1], y[2], y[3]);
      }
      *reinterpret_cast<uint4*>(cout + (32 * j + rsub) * kT + c0) = make_uint4(word[0], word[1], word[2], word[3]);
    }
    __syncthreads();                                  // the shared arrays are rewritten by the next tile
  }
}

}  // namespace

bool noef128_eligible(const KParams& p) {
  return !p.packed && p.res_fmt == CARRY_RES_NONE && p.K == kT && p.V == kT &&
         ((uintptr_t)p.codes_in % 16) == 0 && ((uintptr_t)p.codes_out % 16) == 0;
}

int launch_noef128(const KParams& p, cudaStream_t stream) {
  const long long tiles = (long long)p.B * p.HV;
  if (tiles == 0) return CARRY_GDN_OK;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long cap = (long long)sms * 2 * 8;       // 2 CTAs per SM, a few tiles each
  gdn_noef128_kernel<<<(unsigned)(tiles < cap ? tiles : cap), kThreads, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
}

}  // namespace carry
