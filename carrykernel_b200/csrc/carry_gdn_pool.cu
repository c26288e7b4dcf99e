// Moving a request's state in and out of the slot pool [slots, HV, V, K]:
// quantise a floating-point state into a slot (prefill hand-off), dequantise a
// slot back, and copy whole slots.  All three are plain streaming kernels: a
// CTA works through (request, head) tiles, a warp on four V-rows at a time, a
// lane on VEC consecutive K elements of each.  Rows of K = 32 * VEC elements
// stay in registers between the row maximum and the encoding; other shapes go
// through predicated loops that look at a row two or three times (once from
// DRAM, then from L1).  The tile after the current one is asked into the L2.
#include "carry_gdn_common.cuh"

namespace carry {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRows = 4;    // rows a warp has in flight

__device__ __forceinline__ float warp_max_nonneg(float x) {
  // non-negative floats order like their bit patterns
  return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(x)));
}

// 1/s to within 2^-24 relative (hardware approximation + one Newton step); s is a scale,
// normal and at least 1e-12 / 127.
__device__ __forceinline__ float rcp_refined(float s) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(s));
  return fmaf(y, fmaf(-s, y, 1.0f), y);
}

// round_half_even(x / s) for the VEC elements of a chunk, without dividing.  Adding
// 1.5 * 2^23 to x * (1/s) inside one fused multiply-add rounds the quotient to an integer
// (half to even) and leaves it, two's complement, in the low byte of the float's bits, so
// the result y = code + kMagic is what gets packed; no clamp is needed because |x / s| is at
// most qmax (1 + 2^-23) when s = amax / qmax.  The reciprocal is good to 2^-24, so the
// candidate can only be wrong when the quotient lies within 127 * 2^-24 < 2^-16 of a tie,
// which the exact remainder x - code * s shows; a chunk with such an element (a few in ten
// thousand) is redone with the true division.
constexpr float kMagic = 12582912.0f;              // 1.5 * 2^23, bits 0x4B400000
constexpr float kTieGuard = 0.4999847412109375f;   // 0.5 - 2^-16
template <int VEC>
__device__ __forceinline__ void quantize_chunk(const float (&x)[VEC], float s, float inv, float qmax,
                                               float (&y)[VEC]) {
  float worst = 0.0f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    y[i] = fmaf(x[i], inv, kMagic);
    worst = fmaxf(worst, fabsf(fmaf(kMagic - y[i], s, x[i])));
  }
  if (worst > kTieGuard * s) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) y[i] = quantize_div(x[i], s, qmax) + kMagic;
  }
}

// VEC consecutive elements of a floating-point row as fp32
template <int VEC>
__device__ __forceinline__ void load_row(const void* base, long long off, int dtype, float (&x)[VEC]) {
  if constexpr (VEC == 4) {
    if (dtype == CARRY_F32) {
      const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
      x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
    } else {
      const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + off);
      if (dtype == CARRY_BF16) {
        x[0] = __uint_as_float(t.x << 16); x[1] = __uint_as_float(t.x & 0xffff0000u);
        x[2] = __uint_as_float(t.y << 16); x[3] = __uint_as_float(t.y & 0xffff0000u);
      } else {
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
        const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
        x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
      }
    }
  } else {
    x[0] = load_as_float(base, off, dtype);
  }
}

template <int VEC>
__device__ __forceinline__ void store_row(void* base, long long off, int dtype, const float (&x)[VEC]) {
  if constexpr (VEC == 4) {
    if (dtype == CARRY_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off) = make_float4(x[0], x[1], x[2], x[3]);
    } else if (dtype == CARRY_BF16) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(x[2], x[3]);
      uint2 t;
      t.x = *reinterpret_cast<const uint32_t*>(&lo);
      t.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + off) = t;
    } else {
      const __half2 lo = __floats2half2_rn(x[0], x[1]);
      const __half2 hi = __floats2half2_rn(x[2], x[3]);
      uint2 t;
      t.x = *reinterpret_cast<const uint32_t*>(&lo);
      t.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + off) = t;
    }
  } else {
    store_from_float(base, off, dtype, x[0]);
  }
}

// VEC int8 codes, given as code + kMagic, to byte offset `off` of a row
template <int VEC>
__device__ __forceinline__ void store_codes(int8_t* row, int off, const float (&y)[VEC]) {
  if constexpr (VEC == 4) {
    const uint32_t lo = __byte_perm(__float_as_uint(y[0]), __float_as_uint(y[1]), 0x0040);
    const uint32_t hi = __byte_perm(__float_as_uint(y[2]), __float_as_uint(y[3]), 0x0040);
    *reinterpret_cast<uint32_t*>(row + off) = __byte_perm(lo, hi, 0x5410);
  } else {
    row[off] = (int8_t)(__float_as_uint(y[0]) & 0xffu);
  }
}

// the stored bits of VEC int8 codes, and their values
template <int VEC>
__device__ __forceinline__ uint32_t raw_codes(const int8_t* row, int off) {
  if constexpr (VEC == 4) return *reinterpret_cast<const uint32_t*>(row + off);
  else return (uint8_t)row[off];
}

template <int VEC>
__device__ __forceinline__ void codes_of(uint32_t w, float (&c)[VEC]) {
#pragma unroll
  for (int i = 0; i < VEC; ++i) c[i] = (float)(int)(int8_t)(w >> (8 * i));
}

// VEC packed int4 codes of elements k .. k+VEC-1 (two per byte, even index in the
// low nibble).  With VEC == 1 the odd lane hands its code to the even lane below
// it, so every lane of the warp has to make the call.
template <int VEC>
__device__ __forceinline__ void store_nibbles(int8_t* row, int k, bool valid, const float (&y)[VEC]) {
  if constexpr (VEC == 4) {
    if (valid) {
      const uint32_t w = (__float_as_uint(y[0]) & 0xfu) | ((__float_as_uint(y[1]) & 0xfu) << 4) |
                         ((__float_as_uint(y[2]) & 0xfu) << 8) | ((__float_as_uint(y[3]) & 0xfu) << 12);
      *reinterpret_cast<uint16_t*>(row + (k >> 1)) = (uint16_t)w;
    }
  } else {
    const uint32_t mine = __float_as_uint(y[0]) & 0xfu;
    const uint32_t next = __shfl_down_sync(0xffffffffu, mine, 1);
    if (valid && !(k & 1)) row[k >> 1] = (int8_t)(mine | (next << 4));
  }
}

template <int VEC>
__device__ __forceinline__ uint32_t raw_nibbles(const int8_t* row, int k) {
  if constexpr (VEC == 4) return *reinterpret_cast<const uint16_t*>(row + (k >> 1));
  else return ((uint32_t)(uint8_t)row[k >> 1] >> ((k & 1) * 4)) & 0xfu;
}

template <int VEC>
__device__ __forceinline__ void nibbles_of(uint32_t w, float (&c)[VEC]) {
#pragma unroll
  for (int i = 0; i < VEC; ++i) c[i] = (float)(((int)(w << (28 - 4 * i))) >> 28);
}

// ask the L2 for `bytes` at p, one request per 128-byte line, spread over the CTA
__device__ __forceinline__ void prefetch_l2(const void* p, long long bytes) {
  const char* c = reinterpret_cast<const char*>(p);
  for (long long off = (long long)threadIdx.x * 128; off < bytes; off += (long long)kThreads * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(c + off));
}

struct PoolView {
  int8_t* codes;      // this (slot, head)'s [V, K]
  float* sscale;      // [V]
  int8_t* resid;      // [V, K] or [V, K/2]
  float* rscale;      // [V] or [1]
};

__device__ __forceinline__ PoolView view_of(const CarryGdnPool& pool, int slot, int hv) {
  const long long VK = (long long)pool.V * pool.K;
  const long long rk = pool.res_fmt == CARRY_RES_INT4 ? VK / 2 : VK;
  PoolView t;
  t.codes = pool.state_codes + (long long)slot * pool.stride_state_slot + hv * VK;
  t.sscale = pool.state_scale + (long long)slot * pool.stride_sscale_slot + (long long)hv * pool.V;
  t.resid = pool.resid_codes + (long long)slot * pool.stride_resid_slot + hv * rk;
  t.rscale = pool.resid_scale + (long long)slot * pool.stride_rscale_slot +
             (pool.resid_scale_mode == CARRY_SCALE_PER_HEAD ? (long long)hv : (long long)hv * pool.V);
  return t;
}

// slot id of request n, or -1 for padding / an id outside the pool (flagged)
__device__ __forceinline__ int slot_of(const int32_t* slots, long long stride, int n, int num_slots,
                                       int32_t* status) {
  const int slot = slots[n * stride];
  if (slot <= 0) return -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && status) atomicOr(status, CARRY_GDN_STATUS_BAD_SLOT);
    return -1;
  }
  return slot;
}

// ---------------------------------------------------------------------------
// floating-point state -> slot
// ---------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(kThreads, 3) pool_store_kernel(CarryGdnPoolStoreArgs a) {
  __shared__ float s_emax[kWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const CarryGdnPool& pool = a.pool;
  const int HV = pool.HV, V = pool.V, K = pool.K;
  const bool int4 = pool.res_fmt == CARRY_RES_INT4;
  const bool per_head = pool.resid_scale_mode == CARRY_SCALE_PER_HEAD;
  const float rq = int4 ? 7.0f : 127.0f;
  const int rrow = int4 ? K / 2 : K;
  const int chunks = (K + 32 * VEC - 1) / (32 * VEC);
  const bool whole_rows = K == 32 * VEC && V % kRows == 0;

  // A warp's row groups run one after the other, so the rows of the tile after
  // this one are asked into the L2 while this one is worked on.
  const int h_es = a.h_dtype == CARRY_F32 ? 4 : 2;
  auto prefetch_tile = [&](long long tile) {
    if (tile >= (long long)a.B * HV) return;
    const long long off = (tile / HV) * a.stride_h_req + (tile % HV) * (long long)V * K;
    prefetch_l2(reinterpret_cast<const char*>(a.h) + off * h_es, (long long)V * K * h_es);
  };
  prefetch_tile(blockIdx.x);

  for (long long tile = blockIdx.x; tile < (long long)a.B * HV; tile += gridDim.x) {
    prefetch_tile(tile + gridDim.x);
    const int n = (int)(tile / HV), hv = (int)(tile % HV);
    const int slot = slot_of(a.slots, a.stride_slots, n, pool.num_slots, a.status);
    if (slot < 0) continue;
    const PoolView t = view_of(pool, slot, hv);
    const long long h_tile = (long long)n * a.stride_h_req + (long long)hv * V * K;

    // codes (as code + kMagic) and error of one chunk, the same arithmetic every time it is asked for
    auto encode = [&](int v, int k, float s, float (&y)[VEC], float (&e)[VEC]) {
      float x[VEC];
      load_row<VEC>(a.h, h_tile + (long long)v * K + k, a.h_dtype, x);
      quantize_chunk<VEC>(x, s, rcp_refined(s), a.qmax, y);
      if (a.keep_error) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) e[i] = __fsub_rn(x[i], __fmul_rn(y[i] - kMagic, s));
      }
    };
    auto put_resid = [&](int v, int k, bool valid, const float (&r)[VEC]) {
      if (int4) store_nibbles<VEC>(t.resid + (long long)v * rrow, k, valid, r);
      else if (valid) store_codes<VEC>(t.resid + (long long)v * rrow, k, r);
    };

    // A warp takes kRows rows at a time: their first reads are independent, so
    // that many row loads are in flight per warp while DRAM answers.
    float tile_emax = 0.0f;
    for (int v0 = warp * kRows; v0 < V; v0 += kWarps * kRows) {
      if constexpr (VEC == 4) {
        if (whole_rows) {
          // A row is exactly one chunk and the group is full: the rows stay in registers
          // between the maximum and the encoding, and nothing is predicated.
          const int k = lane * 4;
          const long long at = h_tile + (long long)v0 * K + k;
          int8_t* crow = t.codes + v0 * K + k;
          int8_t* rrow0 = t.resid + v0 * rrow + (int4 ? k >> 1 : k);
          float x[kRows][4], s[kRows];
#pragma unroll
          for (int r = 0; r < kRows; ++r) load_row<4>(a.h, at + r * K, a.h_dtype, x[r]);
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            const float m = fmaxf(fmaxf(fabsf(x[r][0]), fabsf(x[r][1])), fmaxf(fabsf(x[r][2]), fabsf(x[r][3])));
            s[r] = scale_from_amax(warp_max_nonneg(m), a.qmax, CARRY_EPS_ON_AMAX);
          }
          if (lane < kRows) t.sscale[v0 + lane] = lane == 0 ? s[0] : lane == 1 ? s[1] : lane == 2 ? s[2] : s[3];
          float e[kRows][4], emax[kRows] = {};
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            float y[4];
            quantize_chunk<4>(x[r], s[r], rcp_refined(s[r]), a.qmax, y);
            store_codes<4>(crow, r * K, y);
            if (a.keep_error) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                e[r][i] = __fsub_rn(x[r][i], __fmul_rn(y[i] - kMagic, s[r]));
                emax[r] = fmaxf(emax[r], fabsf(e[r][i]));
              }
            } else if (int4) {
              *reinterpret_cast<uint16_t*>(rrow0 + r * rrow) = 0;
            } else {
              *reinterpret_cast<uint32_t*>(rrow0 + r * rrow) = 0u;
            }
          }
          if (!a.keep_error) {
            if (!per_head && lane < kRows) t.rscale[v0 + lane] = 0.0f;
          } else if (!per_head) {
            float es[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) es[r] = scale_from_amax(warp_max_nonneg(emax[r]), rq, CARRY_EPS_ON_SCALE);
            if (lane < kRows) t.rscale[v0 + lane] = lane == 0 ? es[0] : lane == 1 ? es[1] : lane == 2 ? es[2] : es[3];
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
              float q[4];
              quantize_chunk<4>(e[r], es[r], rcp_refined(es[r]), rq, q);
              if (int4) store_nibbles<4>(rrow0 + r * rrow - (k >> 1), k, true, q);
              else store_codes<4>(rrow0, r * rrow, q);
            }
          } else {
#pragma unroll
            for (int r = 0; r < kRows; ++r) tile_emax = fmaxf(tile_emax, emax[r]);
          }
          continue;
        }
      }
      float amax[kRows] = {};
      for (int c = 0; c < chunks; ++c) {
        const int k = (c * 32 + lane) * VEC;
        if (k < K) {
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            if (v0 + r < V) {
              float x[VEC];
              load_row<VEC>(a.h, h_tile + (long long)(v0 + r) * K + k, a.h_dtype, x);
#pragma unroll
              for (int i = 0; i < VEC; ++i) amax[r] = fmaxf(amax[r], fabsf(x[i]));
            }
          }
        }
      }
      float s[kRows], emax[kRows] = {};
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        s[r] = scale_from_amax(warp_max_nonneg(amax[r]), a.qmax, CARRY_EPS_ON_AMAX);
        if (lane == 0 && v0 + r < V) t.sscale[v0 + r] = s[r];
      }

      for (int c = 0; c < chunks; ++c) {
        const int k = (c * 32 + lane) * VEC;
        const bool valid = k < K;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int v = v0 + r;
          if (v >= V) continue;                  // the whole warp skips together
          float zero[VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i) zero[i] = kMagic;
          if (valid) {
            float cd[VEC], e[VEC] = {};
            encode(v, k, s[r], cd, e);
            store_codes<VEC>(t.codes + (long long)v * K, k, cd);
#pragma unroll
            for (int i = 0; i < VEC; ++i) emax[r] = fmaxf(emax[r], fabsf(e[i]));
          }
          if (!a.keep_error) put_resid(v, k, valid, zero);
        }
      }
      if (!a.keep_error) {
#pragma unroll
        for (int r = 0; r < kRows; ++r)
          if (!per_head && lane == 0 && v0 + r < V) t.rscale[v0 + r] = 0.0f;
      } else if (!per_head) {
        float es[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          es[r] = scale_from_amax(warp_max_nonneg(emax[r]), rq, CARRY_EPS_ON_SCALE);
          if (lane == 0 && v0 + r < V) t.rscale[v0 + r] = es[r];
        }
        for (int c = 0; c < chunks; ++c) {
          const int k = (c * 32 + lane) * VEC;
          const bool valid = k < K;
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            const int v = v0 + r;
            if (v >= V) continue;
            float q[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) q[i] = kMagic;
            if (valid) {
              float cd[VEC], e[VEC];
              encode(v, k, s[r], cd, e);
              quantize_chunk<VEC>(e, es[r], rcp_refined(es[r]), rq, q);
            }
            put_resid(v, k, valid, q);
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < kRows; ++r) tile_emax = fmaxf(tile_emax, emax[r]);
      }
    }

    if (per_head) {
      if (!a.keep_error) {
        if (threadIdx.x == 0) t.rscale[0] = 0.0f;
      } else {
        // one residual scale for the whole [V, K] matrix: every warp's maximum first
        tile_emax = warp_max_nonneg(tile_emax);
        if (lane == 0) s_emax[warp] = tile_emax;
        __syncthreads();                       // also publishes the row scales written above
        float emax = s_emax[lane & (kWarps - 1)];
        emax = warp_max_nonneg(emax);
        const float es = scale_from_amax(emax, rq, CARRY_EPS_ON_SCALE);
        const float ies = rcp_refined(es);
        if (threadIdx.x == 0) t.rscale[0] = es;
        bool done = false;
        if constexpr (VEC == 4) {
          if (whole_rows) {                    // same rows, same warps as above, nothing predicated
            const int k = lane * 4;
            for (int v0 = warp * kRows; v0 < V; v0 += kWarps * kRows) {
              const long long at = h_tile + (long long)v0 * K + k;
              float x[kRows][4];
#pragma unroll
              for (int r = 0; r < kRows; ++r) load_row<4>(a.h, at + r * K, a.h_dtype, x[r]);
              const float4 s4 = *reinterpret_cast<const float4*>(t.sscale + v0);
              const float s[kRows] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int r = 0; r < kRows; ++r) {
                float y[4], e[4], q[4];
                quantize_chunk<4>(x[r], s[r], rcp_refined(s[r]), a.qmax, y);
#pragma unroll
                for (int i = 0; i < 4; ++i) e[i] = __fsub_rn(x[r][i], __fmul_rn(y[i] - kMagic, s[r]));
                quantize_chunk<4>(e, es, ies, rq, q);
                int8_t* row = t.resid + (v0 + r) * rrow;
                if (int4) store_nibbles<4>(row, k, true, q);
                else store_codes<4>(row, k, q);
              }
            }
            done = true;
          }
        }
        for (int v = warp; v < V && !done; v += kWarps) {
          const float s = t.sscale[v];
          for (int c = 0; c < chunks; ++c) {
            const int k = (c * 32 + lane) * VEC;
            const bool valid = k < K;
            float r[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) r[i] = kMagic;
            if (valid) {
              float cd[VEC], e[VEC];
              encode(v, k, s, cd, e);
              quantize_chunk<VEC>(e, es, ies, rq, r);
            }
            put_resid(v, k, valid, r);
          }
        }
        __syncthreads();                       // s_emax is reused by the next tile
      }
    }
  }
}

// ---------------------------------------------------------------------------
// slot -> floating-point state
// ---------------------------------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(kThreads, 4) pool_load_kernel(CarryGdnPoolLoadArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const CarryGdnPool& pool = a.pool;
  const int HV = pool.HV, V = pool.V, K = pool.K;
  const bool int4 = pool.res_fmt == CARRY_RES_INT4;
  const bool per_head = pool.resid_scale_mode == CARRY_SCALE_PER_HEAD;
  const int rrow = int4 ? K / 2 : K;
  const int chunks = (K + 32 * VEC - 1) / (32 * VEC);
  // (the host picks VEC == 4 only when four scales of such a group can be read as one float4)
  const bool whole_rows = K == 32 * VEC && V % kRows == 0;

  auto prefetch_tile = [&](long long tile) {
    if (tile >= (long long)a.B * HV) return;
    const int slot = a.slots[(tile / HV) * a.stride_slots];
    if (slot <= 0 || slot >= pool.num_slots) return;
    const PoolView t = view_of(pool, slot, (int)(tile % HV));
    prefetch_l2(t.codes, (long long)V * K);
    if (a.with_residual) prefetch_l2(t.resid, (long long)V * rrow);
  };
  prefetch_tile(blockIdx.x);

  for (long long tile = blockIdx.x; tile < (long long)a.B * HV; tile += gridDim.x) {
    prefetch_tile(tile + gridDim.x);
    const int n = (int)(tile / HV), hv = (int)(tile % HV);
    const int slot = slot_of(a.slots, a.stride_slots, n, pool.num_slots, a.status);
    const long long h_tile = (long long)n * a.stride_h_req + (long long)hv * V * K;
    const PoolView t = view_of(pool, slot >= 0 ? slot : 0, hv);   // slot 0 is never read below
    for (int v0 = warp * kRows; v0 < V; v0 += kWarps * kRows) {
      if constexpr (VEC == 4) {
        if (whole_rows && slot >= 0) {         // a row is one chunk, the group is full: nothing predicated
          const int k = lane * 4;
          const int8_t* crow = t.codes + v0 * K + k;
          const int8_t* rrow0 = t.resid + v0 * rrow + (int4 ? k >> 1 : k);
          uint32_t cw[kRows], rw[kRows] = {};
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            cw[r] = *reinterpret_cast<const uint32_t*>(crow + r * K);
            if (a.with_residual)
              rw[r] = int4 ? (uint32_t)*reinterpret_cast<const uint16_t*>(rrow0 + r * rrow)
                           : *reinterpret_cast<const uint32_t*>(rrow0 + r * rrow);
          }
          const float4 s4 = *reinterpret_cast<const float4*>(t.sscale + v0);
          const float s[kRows] = {s4.x, s4.y, s4.z, s4.w};
          float es[kRows] = {};
          if (a.with_residual) {
            if (per_head) {
              es[0] = es[1] = es[2] = es[3] = t.rscale[0];
            } else {
              const float4 e4 = *reinterpret_cast<const float4*>(t.rscale + v0);
              es[0] = e4.x; es[1] = e4.y; es[2] = e4.z; es[3] = e4.w;
            }
          }
          const long long at = h_tile + (long long)v0 * K + k;
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            float x[4], cd[4], rd[4];
            codes_of<4>(cw[r], cd);
            if (int4) nibbles_of<4>(rw[r], rd);
            else codes_of<4>(rw[r], rd);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              x[i] = __fmul_rn(cd[i], s[r]);
              if (a.with_residual) x[i] = __fadd_rn(x[i], __fmul_rn(rd[i], es[r]));
            }
            store_row<4>(a.h, at + r * K, a.h_dtype, x);
          }
          continue;
        }
      }
      float s[kRows], es[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const bool row = slot >= 0 && v0 + r < V;
        s[r] = row ? t.sscale[v0 + r] : 0.0f;
        es[r] = (row && a.with_residual) ? t.rscale[per_head ? 0 : v0 + r] : 0.0f;
      }
      for (int c = 0; c < chunks; ++c) {
        const int k = (c * 32 + lane) * VEC;
        if (k >= K) continue;
        // all reads of the row group first, then arithmetic and writes
        uint32_t cw[kRows] = {}, rw[kRows] = {};
        if (slot >= 0) {
#pragma unroll
          for (int r = 0; r < kRows; ++r) {
            const int v = v0 + r;
            if (v >= V) continue;
            cw[r] = raw_codes<VEC>(t.codes + (long long)v * K, k);
            if (a.with_residual)
              rw[r] = int4 ? raw_nibbles<VEC>(t.resid + (long long)v * rrow, k)
                           : raw_codes<VEC>(t.resid + (long long)v * rrow, k);
          }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const int v = v0 + r;
          if (v >= V) continue;
          float x[VEC], cd[VEC], rd[VEC];
          codes_of<VEC>(cw[r], cd);
          if (int4) nibbles_of<VEC>(rw[r], rd);
          else codes_of<VEC>(rw[r], rd);
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            x[i] = __fmul_rn(cd[i], s[r]);
            if (a.with_residual) x[i] = __fadd_rn(x[i], __fmul_rn(rd[i], es[r]));
          }
          store_row<VEC>(a.h, h_tile + (long long)v * K + k, a.h_dtype, x);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// slot -> slot
// ---------------------------------------------------------------------------
__device__ __forceinline__ void copy_bytes(void* dst, const void* src, long long bytes) {
  const bool wide = (((uintptr_t)dst | (uintptr_t)src | (uintptr_t)bytes) & 15) == 0;
  if (wide) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    const long long n = bytes / 16;
    long long i = threadIdx.x;
    for (; i + 3 * kThreads < n; i += 4 * kThreads) {      // four reads in flight per thread
      const uint4 x0 = s[i], x1 = s[i + kThreads], x2 = s[i + 2 * kThreads], x3 = s[i + 3 * kThreads];
      d[i] = x0; d[i + kThreads] = x1; d[i + 2 * kThreads] = x2; d[i + 3 * kThreads] = x3;
    }
    for (; i < n; i += kThreads) d[i] = s[i];
  } else {
    const uint8_t* s = reinterpret_cast<const uint8_t*>(src);
    uint8_t* d = reinterpret_cast<uint8_t*>(dst);
    for (long long i = threadIdx.x; i < bytes; i += kThreads) d[i] = s[i];
  }
}

__global__ void __launch_bounds__(kThreads) pool_copy_kernel(CarryGdnPoolCopyArgs a) {
  const int HV = a.src.HV, V = a.src.V, K = a.src.K;
  const long long rbytes = a.src.res_fmt == CARRY_RES_INT4 ? (long long)V * K / 2 : (long long)V * K;
  const bool per_head = a.src.resid_scale_mode == CARRY_SCALE_PER_HEAD;
  for (long long tile = blockIdx.x; tile < (long long)a.B * HV; tile += gridDim.x) {
    const int n = (int)(tile / HV), hv = (int)(tile % HV);
    const int from = slot_of(a.src_slots, a.stride_src_slots, n, a.src.num_slots, a.status);
    const int to = slot_of(a.dst_slots, a.stride_dst_slots, n, a.dst.num_slots, a.status);
    if (from < 0 || to < 0) continue;
    const PoolView s = view_of(a.src, from, hv);
    const PoolView d = view_of(a.dst, to, hv);
    if (s.codes == d.codes) continue;          // a slot onto itself
    copy_bytes(d.codes, s.codes, (long long)V * K);
    copy_bytes(d.resid, s.resid, rbytes);
    copy_bytes(d.sscale, s.sscale, (long long)V * 4);
    copy_bytes(d.rscale, s.rscale, per_head ? 4 : (long long)V * 4);
  }
}

int grid_for(long long tiles) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long cap = (long long)sms * 8;    // 8 CTAs of 256 threads fill an SM
  return (int)(tiles < cap ? tiles : cap);
}

bool aligned(const void* p, int bytes) { return ((uintptr_t)p % bytes) == 0; }

// four elements per lane need rows that start on the vector boundaries
bool vector_ok(const CarryGdnPool& pool, const void* h, long long stride_h_req, int h_dtype) {
  const int es = h_dtype == CARRY_F32 ? 4 : 2;
  if (pool.K % 4) return false;
  if (h && (!aligned(h, 4 * es) || (stride_h_req * es) % (4 * es))) return false;
  if (!aligned(pool.state_codes, 4) || pool.stride_state_slot % 4) return false;
  if (pool.V % 4 == 0) {   // groups of four rows read their scales as one float4
    if (!aligned(pool.state_scale, 16) || pool.stride_sscale_slot % 4) return false;
    if (pool.resid_scale_mode == CARRY_SCALE_PER_V && (!aligned(pool.resid_scale, 16) || pool.stride_rscale_slot % 4))
      return false;
  }
  if (pool.res_fmt == CARRY_RES_INT4) {
    if (!aligned(pool.resid_codes, 2) || pool.stride_resid_slot % 2) return false;
  } else {
    if (!aligned(pool.resid_codes, 4) || pool.stride_resid_slot % 4) return false;
  }
  return true;
}

int finish_launch() { return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH; }

}  // namespace

int launch_pool_store(const CarryGdnPoolStoreArgs& a, cudaStream_t stream) {
  const int grid = grid_for((long long)a.B * a.pool.HV);
  if (vector_ok(a.pool, a.h, a.stride_h_req, a.h_dtype))
    pool_store_kernel<4><<<grid, kThreads, 0, stream>>>(a);
  else
    pool_store_kernel<1><<<grid, kThreads, 0, stream>>>(a);
  return finish_launch();
}

int launch_pool_load(const CarryGdnPoolLoadArgs& a, cudaStream_t stream) {
  const int grid = grid_for((long long)a.B * a.pool.HV);
  if (vector_ok(a.pool, a.h, a.stride_h_req, a.h_dtype))
    pool_load_kernel<4><<<grid, kThreads, 0, stream>>>(a);
  else
    pool_load_kernel<1><<<grid, kThreads, 0, stream>>>(a);
  return finish_launch();
}

int launch_pool_copy(const CarryGdnPoolCopyArgs& a, cudaStream_t stream) {
  const int grid = grid_for((long long)a.B * a.src.HV);
  pool_copy_kernel<<<grid, kThreads, 0, stream>>>(a);
  return finish_launch();
}

}  // namespace carry
