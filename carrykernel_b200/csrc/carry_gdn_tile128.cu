// Streaming kernel for the serving shape: K = V = 128, int8 state, int8 or packed
// int4 residual.  One (request, head) tile is 16 KB of codes + 8/16 KB of
// residual; all of it is contiguous in memory in both layouts, so every tile
// moves with a handful of 1-D bulk async copies (TMA, no tensor map):
//
//   global --cp.async.bulk--> shared stage --(registers)--> same shared stage
//          --cp.async.bulk--> global
//
// Persistent CTAs (two per SM) walk the tile list with a ring of stages: while
// one tile is computed, the loads of the next ones are in flight and the stores
// of the previous one drain.  The state is read from HBM once and written once.
//
// Work split inside a CTA (256 threads = 8 warps): warp w owns memory rows
// 16w..16w+15 of the tile.
//   * slot layout [V][K] (scale per row): lane = (row group rg, column group
//     cg): 4 rows x 16 contiguous columns.  Everything the math reduces over
//     (K) lies along the row, so reductions are 3 shuffle steps inside 8 lanes
//     and warps never wait for each other, except once per tile when the
//     residual scale is per head.
//   * statequant layout [K][V] (scale per column): lane = 4 contiguous columns
//     x the warp's 16 rows; column sums are finished across the 8 warps through
//     shared memory.
// Each warp stores its own 16 rows back, so no CTA-wide barrier guards stores.
//
// Arithmetic keeps the reference's operation order for everything that feeds a
// rounding decision: (code*scale)*alpha, h + (k*dv) with the product rounded
// first, target - (code*scale) with the product rounded first.  round(x / s) is
// evaluated as rint(x * (1/s)) and falls back to the true division only when
// the product lands within 2^-12 of a tie, which is the only place the two can
// differ.
#include "carry_gdn_common.cuh"

namespace carry {
namespace {

constexpr int kT = 128;                 // tile edge
constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr int kSlotCache = 256;

enum { LAYOUT_VK = 0, LAYOUT_KV = 1 };  // slot layout [V][K]; statequant layout [K][V]

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst_gmem, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Bounded wait: after kSpinLimit failed polls the CTA is marked poisoned, the
// status word gets the timeout bit and every later wait returns at once; a
// poisoned CTA stops storing.
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, volatile int* poison, int* status) {
  if (*poison) return;
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return;
    if (spin > 64) __nanosleep(64);
    if ((spin & 1023) == 1023 && *poison) return;
  }
  *poison = 1;
  if (status) atomicOr(status, CARRY_GDN_STATUS_TIMEOUT);
}

// All 8 warps meet here: one arrival per warp, then a bounded wait (never a
// bar.sync inside the tile loop, so nothing in it can wait without a limit).
__device__ __forceinline__ void warps_meet(uint64_t* bar, uint32_t parity, int lane, volatile int* poison,
                                           int* status) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  mbar_wait(bar, parity, poison, status);
}

// ---------------------------------------------------------------------------
// number helpers
// ---------------------------------------------------------------------------
constexpr float kMagicRound = 12582912.0f;      // 1.5 * 2^23: x + M rounds x to an integer (RNE)
constexpr float kMagicByte = 8388736.0f;        // 2^23 + 128

// byte b of w (already XOR-ed with 0x80 per byte) -> float(code)
template <int B>
__device__ __forceinline__ float s8_to_float(uint32_t w_biased) {
  const uint32_t bits = __byte_perm(w_biased, 0x4B000000u, 0x7440 | B);
  return __uint_as_float(bits) - kMagicByte;
}

// rint(x / s) with the reference's semantics.  `inv` is 1/s rounded.
template <bool EXACT>
__device__ __forceinline__ float quant_code(float x, float s, float inv, float& magic_sum) {
  const float qp = __fmul_rn(x, inv);
  magic_sum = __fadd_rn(qp, kMagicRound);
  float code = __fadd_rn(magic_sum, -kMagicRound);
  if (EXACT) {
    const float d = __fadd_rn(qp, -code);
    if (fabsf(d) > 0.5f - 0.000244140625f) {     // within 2^-12 of a tie: decide by the true quotient
      code = rintf(__fdiv_rn(x, s));
      magic_sum = __fadd_rn(code, kMagicRound);
    }
  }
  return code;
}

__device__ __forceinline__ float warp_sum8(float x) {   // over the 8 lanes sharing a row group
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}
__device__ __forceinline__ float warp_max8(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 4));
  return x;
}
__device__ __forceinline__ float warp_sum32(float x) {
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max32(float x) {
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// ---------------------------------------------------------------------------
// shared-memory stage layout (bytes)
// ---------------------------------------------------------------------------
template <int RES, int LAYOUT = 0>
struct StageLayout {
  static constexpr int kResidBytes = (RES == CARRY_RES_INT4) ? kT * kT / 2 : kT * kT;
  static constexpr int kCodes = 0;
  static constexpr int kResid = kT * kT;
  static constexpr int kSScale = kResid + kResidBytes;       // 128 floats
  static constexpr int kRScale = kSScale + 512;              // 128 floats (per V) or a row of per-head scales
  static constexpr int kQ = kRScale + 512;                   // raw q, up to 128 x 4 B
  static constexpr int kK = kQ + 512;
  static constexpr int kV = kK + 512;
  static constexpr int kGateA = kV + 512;                    // row of a (or alpha), up to 128 x 4 B
  static constexpr int kGateB = kGateA + 512;                // row of b (or beta)
  static constexpr int kHeader = kGateB + 512;               // int slot
  static constexpr int kBytes = kHeader + 16;
  // slot layout: two CTAs per SM; the statequant layout also needs 16 KB of
  // cross-warp reduction space, so its int8-residual variant runs one CTA per SM
  static constexpr int kCtasPerSm = (LAYOUT == 1 && RES != CARRY_RES_INT4) ? 1 : 2;
  static constexpr int kStages = (LAYOUT == 0) ? ((RES == CARRY_RES_INT4) ? 4 : 3)
                                               : ((RES == CARRY_RES_INT4) ? 3 : 5);
};

struct TileAddr {
  long long slot;       // <= 0: padding (slot path only)
  const int8_t* codes;
  const uint8_t* resid;
  const float* sscale;
  const float* rscale;  // per V: this tile's 128 floats; per head: start of the row of HV scales
  const uint8_t* q;
  const uint8_t* k;
  const uint8_t* v;
  const uint8_t* ga;    // row of a / alpha
  const uint8_t* gb;
};

__device__ __forceinline__ int esize(int dtype) { return dtype == CARRY_F32 ? 4 : 2; }

template <int RES, int RSCALE>
__device__ __forceinline__ TileAddr tile_addr(const KParams& p, int n, int hv, long long slot) {
  TileAddr t;
  t.slot = slot;
  constexpr long long KV = kT * kT;
  constexpr long long RB = StageLayout<RES>::kResidBytes;
  const int es = esize(p.qkv_dtype);
  if (p.packed) {
    t.codes = p.codes_in + slot * p.stride_state_slot + hv * KV;
    t.resid = reinterpret_cast<const uint8_t*>(p.resid_in) + slot * p.stride_resid_slot + hv * RB;
    t.sscale = p.sscale_in + slot * p.stride_sscale_slot + (long long)hv * kT;
    t.rscale = p.rscale_in + slot * p.stride_rscale_slot + (RSCALE == CARRY_SCALE_PER_V ? (long long)hv * kT : 0);
    const int h = hv / (p.HV / p.H);
    const uint8_t* row = reinterpret_cast<const uint8_t*>(p.q) + (long long)n * p.stride_mixed_tok * es;
    t.q = row + (long long)h * kT * es;
    t.k = row + ((long long)p.H * kT + (long long)h * kT) * es;
    t.v = row + (2LL * p.H * kT + (long long)hv * kT) * es;
    const int ges = esize(p.ab_dtype);
    t.ga = reinterpret_cast<const uint8_t*>(p.a) + (long long)n * p.stride_a_tok * ges;
    t.gb = reinterpret_cast<const uint8_t*>(p.b) + (long long)n * p.stride_b_tok * ges;
  } else {
    const long long nh = (long long)n * p.HV + hv;
    t.codes = p.codes_in + nh * KV;
    t.resid = reinterpret_cast<const uint8_t*>(p.resid_in) + nh * RB;
    t.sscale = p.sscale_in + nh * kT;
    t.rscale = p.rscale_in + (RSCALE == CARRY_SCALE_PER_V ? nh * kT : (long long)n * p.HV);
    t.q = reinterpret_cast<const uint8_t*>(p.q) + nh * kT * es;
    t.k = reinterpret_cast<const uint8_t*>(p.k) + nh * kT * es;
    t.v = reinterpret_cast<const uint8_t*>(p.v) + nh * kT * es;
    t.ga = reinterpret_cast<const uint8_t*>(p.alpha) + (long long)n * p.HV * 4;
    t.gb = reinterpret_cast<const uint8_t*>(p.beta) + (long long)n * p.HV * 4;
  }
  return t;
}

__device__ __forceinline__ float raw_to_float(const uint8_t* base, int i, int dtype) {
  if (dtype == CARRY_F32) return reinterpret_cast<const float*>(base)[i];
  if (dtype == CARRY_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  return __half2float(reinterpret_cast<const __half*>(base)[i]);
}

// 16 consecutive activations starting at element `first` -> fp32
__device__ __forceinline__ void load16(const uint8_t* base, int first, int dtype, float (&out)[16]) {
  if (dtype == CARRY_F32) {
    const float4* p4 = reinterpret_cast<const float4*>(base) + first / 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 x = p4[i];
      out[4 * i] = x.x; out[4 * i + 1] = x.y; out[4 * i + 2] = x.z; out[4 * i + 3] = x.w;
    }
  } else {
    const uint4* p4 = reinterpret_cast<const uint4*>(base) + first / 8;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 x = p4[i];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (dtype == CARRY_BF16) {
          out[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
          out[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        } else {
          const __half2 h2 = *reinterpret_cast<const __half2*>(&w[j]);
          out[8 * i + 2 * j] = __low2float(h2);
          out[8 * i + 2 * j + 1] = __high2float(h2);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int LAYOUT, int RES, int RSCALE, bool EXACT>
__global__ void __launch_bounds__(kThreads, (StageLayout<RES, LAYOUT>::kCtasPerSm))
gdn_tile128_kernel(const __grid_constant__ KParams p) {
  using L = StageLayout<RES, LAYOUT>;
  constexpr int S = L::kStages;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar[S];
  __shared__ __align__(8) uint64_t meet_bar[3];
  __shared__ int done_cnt[S];                        // warps whose stores of a stage have left shared memory
  __shared__ int slot_cache[kSlotCache];             // slot ids of this CTA's first tiles
  __shared__ int poison_flag;
  __shared__ float head_red[2][kWarps];
  __shared__ float gate_A[kT], gate_dt[kT];          // exp(A_log), dt_bias per value head (slot path)
  __shared__ __align__(16) float col_red[(LAYOUT == LAYOUT_KV) ? kWarps * kT * 4 : 4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = p.B * p.HV;
  const int my_tiles = (total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  volatile int* poison = &poison_flag;

  if (tid == 0) {
    poison_flag = 0;
    for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); done_cnt[s] = 0; }
    for (int s = 0; s < 3; ++s) mbar_init(&meet_bar[s], kWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (p.packed) {
    for (int i = tid; i < p.HV; i += kThreads) {
      gate_A[i] = expf(load_as_float(p.A_log, i, p.A_log_dtype));
      gate_dt[i] = load_as_float(p.dt_bias, i, p.dt_bias_dtype);
    }
    for (int i = tid; i < my_tiles && i < kSlotCache; i += kThreads) {
      const int tile = (int)blockIdx.x + i * (int)gridDim.x;
      slot_cache[i] = p.slot_idx[(long long)(tile / p.HV) * p.stride_idx];
    }
  }
  __syncthreads();

  const int qes = esize(p.qkv_dtype);
  const int ges = p.packed ? esize(p.ab_dtype) : 4;
  const uint32_t gate_row_bytes = (uint32_t)p.HV * ges;
  const uint32_t rscale_bytes = (RSCALE == CARRY_SCALE_PER_V) ? 512u : (uint32_t)p.HV * 4u;

  // ---- load tile `it` of this CTA into stage it % S (one thread) ---------------
  auto issue = [&](int it) {
    const int tile = (int)blockIdx.x + it * (int)gridDim.x;
    const int n = tile / p.HV, hv = tile - n * p.HV;
    uint8_t* sb = smem + (size_t)(it % S) * L::kBytes;
    long long slot = 1;
    if (p.packed) {
      slot = (it < kSlotCache) ? slot_cache[it] : p.slot_idx[(long long)n * p.stride_idx];
      if (slot >= p.num_slots) {
        if (p.status) atomicOr(p.status, CARRY_GDN_STATUS_BAD_SLOT);
        slot = 0;
      }
    }
    *reinterpret_cast<volatile int*>(sb + L::kHeader) = (int)slot;
    uint64_t* bar = &full_bar[it % S];
    if (slot <= 0) { mbar_arrive(bar); return; }
    const TileAddr t = tile_addr<RES, RSCALE>(p, n, hv, slot);
    const uint32_t vec = (uint32_t)kT * qes;
    mbar_arrive_expect_tx(bar, kT * kT + L::kResidBytes + 512 + rscale_bytes + 3 * vec + 2 * gate_row_bytes);
    bulk_load(sb + L::kCodes, t.codes, kT * kT, bar);
    bulk_load(sb + L::kResid, t.resid, L::kResidBytes, bar);
    bulk_load(sb + L::kSScale, t.sscale, 512, bar);
    bulk_load(sb + L::kRScale, t.rscale, rscale_bytes, bar);
    bulk_load(sb + L::kQ, t.q, vec, bar);
    bulk_load(sb + L::kK, t.k, vec, bar);
    bulk_load(sb + L::kV, t.v, vec, bar);
    bulk_load(sb + L::kGateA, t.ga, gate_row_bytes, bar);
    bulk_load(sb + L::kGateB, t.gb, gate_row_bytes, bar);
  };

  if (tid == 0) {
    const int pre = my_tiles < S ? my_tiles : S;
    for (int it = 0; it < pre; ++it) issue(it);
  }

  const float rqmax = (RES == CARRY_RES_INT4) ? 7.0f : 127.0f;
  uint32_t meet_parity = 0;            // flips once per computed tile

  for (int it = 0; it < my_tiles; ++it) {
    const int s = it % S;
    const uint32_t parity = (uint32_t)(it / S) & 1u;
    uint8_t* sb = smem + (size_t)s * L::kBytes;
    const int tile = (int)blockIdx.x + it * (int)gridDim.x;
    const int n = tile / p.HV, hv = tile - n * p.HV;

    mbar_wait(&full_bar[s], parity, poison, p.status);
    const int slot = *reinterpret_cast<volatile int*>(sb + L::kHeader);
    const long long out_off = ((long long)n * p.HV + hv) * kT;
    const bool live = slot > 0 && !*poison;

    if (!live) {
      if (slot <= 0 && tid < kT) store_from_float(p.out, out_off + tid, p.o_dtype, 0.f);
    } else {
      // ---- gates ---------------------------------------------------------------
      float alpha, beta;
      if (p.packed) {
        const float a = raw_to_float(sb + L::kGateA, hv, p.ab_dtype);
        const float b = raw_to_float(sb + L::kGateB, hv, p.ab_dtype);
        const float x = a + gate_dt[hv];
        const float sp = (x <= kSoftplusThreshold) ? logf(1.0f + expf(x)) : x;
        alpha = expf(-gate_A[hv] * sp);
        beta = __fdiv_rn(1.0f, 1.0f + expf(-b));
      } else {
        alpha = reinterpret_cast<const float*>(sb + L::kGateA)[hv];
        beta = reinterpret_cast<const float*>(sb + L::kGateB)[hv];
      }
      // ---- L2 norms of q and k (slot path option): every warp on its own --------
      float q_mul = 1.0f, k_mul = 1.0f;
      if (p.packed) {
        if (p.l2norm) {
          float qs = 0.f, ks = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float qv = raw_to_float(sb + L::kQ, 4 * lane + i, p.qkv_dtype);
            const float kv = raw_to_float(sb + L::kK, 4 * lane + i, p.qkv_dtype);
            qs = fmaf(qv, qv, qs);
            ks = fmaf(kv, kv, ks);
          }
          q_mul = __fdiv_rn(1.0f, sqrtf(warp_sum32(qs) + 1e-6f));
          k_mul = __fdiv_rn(1.0f, sqrtf(warp_sum32(ks) + 1e-6f));
        }
      }
      const float* sscale = reinterpret_cast<const float*>(sb + L::kSScale);
      const float* rscale = reinterpret_cast<const float*>(sb + L::kRScale);
      const float es_head = (RSCALE == CARRY_SCALE_PER_HEAD) ? rscale[hv] : 0.f;

      if constexpr (LAYOUT == LAYOUT_VK) {
        // lane: rows r0..r0+3, columns c0..c0+15
        const int cg = lane & 7, rg = lane >> 3;
        const int r0 = 16 * warp + 4 * rg, c0 = 16 * cg;
        float kf[16], qf[16];
        load16(sb + L::kK, c0, p.qkv_dtype, kf);
        load16(sb + L::kQ, c0, p.qkv_dtype, qf);
        if (p.packed) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            kf[j] = __fmul_rn(kf[j], k_mul);
            qf[j] = __fmul_rn(__fmul_rn(qf[j], q_mul), p.qscale);
          }
        }
        float kq = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) kq = fmaf(kf[j], qf[j], kq);
        kq = warp_sum8(kq);

        float h[4][16];
        float dk[4], dq[4], srow[4];
        {
          const float4 s4 = *reinterpret_cast<const float4*>(sscale + r0);
          srow[0] = s4.x; srow[1] = s4.y; srow[2] = s4.z; srow[3] = s4.w;
        }
        // phase 1: dequantise, decay, partial dot products along the row
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 cw = *reinterpret_cast<const uint4*>(sb + L::kCodes + (r0 + i) * kT + c0);
          const uint32_t w[4] = {cw.x ^ 0x80808080u, cw.y ^ 0x80808080u, cw.z ^ 0x80808080u, cw.w ^ 0x80808080u};
          float ak = 0.f, aq = 0.f;
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            float c[4];
            c[0] = s8_to_float<0>(w[m]); c[1] = s8_to_float<1>(w[m]);
            c[2] = s8_to_float<2>(w[m]); c[3] = s8_to_float<3>(w[m]);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const int j = 4 * m + b;
              const float hv_ = __fmul_rn(__fmul_rn(c[b], srow[i]), alpha);
              h[i][j] = hv_;
              ak = fmaf(hv_, kf[j], ak);
              aq = fmaf(hv_, qf[j], aq);
            }
          }
          dk[i] = ak; dq[i] = aq;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) { dk[i] = warp_sum8(dk[i]); dq[i] = warp_sum8(dq[i]); }

        // phase 2: rank-1 write, add the residual, row maxima
        float vrow[4], dv[4], oval[4], amax[4];
        if (p.qkv_dtype == CARRY_F32) {
          const float4 v4 = *reinterpret_cast<const float4*>(sb + L::kV + r0 * 4);
          vrow[0] = v4.x; vrow[1] = v4.y; vrow[2] = v4.z; vrow[3] = v4.w;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) vrow[i] = raw_to_float(sb + L::kV, r0 + i, p.qkv_dtype);
        }
        float es_row[4];
        if (RSCALE == CARRY_SCALE_PER_V) {
          const float4 e4 = *reinterpret_cast<const float4*>(rscale + r0);
          es_row[0] = e4.x; es_row[1] = e4.y; es_row[2] = e4.z; es_row[3] = e4.w;
        } else {
          es_row[0] = es_row[1] = es_row[2] = es_row[3] = es_head;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dv[i] = __fmul_rn(beta, __fadd_rn(vrow[i], -dk[i]));
          oval[i] = fmaf(dv[i], kq, dq[i]);
          float am = 0.f;
          if (RES == CARRY_RES_INT4) {
            const uint2 rw = *reinterpret_cast<const uint2*>(sb + L::kResid + (r0 + i) * (kT / 2) + c0 / 2);
            const uint32_t w[2] = {rw.x ^ 0x88888888u, rw.y ^ 0x88888888u};
            const float es16 = es_row[i] * 0.0625f;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const uint32_t bits = __byte_perm(w[m], 0x4B000000u, 0x7440 | b);
                const float lo = __fmul_rn(__uint_as_float(bits & 0xFFFFFF0Fu) - 8388616.0f, es_row[i]);
                const float hi = __fmul_rn(__uint_as_float(bits & 0xFFFFFFF0u) - kMagicByte, es16);
                const int j = 8 * m + 2 * b;
                const float t0 = __fadd_rn(__fadd_rn(h[i][j], __fmul_rn(kf[j], dv[i])), lo);
                const float t1 = __fadd_rn(__fadd_rn(h[i][j + 1], __fmul_rn(kf[j + 1], dv[i])), hi);
                h[i][j] = t0; h[i][j + 1] = t1;
                am = fmaxf(am, fmaxf(fabsf(t0), fabsf(t1)));
              }
            }
          } else {
            const uint4 rw = *reinterpret_cast<const uint4*>(sb + L::kResid + (r0 + i) * kT + c0);
            const uint32_t w[4] = {rw.x ^ 0x80808080u, rw.y ^ 0x80808080u, rw.z ^ 0x80808080u, rw.w ^ 0x80808080u};
#pragma unroll
            for (int m = 0; m < 4; ++m) {
              float c[4];
              c[0] = s8_to_float<0>(w[m]); c[1] = s8_to_float<1>(w[m]);
              c[2] = s8_to_float<2>(w[m]); c[3] = s8_to_float<3>(w[m]);
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const int j = 4 * m + b;
                const float e = __fmul_rn(c[b], es_row[i]);
                const float t0 = __fadd_rn(__fadd_rn(h[i][j], __fmul_rn(kf[j], dv[i])), e);
                h[i][j] = t0;
                am = fmaxf(am, fabsf(t0));
              }
            }
          }
          amax[i] = am;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) amax[i] = warp_max8(amax[i]);

        // the output row goes straight to global memory
        if (cg == 0) {
          if (p.o_dtype == CARRY_F32) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + out_off + r0) =
                make_float4(oval[0], oval[1], oval[2], oval[3]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) store_from_float(p.out, out_off + r0 + i, p.o_dtype, oval[i]);
          }
        }

        // phase 3: state codes, new residual
        float snew[4], eamax[4];
        float eamax_all = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          snew[i] = scale_from_amax(amax[i], p.qmax, p.eps_mode);
          const float inv = __fdiv_rn(1.0f, snew[i]);
          uint32_t packed[4];
          float em = 0.f;
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            uint32_t y[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const int j = 4 * m + b;
              float ms;
              const float code = quant_code<EXACT>(h[i][j], snew[i], inv, ms);
              y[b] = __float_as_uint(ms);
              const float en = __fadd_rn(h[i][j], -__fmul_rn(code, snew[i]));
              h[i][j] = en;
              em = fmaxf(em, fabsf(en));
            }
            packed[m] = __byte_perm(__byte_perm(y[0], y[1], 0x0040), __byte_perm(y[2], y[3], 0x0040), 0x5410);
          }
          *reinterpret_cast<uint4*>(sb + L::kCodes + (r0 + i) * kT + c0) =
              make_uint4(packed[0], packed[1], packed[2], packed[3]);
          eamax[i] = em;
          eamax_all = fmaxf(eamax_all, em);
        }

        // phase 4: residual scale and codes
        float esn[4];
        if (RSCALE == CARRY_SCALE_PER_V) {
#pragma unroll
          for (int i = 0; i < 4; ++i) esn[i] = scale_from_amax(warp_max8(eamax[i]), rqmax, p.eps_mode);
        } else {
          eamax_all = warp_max32(eamax_all);
          if (lane == 0) head_red[it & 1][warp] = eamax_all;
          warps_meet(&meet_bar[2], meet_parity, lane, poison, p.status);
          float m = head_red[it & 1][0];
#pragma unroll
          for (int w = 1; w < kWarps; ++w) m = fmaxf(m, head_red[it & 1][w]);
          const float e1 = scale_from_amax(m, rqmax, p.eps_mode);
          esn[0] = esn[1] = esn[2] = esn[3] = e1;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float inv = __fdiv_rn(1.0f, esn[i]);
          if (RES == CARRY_RES_INT4) {
            uint32_t words[2];
#pragma unroll
            for (int m = 0; m < 2; ++m) {
              uint32_t acc = 0;
#pragma unroll
              for (int b = 7; b >= 0; --b) {
                float ms;
                quant_code<EXACT>(h[i][8 * m + b], esn[i], inv, ms);
                acc = (acc << 4) | (__float_as_uint(ms) & 0xFu);
              }
              words[m] = acc;
            }
            *reinterpret_cast<uint2*>(sb + L::kResid + (r0 + i) * (kT / 2) + c0 / 2) = make_uint2(words[0], words[1]);
          } else {
            uint32_t packed[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
              uint32_t y[4];
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                float ms;
                quant_code<EXACT>(h[i][4 * m + b], esn[i], inv, ms);
                y[b] = __float_as_uint(ms);
              }
              packed[m] = __byte_perm(__byte_perm(y[0], y[1], 0x0040), __byte_perm(y[2], y[3], 0x0040), 0x5410);
            }
            *reinterpret_cast<uint4*>(sb + L::kResid + (r0 + i) * kT + c0) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
        if (cg == 0) {
          *reinterpret_cast<float4*>(sb + L::kSScale + r0 * 4) = make_float4(snew[0], snew[1], snew[2], snew[3]);
          if (RSCALE == CARRY_SCALE_PER_V)
            *reinterpret_cast<float4*>(sb + L::kRScale + r0 * 4) = make_float4(esn[0], esn[1], esn[2], esn[3]);
        }
        if (RSCALE == CARRY_SCALE_PER_HEAD && tid == 0) {
          float* dst = p.packed ? p.rscale_out + (long long)slot * p.stride_rscale_slot + hv
                                : p.rscale_out + (long long)n * p.HV + hv;
          *dst = esn[0];
        }
      } else {
        // ---------------- statequant layout [K][V]: lane = 4 columns x 16 rows ----
        const int r0 = 16 * warp, c0 = 4 * lane;
        float* red_dot = col_red;                       // [warp][col][2]
        float* red_max = col_red + kWarps * kT * 2;     // [warp][col]
        float* red_emax = red_max + kWarps * kT;        // [warp][col]
        float krow[16], qrow[16];
        load16(sb + L::kK, r0, p.qkv_dtype, krow);
        load16(sb + L::kQ, r0, p.qkv_dtype, qrow);
        float kq = 0.f;
        {
          float part = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            part = fmaf(raw_to_float(sb + L::kK, 4 * lane + i, p.qkv_dtype),
                        raw_to_float(sb + L::kQ, 4 * lane + i, p.qkv_dtype), part);
          kq = warp_sum32(part);
        }
        float scol[4];
        {
          const float4 s4 = *reinterpret_cast<const float4*>(sscale + c0);
          scol[0] = s4.x; scol[1] = s4.y; scol[2] = s4.z; scol[3] = s4.w;
        }
        float h[16][4];
        float dk[4] = {0.f, 0.f, 0.f, 0.f}, dq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(sb + L::kCodes + (r0 + i) * kT + c0) ^ 0x80808080u;
          float c[4];
          c[0] = s8_to_float<0>(w); c[1] = s8_to_float<1>(w); c[2] = s8_to_float<2>(w); c[3] = s8_to_float<3>(w);
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const float hv_ = __fmul_rn(__fmul_rn(c[b], scol[b]), alpha);
            h[i][b] = hv_;
            dk[b] = fmaf(hv_, krow[i], dk[b]);
            dq[b] = fmaf(hv_, qrow[i], dq[b]);
          }
        }
        // finish the column sums across the 8 warps
        {
          float4* dst = reinterpret_cast<float4*>(red_dot + ((size_t)warp * kT + c0) * 2);
          dst[0] = make_float4(dk[0], dq[0], dk[1], dq[1]);
          dst[1] = make_float4(dk[2], dq[2], dk[3], dq[3]);
          warps_meet(&meet_bar[0], meet_parity, lane, poison, p.status);
#pragma unroll
          for (int b = 0; b < 4; ++b) { dk[b] = 0.f; dq[b] = 0.f; }
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const float4* src = reinterpret_cast<const float4*>(red_dot + ((size_t)w * kT + c0) * 2);
            const float4 x0 = src[0], x1 = src[1];
            dk[0] += x0.x; dq[0] += x0.y; dk[1] += x0.z; dq[1] += x0.w;
            dk[2] += x1.x; dq[2] += x1.y; dk[3] += x1.z; dq[3] += x1.w;
          }
        }
        float vcol[4], dv[4], oval[4];
        if (p.qkv_dtype == CARRY_F32) {
          const float4 v4 = *reinterpret_cast<const float4*>(sb + L::kV + c0 * 4);
          vcol[0] = v4.x; vcol[1] = v4.y; vcol[2] = v4.z; vcol[3] = v4.w;
        } else {
#pragma unroll
          for (int b = 0; b < 4; ++b) vcol[b] = raw_to_float(sb + L::kV, c0 + b, p.qkv_dtype);
        }
        float es_col[4];
        if (RSCALE == CARRY_SCALE_PER_V) {
          const float4 e4 = *reinterpret_cast<const float4*>(rscale + c0);
          es_col[0] = e4.x; es_col[1] = e4.y; es_col[2] = e4.z; es_col[3] = e4.w;
        } else {
          es_col[0] = es_col[1] = es_col[2] = es_col[3] = es_head;
        }
        float amax[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          dv[b] = __fmul_rn(beta, __fadd_rn(vcol[b], -dk[b]));
          oval[b] = fmaf(dv[b], kq, dq[b]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float e[4];
          if (RES == CARRY_RES_INT4) {
            const uint32_t w =
                (uint32_t)(*reinterpret_cast<const uint16_t*>(sb + L::kResid + (r0 + i) * (kT / 2) + c0 / 2)) ^ 0x8888u;
#pragma unroll
            for (int b2 = 0; b2 < 2; ++b2) {
              const uint32_t bits = __byte_perm(w, 0x4B000000u, 0x7440 | b2);
              e[2 * b2] = __fmul_rn(__uint_as_float(bits & 0xFFFFFF0Fu) - 8388616.0f, es_col[2 * b2]);
              e[2 * b2 + 1] = __fmul_rn(__uint_as_float(bits & 0xFFFFFFF0u) - kMagicByte, es_col[2 * b2 + 1] * 0.0625f);
            }
          } else {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(sb + L::kResid + (r0 + i) * kT + c0) ^ 0x80808080u;
            e[0] = __fmul_rn(s8_to_float<0>(w), es_col[0]); e[1] = __fmul_rn(s8_to_float<1>(w), es_col[1]);
            e[2] = __fmul_rn(s8_to_float<2>(w), es_col[2]); e[3] = __fmul_rn(s8_to_float<3>(w), es_col[3]);
          }
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const float t0 = __fadd_rn(__fadd_rn(h[i][b], __fmul_rn(krow[i], dv[b])), e[b]);
            h[i][b] = t0;
            amax[b] = fmaxf(amax[b], fabsf(t0));
          }
        }
        if (warp == 0) {
          if (p.o_dtype == CARRY_F32) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + out_off + c0) =
                make_float4(oval[0], oval[1], oval[2], oval[3]);
          } else {
#pragma unroll
            for (int b = 0; b < 4; ++b) store_from_float(p.out, out_off + c0 + b, p.o_dtype, oval[b]);
          }
        }
        *reinterpret_cast<float4*>(red_max + (size_t)warp * kT + c0) = make_float4(amax[0], amax[1], amax[2], amax[3]);
        warps_meet(&meet_bar[1], meet_parity, lane, poison, p.status);
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float4 x = *reinterpret_cast<const float4*>(red_max + (size_t)w * kT + c0);
          amax[0] = fmaxf(amax[0], x.x); amax[1] = fmaxf(amax[1], x.y);
          amax[2] = fmaxf(amax[2], x.z); amax[3] = fmaxf(amax[3], x.w);
        }
        float snew[4], inv_s[4], eamax[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          snew[b] = scale_from_amax(amax[b], p.qmax, p.eps_mode);
          inv_s[b] = __fdiv_rn(1.0f, snew[b]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          uint32_t y[4];
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            float ms;
            const float code = quant_code<EXACT>(h[i][b], snew[b], inv_s[b], ms);
            y[b] = __float_as_uint(ms);
            const float en = __fadd_rn(h[i][b], -__fmul_rn(code, snew[b]));
            h[i][b] = en;
            eamax[b] = fmaxf(eamax[b], fabsf(en));
          }
          *reinterpret_cast<uint32_t*>(sb + L::kCodes + (r0 + i) * kT + c0) =
              __byte_perm(__byte_perm(y[0], y[1], 0x0040), __byte_perm(y[2], y[3], 0x0040), 0x5410);
        }
        float esn[4];
        if (RSCALE == CARRY_SCALE_PER_V) {
          *reinterpret_cast<float4*>(red_emax + (size_t)warp * kT + c0) =
              make_float4(eamax[0], eamax[1], eamax[2], eamax[3]);
          warps_meet(&meet_bar[2], meet_parity, lane, poison, p.status);
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const float4 x = *reinterpret_cast<const float4*>(red_emax + (size_t)w * kT + c0);
            eamax[0] = fmaxf(eamax[0], x.x); eamax[1] = fmaxf(eamax[1], x.y);
            eamax[2] = fmaxf(eamax[2], x.z); eamax[3] = fmaxf(eamax[3], x.w);
          }
#pragma unroll
          for (int b = 0; b < 4; ++b) esn[b] = scale_from_amax(eamax[b], rqmax, p.eps_mode);
        } else {
          float m = warp_max32(fmaxf(fmaxf(eamax[0], eamax[1]), fmaxf(eamax[2], eamax[3])));
          if (lane == 0) head_red[it & 1][warp] = m;
          warps_meet(&meet_bar[2], meet_parity, lane, poison, p.status);
          m = head_red[it & 1][0];
#pragma unroll
          for (int w = 1; w < kWarps; ++w) m = fmaxf(m, head_red[it & 1][w]);
          esn[0] = esn[1] = esn[2] = esn[3] = scale_from_amax(m, rqmax, p.eps_mode);
        }
        float inv_e[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) inv_e[b] = __fdiv_rn(1.0f, esn[b]);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          uint32_t y[4];
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            float ms;
            quant_code<EXACT>(h[i][b], esn[b], inv_e[b], ms);
            y[b] = __float_as_uint(ms);
          }
          if (RES == CARRY_RES_INT4) {
            const uint32_t v16 = (y[0] & 0xFu) | ((y[1] & 0xFu) << 4) | ((y[2] & 0xFu) << 8) | ((y[3] & 0xFu) << 12);
            *reinterpret_cast<uint16_t*>(sb + L::kResid + (r0 + i) * (kT / 2) + c0 / 2) = (uint16_t)v16;
          } else {
            *reinterpret_cast<uint32_t*>(sb + L::kResid + (r0 + i) * kT + c0) =
                __byte_perm(__byte_perm(y[0], y[1], 0x0040), __byte_perm(y[2], y[3], 0x0040), 0x5410);
          }
        }
        // scales: every warp holds all 128 of them; warp w publishes its 16-column share
        // (columns 16w..16w+15 are held by lanes 4w..4w+3)
        if ((lane >> 2) == warp) {
          *reinterpret_cast<float4*>(sb + L::kSScale + c0 * 4) = make_float4(snew[0], snew[1], snew[2], snew[3]);
          if (RSCALE == CARRY_SCALE_PER_V)
            *reinterpret_cast<float4*>(sb + L::kRScale + c0 * 4) = make_float4(esn[0], esn[1], esn[2], esn[3]);
        }
        if (RSCALE == CARRY_SCALE_PER_HEAD && tid == 0) p.rscale_out[(long long)n * p.HV + hv] = esn[0];
      }
    }

    if (live) meet_parity ^= 1u;

    // ---- this warp's 16 rows go back; free the previous stage; refill it ---------
    __syncwarp();
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (live && !*poison) {
        int8_t* codes_out;
        uint8_t* resid_out;
        float *ss_out, *rs_out;
        if (p.packed) {
          codes_out = p.codes_out + (long long)slot * p.stride_state_slot + (long long)hv * kT * kT;
          resid_out = reinterpret_cast<uint8_t*>(p.resid_out) + (long long)slot * p.stride_resid_slot +
                      (long long)hv * L::kResidBytes;
          ss_out = p.sscale_out + (long long)slot * p.stride_sscale_slot + (long long)hv * kT;
          rs_out = p.rscale_out + (long long)slot * p.stride_rscale_slot + (long long)hv * kT;
        } else {
          const long long nh = (long long)n * p.HV + hv;
          codes_out = p.codes_out + nh * kT * kT;
          resid_out = reinterpret_cast<uint8_t*>(p.resid_out) + nh * L::kResidBytes;
          ss_out = p.sscale_out + nh * kT;
          rs_out = p.rscale_out + nh * kT;
        }
        constexpr int kRowsB = 16 * kT;                       // bytes of 16 rows of codes
        constexpr int kResRowsB = L::kResidBytes / kWarps;    // bytes of 16 rows of residual
        bulk_store(codes_out + warp * kRowsB, sb + L::kCodes + warp * kRowsB, kRowsB);
        bulk_store(resid_out + warp * kResRowsB, sb + L::kResid + warp * kResRowsB, kResRowsB);
        bulk_store(ss_out + warp * 16, sb + L::kSScale + warp * 64, 64);
        if (RSCALE == CARRY_SCALE_PER_V) bulk_store(rs_out + warp * 16, sb + L::kRScale + warp * 64, 64);
      }
      bulk_commit();
      // Stage (it-1) % S is free once every warp's stores of tile it-1 have left
      // shared memory.  The warp that observes this last refills the stage, so
      // nobody waits here.
      if (it > 0 && it - 1 + S < my_tiles) {
        bulk_wait_read<1>();
        __threadfence_block();
        const int prev = (it - 1) % S;
        if (atomicAdd(&done_cnt[prev], 1) == kWarps - 1) {
          __threadfence_block();
          done_cnt[prev] = 0;
          if (!*poison) issue(it - 1 + S);
        }
      }
    }
  }
  if (lane == 0) bulk_wait_read<0>();
  __syncthreads();
}

template <int LAYOUT, int RES, int RSCALE>
int launch_variant(const KParams& p, cudaStream_t stream, int sms) {
  auto kern = gdn_tile128_kernel<LAYOUT, RES, RSCALE, true>;
  using L = StageLayout<RES, LAYOUT>;
  const size_t smem = (size_t)L::kBytes * L::kStages;
  static thread_local bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return CARRY_GDN_ERR_NO_DEVICE;
  if (dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return CARRY_GDN_ERR_NO_DEVICE;
    }
    configured[dev] = true;
  }
  const long long tiles = (long long)p.B * p.HV;
  const long long ctas = (long long)L::kCtasPerSm * sms;
  const int grid = (int)(tiles < ctas ? tiles : ctas);
  kern<<<grid, kThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// The streaming kernel needs 16-byte aligned, dense rows for every bulk copy.
bool tile128_eligible(const KParams& p) {
  if (p.K != kT || p.V != kT) return false;
  if (p.res_fmt != CARRY_RES_INT8 && p.res_fmt != CARRY_RES_INT4) return false;
  if (p.sscale_mode != CARRY_SCALE_PER_V) return false;
  if (p.HV > kT || (long long)p.B * p.HV > 0x7fffffffLL) return false;
  const int qes = p.qkv_dtype == CARRY_F32 ? 4 : 2;
  if (!aligned16(p.codes_in) || !aligned16(p.codes_out) || !aligned16(p.resid_in) || !aligned16(p.resid_out) ||
      !aligned16(p.sscale_in) || !aligned16(p.sscale_out) || !aligned16(p.rscale_in) || !aligned16(p.rscale_out) ||
      !aligned16(p.q) || !aligned16(p.k) || !aligned16(p.v) || !aligned16(p.out))
    return false;
  if (p.packed) {
    const int ges = p.ab_dtype == CARRY_F32 ? 4 : 2;
    if (!aligned16(p.a) || !aligned16(p.b)) return false;
    if ((p.stride_a_tok * ges) % 16 || (p.stride_b_tok * ges) % 16 || (p.HV * ges) % 16) return false;
    if ((p.stride_mixed_tok * qes) % 16) return false;
    if (p.stride_state_slot % 16 || p.stride_resid_slot % 16 || p.stride_sscale_slot % 4) return false;
    if (p.rscale_mode == CARRY_SCALE_PER_V ? (p.stride_rscale_slot % 4) : (p.stride_rscale_slot % 4 || p.HV % 4))
      return false;
  } else {
    if (!aligned16(p.alpha) || !aligned16(p.beta) || p.HV % 4) return false;
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
  const int n = sms[dev];
  const bool i4 = p.res_fmt == CARRY_RES_INT4, pv = p.rscale_mode == CARRY_SCALE_PER_V;
  if (p.packed) {
    if (i4) return pv ? launch_variant<LAYOUT_VK, CARRY_RES_INT4, CARRY_SCALE_PER_V>(p, stream, n)
                      : launch_variant<LAYOUT_VK, CARRY_RES_INT4, CARRY_SCALE_PER_HEAD>(p, stream, n);
    return pv ? launch_variant<LAYOUT_VK, CARRY_RES_INT8, CARRY_SCALE_PER_V>(p, stream, n)
              : launch_variant<LAYOUT_VK, CARRY_RES_INT8, CARRY_SCALE_PER_HEAD>(p, stream, n);
  }
  if (i4) return pv ? launch_variant<LAYOUT_KV, CARRY_RES_INT4, CARRY_SCALE_PER_V>(p, stream, n)
                    : launch_variant<LAYOUT_KV, CARRY_RES_INT4, CARRY_SCALE_PER_HEAD>(p, stream, n);
  return pv ? launch_variant<LAYOUT_KV, CARRY_RES_INT8, CARRY_SCALE_PER_V>(p, stream, n)
            : launch_variant<LAYOUT_KV, CARRY_RES_INT8, CARRY_SCALE_PER_HEAD>(p, stream, n);
}

}  // namespace carry
