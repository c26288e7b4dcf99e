// Streaming kernel for the serving shape: K = V = 128, int8 state, int8 or packed
// int4 residual.  One (request, head) tile is 16 KB of codes + 8/16 KB of
// residual; all of it is contiguous in memory in both layouts, so every tile
// moves with a handful of 1-D bulk async copies (TMA, no tensor map):
//
//   global --cp.async.bulk--> shared stage --> registers --16-byte stores--> global
//
// One persistent CTA per SM walks its share of the tile list (tile = blockIdx.x +
// number * gridDim.x) through a ring of stages: while tiles are computed, the loads
// of the next ones are in flight.  The CTA holds two groups of 8 warps (a single
// group only if two stages per group did not fit); each group works on a
// whole tile, and the groups take tiles off the CTA's list as they go, because the
// two do not get equal shares of the SM's issue slots.  A stage is handed back
// right after the tile's last meeting, when its last byte has been read, and
// results leave straight from registers as 16-byte vector stores that cover whole
// 128-byte lines.  The state is read from HBM once and written once.
//
// Work split inside a group (256 threads = 8 warps): warp w owns memory rows
// 16w..16w+15 of the tile.
//   * slot layout [V][K] (scale per row): lane = (row group rg, column group
//     cg): 4 rows x 16 contiguous columns.  Everything the math reduces over
//     (K) lies along the row, so reductions are shuffles inside 8 lanes; the
//     warps meet once per tile (for the per-head residual scale, and to agree on
//     the next tile).
//   * statequant layout [K][V] (scale per column): lane = 4 contiguous columns
//     x the warp's 16 rows; column sums are finished across the 8 warps through
//     shared memory (three meetings per tile).
//
// Arithmetic.  Everything that feeds a state code keeps the reference's operation
// order, with the contractions written out as explicit fused multiply-adds:
// h = (code*scale)*alpha, h' = fma(k, dv, h), target = fma(resid_code, resid_scale, h'),
// remainder = fma(code', -scale', target).  Scales are amax / qmax by an exact
// shortcut (div_qmax).  round(target / s) is evaluated as rint(target * (1/s)) with a
// reciprocal good to 2^-24; the two can only differ when the quotient is within ~8e-6
// of a tie, which shows up as a remainder within 2^-16 of half a step -- rows where
// that happens are re-decided with the true division.  Residual codes use
// rint(e * (1/es)) as is.  Math runs as packed f32x2 (IEEE round-to-nearest per
// component).
#pragma once
#include "carry_gdn_common.cuh"

namespace carry {
namespace {

constexpr int kT = 128;                 // tile edge
constexpr int kThreads = 256;          // threads of one group: the 8 warps that share a tile
constexpr int kWarps = 8;
// Polls of a stage barrier before a wait gives up.  CARRY_TEST_WAIT_EXPIRY builds a test-only library in
// which the copies of global tile 1 announce 16 bytes more than they bring, so that its barrier never
// completes, and the limit is short: the expiry path (status bit, poisoned CTA, pool left untouched) then
// runs in a fraction of a millisecond without anything faulting or hanging.  In the same library the
// streaming kernel treats the set-up inputs of every tile whose index has bit 1 set as changed under its
// feet (see the kernel's prologue), so that the path of a launch whose inputs were still being written
// when it looked at them first runs too -- results must not depend on it.
#ifdef CARRY_TEST_WAIT_EXPIRY
constexpr uint32_t kSpinLimit = 1u << 11;
__device__ __forceinline__ uint32_t test_extra_tx(int tile) { return tile == 1 ? 16u : 0u; }
__device__ __forceinline__ bool test_inputs_changed(int tile) { return (tile & 2) != 0; }
// ... and reports, in a status bit of its own, when a tile's inputs really had changed between the two looks
// (tests/test_gpu_wait_expiry.py provokes that with a kernel that writes them late)
constexpr int kTestStatusInputsChanged = 1 << 30;
__device__ __forceinline__ void test_note_changed(int* status, bool same) {
  if (!same && status) atomicOr(status, kTestStatusInputsChanged);
}
#else
constexpr uint32_t kSpinLimit = 1u << 22;
__device__ __forceinline__ uint32_t test_extra_tx(int) { return 0u; }
__device__ __forceinline__ bool test_inputs_changed(int) { return false; }
__device__ __forceinline__ void test_note_changed(int*, bool) {}
#endif
constexpr int kTileCache = 64;         // per group: cached slot ids and gates of the CTA's first tiles

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

// Hints to the L2 (no data is consumed, nothing waits): a whole run of bytes, or the lines of a short vector.
__device__ __forceinline__ void l2_prefetch_bulk(const void* src_gmem, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void l2_prefetch_line(const void* src_gmem) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(src_gmem));
}

// Bounded wait: after kSpinLimit failed polls the CTA is marked poisoned, the
// status word gets the timeout bit and every later wait returns at once; a
// poisoned CTA stops loading and storing.
__device__ __noinline__ void mbar_wait_slow(uint64_t* bar, uint32_t parity, volatile int* poison, int* status) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return;
    if (spin > 64) __nanosleep(64);
    if ((spin & 1023) == 1023 && *poison) return;
  }
  *poison = 1;
  if (status) atomicOr(status, CARRY_GDN_STATUS_TIMEOUT);
}
// returns false when the CTA is poisoned (the data behind the barrier must not be used)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* poison, int* status) {
  if (mbar_try_wait(bar, parity)) return true;
  if (!*poison) mbar_wait_slow(bar, parity, poison, status);
  return !*poison;
}
// The wait of the streaming kernel's ring.  A stage holds the tile whose number `*requested` says (written
// by the thread that requests a tile, before the request): a group that has got ahead of a stalled one
// reaches tiles nobody has requested yet -- the request for tile n + S is made when tile n is done -- and
// must not take the stage's previous phase for theirs.  It polls here, within the same limit, instead.
__device__ __noinline__ void tile_wait_slow(uint64_t* bar, uint32_t parity, const volatile int* requested, int num,
                                            volatile int* poison, int* status) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (*requested == num && mbar_try_wait(bar, parity)) return;
    if (spin > 64) __nanosleep(64);
    if ((spin & 1023) == 1023 && *poison) return;
  }
  *poison = 1;
  if (status) atomicOr(status, CARRY_GDN_STATUS_TIMEOUT);
}
__device__ __forceinline__ bool tile_wait(uint64_t* bar, uint32_t parity, const volatile int* requested, int num,
                                          volatile int* poison, int* status) {
  const int req = *requested;                        // both looks are on their way before either is needed
  const bool landed = mbar_try_wait(bar, parity);
  if (landed & (req == num)) return true;
  if (!*poison) tile_wait_slow(bar, parity, requested, num, poison, status);
  return !*poison;
}
__device__ __forceinline__ uint4 lds_v4(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void stg_v4(unsigned long long addr, uint4 v) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// the same with a compile-time byte offset, so that one base register serves a run of stores
template <int OFF>
__device__ __forceinline__ void stg_v4_at(unsigned long long base, uint4 v) {
  asm volatile("st.global.v4.b32 [%0+%5], {%1, %2, %3, %4};" ::"l"(base), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ void stg_v2_at(unsigned long long base, uint2 v) {
  asm volatile("st.global.v2.b32 [%0+%3], {%1, %2};" ::"l"(base), "r"(v.x), "r"(v.y), "n"(OFF));
}
// A shared-memory load the compiler may schedule freely (it is not volatile and claims no memory
// effect) but may neither merge with the same load of another row (TAG differs) nor keep in registers
// across rows.  Ordering against the stores that filled the location comes from `base`: it has to be
// derived from order_token(), called after those stores and the barrier that publishes them.
template <int OFF, int TAG>
__device__ __forceinline__ float4 lds_f4_at(uint32_t base) {
  float4 v;
  asm("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];  // row %6" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
      : "r"(base), "n"(OFF), "n"(TAG));
  return v;
}
// a zero the compiler cannot see through, defined at this point of the program
__device__ __forceinline__ uint32_t order_token() {
  uint32_t t;
  asm volatile("mov.u32 %0, 0;" : "=r"(t) : : "memory");
  return t;
}
__device__ __forceinline__ void stg_b32(unsigned long long addr, uint32_t v) {
  asm volatile("st.global.b32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void stg_b16(unsigned long long addr, uint32_t v) {
  asm volatile("st.global.b16 [%0], %1;" ::"l"(addr), "h"((unsigned short)v) : "memory");
}

// The 8 warps of a group meet on a hardware named barrier (ids 1..3 for group 0, 4..6 for group 1).
// Every thread of a group runs the same tiles and reaches the same number of meetings in each of them
// whether or not the tile is live (skipped tiles take them in the else branch), so a meeting cannot be
// left waiting for a warp that never comes.  Waits on data in flight (the stage barriers) are the
// bounded ones.
__device__ __forceinline__ void warps_meet(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kThreads) : "memory"); }

// ---------------------------------------------------------------------------
// packed fp32 helpers (each maps to one f32x2 instruction)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 splat(float x) { return make_float2(x, x); }
__device__ __forceinline__ float max3abs(float m, float2 x) { return fmaxf(fmaxf(m, fabsf(x.x)), fabsf(x.y)); }

constexpr float kMagicRound = 12582912.0f;      // 1.5 * 2^23: x + M rounds x to an integer (RNE)
constexpr float kMagicByte = 8388736.0f;        // 2^23 + 128
constexpr float kMagicNib = 8388616.0f;         // 2^23 + 8
constexpr float kTieGuard = 0.4999847412109375f;  // 0.5 - 2^-16

// bytes A and B of w (each already XOR-ed with 0x80) -> {float(code A), float(code B)}
template <int A, int B>
__device__ __forceinline__ float2 s8x2_to_float(uint32_t w) {
  const float2 m = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440 | A)),
                               __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440 | B)));
  return add2(m, splat(-kMagicByte));
}
// signed bytes A and B of w (as stored, no bias) -> floats, by the conversion instruction, which picks the
// byte itself.  It runs on the quarter-rate conversion pipe, which has nothing else to do in these kernels:
// against the byte-permute route (s8x2_to_float) it frees 1.25 ALU instructions and half a packed add per
// element on the two pipes that bound the kernel.
template <int A, int B>
__device__ __forceinline__ float2 s8x2_cvt(uint32_t w) {
  return make_float2((float)(signed char)((w >> (8 * A)) & 0xffu), (float)(signed char)((w >> (8 * B)) & 0xffu));
}
// bytes A and B of w, each a nibble in offset binary (0..15 = code + 8) -> {136 + code A, 136 + code B}:
// the byte is placed right above the low half-word of a float whose exponent byte says 128
template <int A, int B>
__device__ __forceinline__ float2 nib2_biased(uint32_t w) {
  return make_float2(__uint_as_float(__byte_perm(w, 0x43000000u, 0x7044 | (A << 8))),
                     __uint_as_float(__byte_perm(w, 0x43000000u, 0x7044 | (B << 8))));
}
// four fp8-e5m2 values in a word -> floats.  An e5m2 value is the upper byte of the half with the same
// value, so each pair of bytes becomes a half2 by one byte permute.
__device__ __forceinline__ void e5m2x4_to_float(uint32_t w, float2& ab, float2& cd) {
  const uint32_t h01 = __byte_perm(w, 0u, 0x1404), h23 = __byte_perm(w, 0u, 0x3424);
  ab = __half22float2(*reinterpret_cast<const __half2*>(&h01));
  cd = __half22float2(*reinterpret_cast<const __half2*>(&h23));
}
// ... and back, round to nearest even, saturating at the largest finite value
__device__ __forceinline__ uint32_t float4_to_e5m2x4(float2 ab, float2 cd) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(ab, __NV_SATFINITE, __NV_E5M2);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(cd, __NV_SATFINITE, __NV_E5M2);
  return lo | (hi << 16);
}
// bytes A and B of w (each nibble already XOR-ed with 8): {low nibbles}, {16 * high nibbles}
template <int A, int B>
__device__ __forceinline__ void s4x4_to_float(uint32_t w, float2& lo, float2& hi16) {
  const uint32_t a = __byte_perm(w, 0x4B000000u, 0x7440 | A), b = __byte_perm(w, 0x4B000000u, 0x7440 | B);
  lo = add2(make_float2(__uint_as_float(a & 0xFFFFFF0Fu), __uint_as_float(b & 0xFFFFFF0Fu)), splat(-kMagicNib));
  hi16 = add2(make_float2(__uint_as_float(a & 0xFFFFFFF0u), __uint_as_float(b & 0xFFFFFFF0u)), splat(-kMagicByte));
}
// the same from a word whose low nibbles (wl = w & 0x0F0F0F0F) and high nibbles (wh = w & 0xF0F0F0F0)
// were separated beforehand: two masks per word instead of four per byte pair
template <int A, int B>
__device__ __forceinline__ void s4x4_split_to_float(uint32_t wl, uint32_t wh, float2& lo, float2& hi16) {
  lo = add2(make_float2(__uint_as_float(__byte_perm(wl, 0x4B000000u, 0x7440 | A)),
                        __uint_as_float(__byte_perm(wl, 0x4B000000u, 0x7440 | B))), splat(-kMagicNib));
  hi16 = add2(make_float2(__uint_as_float(__byte_perm(wh, 0x4B000000u, 0x7440 | A)),
                          __uint_as_float(__byte_perm(wh, 0x4B000000u, 0x7440 | B))), splat(-kMagicByte));
}
// low bytes of four words -> one word (a | b<<8 | c<<16 | d<<24)
__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// max of a non-negative float over the whole warp: for non-negative floats the order of the bit
// patterns is the order of the values, so the integer warp reduction does it in one instruction.
// (Only with the full mask: a reduction over part of a warp costs some 300 cycles on sm_100.)
__device__ __forceinline__ float warp_max_nonneg(float x) {
  return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(x)));
}

// Four values per lane, each to be maximised over the 8 lanes of a row group.  Halving exchange: lane g
// of the group ends up with the maximum of x[(g >> 1) & 3], at 4 shuffles instead of 12.
__device__ __forceinline__ float group_max4_transposed(const float (&x)[4], int g) {
  const bool up4 = g & 4, up2 = g & 2;
  float a[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float keep = up4 ? x[2 + i] : x[i], send = up4 ? x[i] : x[2 + i];
    a[i] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 4));
  }
  const float keep = up2 ? a[1] : a[0], send = up2 ? a[0] : a[1];
  const float b = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, 2));
  return fmaxf(b, __shfl_xor_sync(0xffffffffu, b, 1));
}

// 1/s to within 2^-24 (1 + 2^-20) relative: the hardware approximation (1 ulp) and one Newton step.  The
// rounding routine only needs the reciprocal that close -- quotients that the difference could tip over a
// tie are caught by the tie guard and re-decided by a true division -- and this is a third of the
// latency of the correctly rounded routine.  s is a scale: normal, between 1e-12 and 1e37.
__device__ __forceinline__ float rcp_refined(float s) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(s));
  return fmaf(y, fmaf(-s, y, 1.0f), y);
}

// Eight values per lane (x[0..3], y[0..3]), each to be summed over the 8 lanes of a row group.
// Halving exchange: after three rounds lane g of the group holds one total -- x[g] for g < 4,
// y[g - 4] otherwise -- at 7 shuffles instead of 24.
__device__ __forceinline__ float group_sum8_transposed(const float (&x)[4], const float (&y)[4], int g) {
  const bool up4 = g & 4, up2 = g & 2, up1 = g & 1;
  float a[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float keep = up4 ? y[i] : x[i], send = up4 ? x[i] : y[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
  float b[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float keep = up2 ? a[2 + i] : a[i], send = up2 ? a[i] : a[2 + i];
    b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  const float keep = up1 ? b[1] : b[0], send = up1 ? b[0] : b[1];
  return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

// amax / qmax, correctly rounded, without the division routine.  `rq` is 1/qmax rounded to nearest;
// a * rq is within an ulp of the quotient, the remainder a - qmax * q0 is exact in one fused
// multiply-add and corrects it.  Equal to IEEE division for every float a >= 2^-100 when qmax is one of
// 3, 7, 15, 31, 63, 127 (checked over every mantissa; tests/test_host_api.py repeats the check), and the
// launcher admits no other qmax.  Smaller a end at the 1e-12 floor either way.
__device__ __forceinline__ float div_qmax(float a, float qmax, float rq) {
  const float q0 = __fmul_rn(a, rq);
  return fmaf(fmaf(-qmax, q0, a), rq, q0);
}
__device__ __forceinline__ float scale_fast(float amax, float qmax, float rq, int eps_mode) {
  if (eps_mode == CARRY_EPS_ON_AMAX) return div_qmax(fmaxf(amax, kEps), qmax, rq);
  return fmaxf(div_qmax(amax, qmax, rq), kEps);
}


// ---------------------------------------------------------------------------
// shared-memory stage layout (bytes)
// ---------------------------------------------------------------------------
// Static shared memory next to the stage ring: barriers, the per-CTA tile caches,
// the per-warp q scratch (slot layout) or the column-reduction space (statequant
// layout).  Upper bounds, used to size the ring.
constexpr int kStaticVK = 11776;        // per group
constexpr int kStaticKV = 24064;
constexpr int kStaticOf(int layout) { return layout == 0 ? kStaticVK : kStaticKV; }
constexpr int kSmemPerCta = 231424;     // one CTA per SM: 227 KB less 1 KB

template <int RES, int LAYOUT, int QDT, int RSCALE>
struct StageLayout {
  static constexpr int kVecBytes = kT * (QDT == CARRY_F32 ? 4 : 2);
  // integer residuals carry a scale (per V or per head); the float ones (fp32, fp16, fp8-e5m2) do not
  static constexpr bool kFloatResid = RES == CARRY_RES_FP32 || RES == CARRY_RES_FP16 || RES == CARRY_RES_FP8;
  static constexpr int kResidBytes = (RES == CARRY_RES_INT4) ? kT * kT / 2
                                     : (RES == CARRY_RES_FP32) ? kT * kT * 4
                                     : (RES == CARRY_RES_FP16) ? kT * kT * 2 : kT * kT;
  static constexpr int kCodes = 0;
  static constexpr int kResid = kT * kT;
  static constexpr int kSScale = kResid + kResidBytes;       // 128 floats
  static constexpr int kRScale = kSScale + 512;              // 128 floats (per V), or the 16 bytes that hold
  static constexpr int kRScaleBytes = kFloatResid ? 0 : (RSCALE == CARRY_SCALE_PER_V) ? 512 : 16;   // this head's scale (per head)
  static constexpr int kQ = kRScale + (kFloatResid ? 0 : (RSCALE == CARRY_SCALE_PER_V) ? 512 : 128);   // raw q, k, v of this head
  static constexpr int kK = kQ + kVecBytes;
  static constexpr int kV = kK + kVecBytes;
  static constexpr int kBytes = kV + kVecBytes;
  static_assert(kBytes % 128 == 0, "stages keep the ring's 128-byte alignment");
  // Two groups of 8 warps share one CTA (and one SM) when at least 2 stages per group fit (every
  // variant today; 128 registers per thread then), else the CTA is a single group.
  static constexpr int kGroups =
      ((4 * kBytes + 2 * kStaticOf(LAYOUT) <= kSmemPerCta) ? 2 : 1);
  static constexpr int kStatic = kGroups * kStaticOf(LAYOUT);
  static constexpr int kBudget = kSmemPerCta - kStatic;
  static constexpr int kFit = kBudget / kBytes;
  // a deeper ring does not help (a tile takes several times longer to compute than to load) and makes the
  // burst of requests at the start of a launch larger: 6 stages measured best for two groups (4..8 tried)
  static constexpr int kStageCap = (kGroups == 2) ? 6 : 5;
  static constexpr int kStages = kFit > kStageCap ? kStageCap : kFit;
};




// activations of one head as they sit in the stage (element type QDT) -> fp32
template <int QDT>
__device__ __forceinline__ float act(const uint8_t* base, int i) {
  if (QDT == CARRY_F32) return reinterpret_cast<const float*>(base)[i];
  if (QDT == CARRY_BF16) return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(base)[i] << 16);
  return __half2float(reinterpret_cast<const __half*>(base)[i]);
}
// two consecutive 16-bit activations packed in one word -> {first, second}
template <int QDT>
__device__ __forceinline__ float2 act_pair(uint32_t w) {
  if (QDT == CARRY_BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
// four consecutive activations starting at element `first` (a multiple of 4)
template <int QDT>
__device__ __forceinline__ float4 act4(const uint8_t* base, int first) {
  if (QDT == CARRY_F32) return *reinterpret_cast<const float4*>(base + first * 4);
  const uint2 w = *reinterpret_cast<const uint2*>(base + first * 2);
  const float2 a = act_pair<QDT>(w.x), b = act_pair<QDT>(w.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
// 16 consecutive activations starting at `first` (a multiple of 16), as column pairs per quad:
// E[m] = {x[4m], x[4m+2]}, O[m] = {x[4m+1], x[4m+3]}, each times `mul`
template <int QDT>
__device__ __forceinline__ void act16_pairs(const uint8_t* base, int first, float mul, float2 (&E)[4], float2 (&O)[4]) {
  const float2 m2 = make_float2(mul, mul);
  if (QDT == CARRY_F32) {
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const float4 x = *reinterpret_cast<const float4*>(base + (first + 4 * m) * 4);
      E[m] = __fmul2_rn(make_float2(x.x, x.z), m2);
      O[m] = __fmul2_rn(make_float2(x.y, x.w), m2);
    }
  } else {
    const uint4 lo = *reinterpret_cast<const uint4*>(base + first * 2);
    const uint4 hi = *reinterpret_cast<const uint4*>(base + first * 2 + 16);
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const float2 a = act_pair<QDT>(w[2 * m]), b = act_pair<QDT>(w[2 * m + 1]);
      E[m] = __fmul2_rn(make_float2(a.x, b.x), m2);
      O[m] = __fmul2_rn(make_float2(a.y, b.y), m2);
    }
  }
}

__device__ __noinline__ float exact_code(float t, float s) { return rintf(__fdiv_rn(t, s)); }

// Re-decide one element whose remainder sits within the tie guard: its code becomes rint of the
// true quotient target / s.  `y` is code + kMagicRound, `e` the remainder; the target is rebuilt
// exactly from them (remainder and code * s add up to a representable number).
__device__ __forceinline__ void redecide_rec(float& e, float& y, float s, float thr) {
  if (fabsf(e) > thr) {
    const float t = fmaf(__fadd_rn(y, -kMagicRound), s, e);
    const float code = exact_code(t, s);
    y = __fadd_rn(code, kMagicRound);
    e = fmaf(code, -s, t);
  }
}

// One scalar of element type `dtype` as raw bits, and the bits as a float.  Split in two so that a caller
// can have all its loads in flight before the first conversion waits for one: load_as_float() in a row
// makes every load wait for the previous one's conversion (a trip to memory each).
__device__ __forceinline__ uint32_t load_raw(const void* p, long long i, int dtype) {
  if (dtype == CARRY_F32) return __ldcg(reinterpret_cast<const uint32_t*>(p) + i);
  return __ldcg(reinterpret_cast<const unsigned short*>(p) + i);
}
__device__ __forceinline__ float raw_to_float(uint32_t r, int dtype) {
  if (dtype == CARRY_F32) return __uint_as_float(r);
  if (dtype == CARRY_BF16) return __uint_as_float(r << 16);
  return __half2float(__ushort_as_half((unsigned short)r));
}

// Gates of one (request, head): derived in the kernel on the slot path, given on the other.  The loads
// (gate_loads) and the arithmetic (gates_from) are separate calls for the reason above.
struct GateRaw { uint32_t a, b, A_log, dt_bias; };
__device__ __forceinline__ GateRaw gate_loads(const KParams& p, int n, int hv, long long tok_a, long long tok_b) {
  GateRaw r;
  if (p.packed) {
    r.a = load_raw(p.a, (long long)n * p.stride_a_tok + hv + tok_a, p.ab_dtype);
    r.b = load_raw(p.b, (long long)n * p.stride_b_tok + hv + tok_b, p.ab_dtype);
    r.A_log = load_raw(p.A_log, hv, p.A_log_dtype);
    r.dt_bias = load_raw(p.dt_bias, hv, p.dt_bias_dtype);
  } else {
    r.a = __float_as_uint(__ldcg(p.alpha + (long long)n * p.HV + hv));
    r.b = __float_as_uint(__ldcg(p.beta + (long long)n * p.HV + hv));
    r.A_log = r.dt_bias = 0u;
  }
  return r;
}
__device__ __forceinline__ void gates_from(const KParams& p, const GateRaw& r, float& alpha, float& beta) {
  if (p.packed) {
    slot_gates(raw_to_float(r.a, p.ab_dtype), raw_to_float(r.b, p.ab_dtype), raw_to_float(r.A_log, p.A_log_dtype),
               raw_to_float(r.dt_bias, p.dt_bias_dtype), alpha, beta);
  } else {
    alpha = __uint_as_float(r.a);
    beta = __uint_as_float(r.b);
  }
}

// tile index -> request row, value head, key head; shifts when the head counts are powers of two
__device__ __forceinline__ void split_tile(const KParams& p, int tile, int& n, int& hv, int& h) {
  if (p.hv_shift >= 0) { n = tile >> p.hv_shift; hv = tile & (p.HV - 1); }
  else { n = tile / p.HV; hv = tile - n * p.HV; }
  h = !p.packed ? hv : (p.group_shift >= 0 ? (hv >> p.group_shift) : hv / p.group);
}

// What a CTA needs to know about one of its tiles before the data arrives.
struct __align__(16) TileMeta {
  int n, hv, slot;
  float alpha, beta;
  float k_mul, q_mul;   // 1/|k| and scale/|q| (1 when the L2 norm is off or on the statequant path)
  float kq;             // <k, q> after those factors
};
static_assert(sizeof(TileMeta) == 32, "TileMeta is read as two 16-byte words");

// Where a tile's data lives: the four places its results go (codes, residual, state scales, residual
// scale(s)), then the sources that are not one of those (residual scales as read, q, k, v).  Codes,
// residual and state scales are read from the destination plus the launch-wide offset between the input
// and the output arrays (zero on the slot path, which works in place).
struct __align__(16) TileDesc {
  unsigned long long a[8];
};
enum { D_CODES = 0, D_RESID = 1, D_SSCALE = 2, D_RSCALE = 3, D_RSCALE_IN = 4, D_Q = 5, D_K = 6, D_V = 7 };

template <int RES, int RSCALE, int QDT>
__device__ __forceinline__ void tile_addresses(const KParams& p, int n, int hv, int h, long long slot,
                                               unsigned long long (&a)[8]) {
  constexpr int qes = (QDT == CARRY_F32) ? 4 : 2;
  constexpr long long KV = kT * kT;
  constexpr long long RB = (RES == CARRY_RES_INT4) ? KV / 2 : (RES == CARRY_RES_FP32) ? 4 * KV
                           : (RES == CARRY_RES_FP16) ? 2 * KV : KV;
  const long long nh = (long long)n * p.HV + hv;
  if (p.packed) {
    a[D_CODES] = reinterpret_cast<unsigned long long>(p.codes_out + slot * p.stride_state_slot + hv * KV);
    a[D_RESID] = reinterpret_cast<unsigned long long>(reinterpret_cast<uint8_t*>(p.resid_out) + slot * p.stride_resid_slot + hv * RB);
    a[D_SSCALE] = reinterpret_cast<unsigned long long>(p.sscale_out + slot * p.stride_sscale_slot + (long long)hv * kT);
    const float* rs = p.rscale_out + slot * p.stride_rscale_slot;
    a[D_RSCALE] = reinterpret_cast<unsigned long long>(rs + (RSCALE == CARRY_SCALE_PER_V ? (long long)hv * kT : (long long)hv));
    a[D_RSCALE_IN] = reinterpret_cast<unsigned long long>(rs + (RSCALE == CARRY_SCALE_PER_V ? (long long)hv * kT : (long long)(hv & ~3)));
    const uint8_t* row = reinterpret_cast<const uint8_t*>(p.q) + (long long)n * p.stride_mixed_tok * qes;
    a[D_Q] = reinterpret_cast<unsigned long long>(row + (long long)h * kT * qes);
    a[D_K] = reinterpret_cast<unsigned long long>(row + ((long long)p.H + h) * kT * qes);
    a[D_V] = reinterpret_cast<unsigned long long>(row + (2LL * p.H + hv) * kT * qes);
  } else {
    a[D_CODES] = reinterpret_cast<unsigned long long>(p.codes_out + nh * KV);
    a[D_RESID] = reinterpret_cast<unsigned long long>(reinterpret_cast<uint8_t*>(p.resid_out) + nh * RB);
    a[D_SSCALE] = reinterpret_cast<unsigned long long>(p.sscale_out + nh * kT);
    a[D_RSCALE] = reinterpret_cast<unsigned long long>(p.rscale_out + (RSCALE == CARRY_SCALE_PER_V ? nh * kT : nh));
    a[D_RSCALE_IN] = reinterpret_cast<unsigned long long>(p.rscale_in + (RSCALE == CARRY_SCALE_PER_V ? nh * kT : (nh & ~3LL)));
    a[D_Q] = reinterpret_cast<unsigned long long>(reinterpret_cast<const uint8_t*>(p.q) + nh * kT * qes);
    a[D_K] = reinterpret_cast<unsigned long long>(reinterpret_cast<const uint8_t*>(p.k) + nh * kT * qes);
    a[D_V] = reinterpret_cast<unsigned long long>(reinterpret_cast<const uint8_t*>(p.v) + nh * kT * qes);
  }
}

// A tile's set-up -- slot id, gates, the norms of k and q -- is worked out by LPT consecutive lanes (4, 8 or
// 32) straight from global memory: 128 / LPT elements of q and k per lane, then sums over the LPT lanes.
// Every load depends on the tile index alone, so the whole thing is one trip to memory however many tiles
// a CTA prepares at once.  The more lanes share a tile the shorter each lane's instruction stream: a CTA
// with few tiles (a small batch) gives a whole warp to each, and its first tile can start that much sooner.
// The sums are always taken in the same order -- groups of four consecutive elements, then a balanced tree
// over the groups in index order -- so the result does not depend on LPT (nor on which kernel of this
// library asks).  The routine comes in pieces -- the loads (meta_load: raw words, all in flight together,
// past the L1), the arithmetic, a pure function of those words (meta_math, meta_addresses), and the
// hand-over to shared memory (meta_put) -- because the streaming kernel runs the first two BEFORE its dependency wait,
// on whatever the inputs hold then, and afterwards only loads the words again: if they have not changed
// (meta_unchanged; the rule, since the arithmetic takes a microsecond and the kernel before this one has
// usually written them long ago) the result stands; if they have, tile_meta() below does it all over.
template <int QDT, int LPT>
struct MetaRaw {
  static_assert(LPT == 4 || LPT == 8 || LPT == 32, "lanes per tile");
  static constexpr int kElems = kT / LPT;                                     // elements per lane and vector
  static constexpr int kWords = kElems * ((QDT == CARRY_F32) ? 4 : 2) / 4;    // 32-bit words per lane and vector
  uint32_t qw[kWords], kw[kWords];
  int slot;
  GateRaw g;
};
// where a lane's share of q and k starts
template <int QDT, int LPT>
__device__ __forceinline__ void meta_vectors(const KParams& p, int n, int hv, int h, int sub, long long tok_qkv,
                                             const uint8_t*& qp, const uint8_t*& kp) {
  constexpr int qes = (QDT == CARRY_F32) ? 4 : 2;
  long long q_off, k_off;
  if (p.packed) {
    q_off = (long long)n * p.stride_mixed_tok + (long long)h * kT + tok_qkv;
    k_off = q_off + (long long)p.H * kT;
  } else {
    q_off = k_off = ((long long)n * p.HV + hv) * kT;
  }
  qp = reinterpret_cast<const uint8_t*>(p.q) + (q_off + MetaRaw<QDT, LPT>::kElems * sub) * qes;
  kp = reinterpret_cast<const uint8_t*>(p.k) + (k_off + MetaRaw<QDT, LPT>::kElems * sub) * qes;
}
template <int QDT, int LPT>
__device__ __forceinline__ void meta_load(const KParams& p, int n, int hv, int h, int sub, long long tok_qkv,
                                          long long tok_a, long long tok_b, MetaRaw<QDT, LPT>& r) {
  using R = MetaRaw<QDT, LPT>;
  const uint8_t *qp, *kp;
  meta_vectors<QDT, LPT>(p, n, hv, h, sub, tok_qkv, qp, kp);
  if constexpr (R::kWords >= 4) {
#pragma unroll
    for (int j = 0; j < R::kWords / 4; ++j) {
      const uint4 a = __ldcg(reinterpret_cast<const uint4*>(qp) + j), b = __ldcg(reinterpret_cast<const uint4*>(kp) + j);
      r.qw[4 * j] = a.x; r.qw[4 * j + 1] = a.y; r.qw[4 * j + 2] = a.z; r.qw[4 * j + 3] = a.w;
      r.kw[4 * j] = b.x; r.kw[4 * j + 1] = b.y; r.kw[4 * j + 2] = b.z; r.kw[4 * j + 3] = b.w;
    }
  } else {
    static_assert(R::kWords == 2, "a lane's share of a vector is at least 8 bytes");
    const uint2 a = __ldcg(reinterpret_cast<const uint2*>(qp)), b = __ldcg(reinterpret_cast<const uint2*>(kp));
    r.qw[0] = a.x; r.qw[1] = a.y; r.kw[0] = b.x; r.kw[1] = b.y;
  }
  r.slot = p.packed ? __ldcg(p.slot_idx + (long long)n * p.stride_idx) : 1;
  r.g = gate_loads(p, n, hv, tok_a, tok_b);
}
// The same loads again, compared with `x` as they come in: true when no word differs.  At most four 16-byte
// loads per vector are in flight at a time, so that the second look needs no second set of registers for
// the 32 words per vector of fp32 activations at four lanes per tile.
template <int QDT, int LPT>
__device__ __forceinline__ bool meta_unchanged(const KParams& p, int n, int hv, int h, int sub,
                                               const MetaRaw<QDT, LPT>& x) {
  using R = MetaRaw<QDT, LPT>;
  const uint8_t *qp, *kp;
  meta_vectors<QDT, LPT>(p, n, hv, h, sub, 0, qp, kp);
  const int slot = p.packed ? __ldcg(p.slot_idx + (long long)n * p.stride_idx) : 1;
  const GateRaw g = gate_loads(p, n, hv, 0, 0);
  uint32_t d = 0u;
  if constexpr (R::kWords >= 4) {
    constexpr int kQuads = R::kWords / 4, kBatch = kQuads < 4 ? kQuads : 4;
#pragma unroll
    for (int j0 = 0; j0 < kQuads; j0 += kBatch) {
      uint4 a[kBatch], b[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        a[j] = __ldcg(reinterpret_cast<const uint4*>(qp) + j0 + j);
        b[j] = __ldcg(reinterpret_cast<const uint4*>(kp) + j0 + j);
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        const int w = 4 * (j0 + j);
        d |= (a[j].x ^ x.qw[w]) | (a[j].y ^ x.qw[w + 1]) | (a[j].z ^ x.qw[w + 2]) | (a[j].w ^ x.qw[w + 3]);
        d |= (b[j].x ^ x.kw[w]) | (b[j].y ^ x.kw[w + 1]) | (b[j].z ^ x.kw[w + 2]) | (b[j].w ^ x.kw[w + 3]);
      }
      if (j0 + kBatch < kQuads) asm volatile("" ::: "memory");   // the next batch's loads stay behind this one's use
    }
  } else {
    const uint2 a = __ldcg(reinterpret_cast<const uint2*>(qp)), b = __ldcg(reinterpret_cast<const uint2*>(kp));
    d = (a.x ^ x.qw[0]) | (a.y ^ x.qw[1]) | (b.x ^ x.kw[0]) | (b.y ^ x.kw[1]);
  }
  d |= (uint32_t)(slot ^ x.slot) | (g.a ^ x.g.a) | (g.b ^ x.g.b) | (g.A_log ^ x.g.A_log) | (g.dt_bias ^ x.g.dt_bias);
  return d == 0u;
}
// fills m.alpha, beta, k_mul, q_mul, kq (all 32 lanes of a warp together: the sums go over lanes)
template <int QDT, int LPT>
__device__ __forceinline__ void meta_math(const KParams& p, const MetaRaw<QDT, LPT>& r, TileMeta& m) {
  constexpr int kGroups4 = MetaRaw<QDT, LPT>::kElems / 4;   // groups of four elements per lane
  gates_from(p, r.g, m.alpha, m.beta);
  float ks[kGroups4], qs[kGroups4], kq[kGroups4];
#pragma unroll
  for (int g = 0; g < kGroups4; ++g) {                 // four consecutive elements: one chain each
    float a[4], b[4];
    if (QDT == CARRY_F32) {
#pragma unroll
      for (int c = 0; c < 4; ++c) { a[c] = __uint_as_float(r.kw[4 * g + c]); b[c] = __uint_as_float(r.qw[4 * g + c]); }
    } else {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float2 ka = act_pair<QDT>(r.kw[2 * g + c]), qa = act_pair<QDT>(r.qw[2 * g + c]);
        a[2 * c] = ka.x; a[2 * c + 1] = ka.y; b[2 * c] = qa.x; b[2 * c + 1] = qa.y;
      }
    }
    float s0 = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) { s0 = fmaf(a[c], a[c], s0); s1 = fmaf(b[c], b[c], s1); s2 = fmaf(a[c], b[c], s2); }
    ks[g] = s0; qs[g] = s1; kq[g] = s2;
  }
#pragma unroll
  for (int stride = 1; stride < kGroups4; stride *= 2)   // balanced tree over this lane's groups, in index order
#pragma unroll
    for (int g = 0; g + stride < kGroups4; g += 2 * stride) { ks[g] += ks[g + stride]; qs[g] += qs[g + stride]; kq[g] += kq[g + stride]; }
  float ksum = ks[0], qsum = qs[0], kqsum = kq[0];
#pragma unroll
  for (int o = 1; o < LPT; o <<= 1) {                    // ... and on over the tile's lanes
    ksum += __shfl_xor_sync(0xffffffffu, ksum, o);
    qsum += __shfl_xor_sync(0xffffffffu, qsum, o);
    kqsum += __shfl_xor_sync(0xffffffffu, kqsum, o);
  }
  m.k_mul = 1.0f; m.q_mul = 1.0f;
  if (p.packed) {
    if (p.l2norm) {
      m.k_mul = __frcp_rn(sqrtf(ksum + 1e-6f));
      m.q_mul = __frcp_rn(sqrtf(qsum + 1e-6f));
    }
    m.q_mul *= p.qscale;
  }
  m.kq = kqsum * (m.k_mul * m.q_mul);
}
// A slot id beyond the pool is treated as padding (and reported by meta_put); the tile's addresses follow
// from the slot id that is left.  No side effects: this, too, can run ahead of the dependency wait.
template <int RES, int RSCALE, int QDT>
__device__ __forceinline__ bool meta_addresses(const KParams& p, TileMeta& m, int hv, int h, unsigned long long (&a)[8]) {
  const bool bad = p.packed && m.slot >= p.num_slots;
  if (bad) m.slot = 0;
  tile_addresses<RES, RSCALE, QDT>(p, m.n, hv, h, m.slot > 0 ? m.slot : 0, a);
  return bad;
}
// Lane 0 of a tile's lanes writes `dst`, lanes 0..3 a quarter of the tile's addresses each to `ddst` (which
// may be null); a bad slot id goes to the status word.
__device__ __forceinline__ void meta_put(const KParams& p, const TileMeta& m, const unsigned long long (&a)[8], bool bad,
                                         int sub, TileMeta* dst, TileDesc* ddst) {
  if (bad && sub == 0 && p.status) atomicOr(p.status, CARRY_GDN_STATUS_BAD_SLOT);
  if (sub == 0) *dst = m;
  if (ddst && sub < 4) {
    const unsigned long long lo = (sub == 0) ? a[0] : (sub == 1) ? a[2] : (sub == 2) ? a[4] : a[6];
    const unsigned long long hi = (sub == 0) ? a[1] : (sub == 1) ? a[3] : (sub == 2) ? a[5] : a[7];
    *reinterpret_cast<ulonglong2*>(&ddst->a[2 * sub]) = make_ulonglong2(lo, hi);
  }
}
template <int N> struct LanesPerTile { static constexpr int value = N; };
// The pieces in a row.  All 32 lanes of a warp must call this together; nothing is written when
// `store` is false.  (tok_*: element offsets of the token within its request, for callers that take several
// tokens per request.)
template <int RES, int RSCALE, int QDT, int LPT>
__device__ __noinline__ void tile_meta(const KParams& p, int tile, int sub, bool store, TileMeta* dst, TileDesc* ddst,
                                       long long tok_qkv = 0, long long tok_a = 0, long long tok_b = 0) {
  TileMeta m;
  int hv, h;
  split_tile(p, tile, m.n, hv, h);
  m.hv = hv;
  MetaRaw<QDT, LPT> r;
  meta_load<QDT, LPT>(p, m.n, hv, h, sub, tok_qkv, tok_a, tok_b, r);   // every load of this routine is in flight now
  m.slot = r.slot;
  meta_math<QDT, LPT>(p, r, m);
  unsigned long long a[8];
  const bool bad = meta_addresses<RES, RSCALE, QDT>(p, m, hv, h, a);
  if (store) meta_put(p, m, a, bad, sub, dst, ddst);
}

// Request one tile into the stage at `sb` (called by one thread): the stage barrier's single arrival
// announcing the bytes to come, then the seven bulk copies -- in that order: copies started before their
// bytes were announced cost 20 % of the kernel's time when measured.  `slot` <= 0 marks a padding request:
// nothing is copied.
template <int LAYOUT, int RES, int RSCALE, int QDT>
__device__ __forceinline__ void issue_copies(const KParams& p, uint8_t* sb, uint64_t* bar, const unsigned long long (&a)[8],
                                             int tile) {
  using L = StageLayout<RES, LAYOUT, QDT, RSCALE>;
  constexpr uint32_t rscale_bytes = L::kRScaleBytes;
  // launch-wide offsets from where results go to where the state is read (zero when in place)
  const long long d_codes = reinterpret_cast<const uint8_t*>(p.codes_in) - reinterpret_cast<const uint8_t*>(p.codes_out);
  const long long d_resid = reinterpret_cast<const uint8_t*>(p.resid_in) - reinterpret_cast<const uint8_t*>(p.resid_out);
  const long long d_sscale = reinterpret_cast<const uint8_t*>(p.sscale_in) - reinterpret_cast<const uint8_t*>(p.sscale_out);
  mbar_arrive_expect_tx(bar, kT * kT + L::kResidBytes + 512 + rscale_bytes + 3 * L::kVecBytes + test_extra_tx(tile));
  bulk_load(sb + L::kCodes, reinterpret_cast<const void*>(a[D_CODES] + d_codes), kT * kT, bar);
  bulk_load(sb + L::kResid, reinterpret_cast<const void*>(a[D_RESID] + d_resid), L::kResidBytes, bar);
  bulk_load(sb + L::kSScale, reinterpret_cast<const void*>(a[D_SSCALE] + d_sscale), 512, bar);
  if constexpr (rscale_bytes > 0) bulk_load(sb + L::kRScale, reinterpret_cast<const void*>(a[D_RSCALE_IN]), rscale_bytes, bar);
  bulk_load(sb + L::kQ, reinterpret_cast<const void*>(a[D_Q]), L::kVecBytes, bar);
  bulk_load(sb + L::kK, reinterpret_cast<const void*>(a[D_K]), L::kVecBytes, bar);
  bulk_load(sb + L::kV, reinterpret_cast<const void*>(a[D_V]), L::kVecBytes, bar);
}
// ... from the tile's facts (the CTA's first requests, and tiles beyond the cached ones)
template <int LAYOUT, int RES, int RSCALE, int QDT>
__device__ __noinline__ void issue_tile(const KParams& p, uint8_t* sb, uint64_t* bar, int n, int hv, int h, long long slot) {
  if (slot <= 0 || (p.packed && slot >= p.num_slots)) { mbar_arrive(bar); return; }
  unsigned long long a[8];
  tile_addresses<RES, RSCALE, QDT>(p, n, hv, h, slot, a);
  issue_copies<LAYOUT, RES, RSCALE, QDT>(p, sb, bar, a, n * p.HV + hv);
}
// ... from the addresses worked out when the CTA started
template <int LAYOUT, int RES, int RSCALE, int QDT>
__device__ __noinline__ void issue_cached(const KParams& p, uint8_t* sb, uint64_t* bar, const TileDesc* d, int slot,
                                          int tile) {
  if (slot <= 0) { mbar_arrive(bar); return; }
  const uint4 w0 = lds_v4(d), w1 = lds_v4(reinterpret_cast<const uint8_t*>(d) + 16);
  const uint4 w2 = lds_v4(reinterpret_cast<const uint8_t*>(d) + 32), w3 = lds_v4(reinterpret_cast<const uint8_t*>(d) + 48);
  auto u64 = [](uint32_t lo, uint32_t hi) { return ((unsigned long long)hi << 32) | lo; };
  const unsigned long long a[8] = {u64(w0.x, w0.y), u64(w0.z, w0.w), u64(w1.x, w1.y), u64(w1.z, w1.w),
                                   u64(w2.x, w2.y), u64(w2.z, w2.w), u64(w3.x, w3.y), u64(w3.z, w3.w)};
  issue_copies<LAYOUT, RES, RSCALE, QDT>(p, sb, bar, a, tile);
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <int LAYOUT, int RES, int RSCALE, int QDT>
__global__ void __launch_bounds__(kThreads * StageLayout<RES, LAYOUT, QDT, RSCALE>::kGroups, 1)
gdn_tile128_kernel(const __grid_constant__ KParams p) {
  using L = StageLayout<RES, LAYOUT, QDT, RSCALE>;
  constexpr int S = L::kStages;
  constexpr int G = L::kGroups;
  constexpr int kCache = kTileCache * G;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar[S];
  __shared__ int next_seq;                           // next tile of this CTA nobody has taken yet
  __shared__ int claimed[G][2];                      // the tile a group goes on with, by parity of its tile count
  __shared__ int first_cnt[G][2];                    // arrivals at the last meeting of a tile, by the same parity
  __shared__ int poison_flag;
  __shared__ int stage_tile[S];                      // number of the tile last requested into each stage
  __shared__ float head_red[G][2][kWarps];
  __shared__ TileMeta meta_cache[kCache + G * kWarps];   // this CTA's first tiles; one spare entry per warp
  __shared__ TileDesc desc_cache[kCache + G * kWarps];   // their addresses
  __shared__ __align__(16) float q_warp[(LAYOUT == LAYOUT_VK) ? G * kWarps * kT : 4];   // per warp: q, scaled, as pairs
  __shared__ __align__(16) float col_red_all[(LAYOUT == LAYOUT_KV) ? G * kWarps * kT * 4 : 4];
  static_assert(sizeof(full_bar) + sizeof(claimed) + sizeof(first_cnt) + sizeof(stage_tile) + sizeof(head_red) + sizeof(meta_cache) + sizeof(desc_cache) +
                        sizeof(q_warp) + sizeof(col_red_all) + 64 <= L::kStatic,
                "static shared memory exceeds what the stage ring was sized for");
  static_assert(S >= 2 * G, "every group needs a stage in use and one on the way");

  // warp: index within the whole CTA (per-warp scratch); gw, gtid: within the group (rows of the tile)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = (G == 1) ? 0 : (warp >> 3), gw = warp & 7, gtid = tid & (kThreads - 1);
  const int bar0 = 3 * grp;                          // this group's named barriers are bar0 + 1 .. bar0 + 3
  float* col_red = col_red_all + ((LAYOUT == LAYOUT_KV) ? grp * kWarps * kT * 4 : 0);
  const int total = p.B * p.HV;
  const int my_tiles = (total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  volatile int* poison = &poison_flag;

  // let the next kernel in the stream, if it asked for it, move in behind this one (see launch_variant)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // the CTA's bookkeeping is set up by its last thread (the last warp is the one least likely to have a tile
  // to prepare) and published by the meeting right before the dependency wait: nothing ahead of that
  // meeting touches it, so the set-up's loads are on their way first
  if (tid == G * kThreads - 1) {
    poison_flag = 0;
    next_seq = G;                                    // tiles 0 .. G-1 are the groups' first ones
    for (int s = 0; s < S; ++s) { mbar_init(&full_bar[s], 1); stage_tile[s] = -1; }
    for (int g = 0; g < G; ++g) first_cnt[g][0] = first_cnt[g][1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Tiles of this CTA are numbered 0, 1, 2, ... (tile = blockIdx.x + number * gridDim.x) and sit in stage
  // number % S.  Set-up of the first ones (up to the cache's size), by all threads at 32, 8 or 4 lanes per
  // tile -- as many as the tile count leaves room for in one pass -- in two halves around the dependency
  // wait:
  //   before it, while the kernel ahead in the stream finishes: load the tiles' inputs past the L1, work
  //     out slot id, gates and norms from whatever they hold, keep both in registers; hint the L2 at the
  //     state of the groups' first tiles and at the v rows.  Nothing here writes memory or hands a value on.
  //   after it: the same loads again, now ordered after every write of that kernel.  Equal words mean the
  //     figures worked out beforehand are the ones this launch must use: the groups' first tiles are
  //     requested at once, from the addresses already in registers (the rest of the ring only after all
  //     threads have met, so that the first tiles are not queued behind it), and the figures go to the
  //     cache.  A warp that sees a difference runs the whole routine again.
  // Right after a kernel that left tens of MB of results in the L2 a first touch of memory takes some 2 us
  // and the routine's arithmetic, fetched cold, another microsecond: this way both pass while the CTA would
  // otherwise sit in the wait, and what is left behind it is one trip to the L2.
  const int cached = my_tiles < kCache ? my_tiles : kCache;
  auto setup = [&](auto lanes_per_tile) {
    constexpr int LPT = decltype(lanes_per_tile)::value;
    constexpr int qes = (QDT == CARRY_F32) ? 4 : 2;
    const int num = (LPT == 32) ? warp : (LPT == 8) ? (tid >> 3) : (tid >> 2);   // the tile these lanes prepare
    const int sub = (LPT == 32) ? lane : (LPT == 8) ? (tid & 7) : (tid & 3);
    const bool valid = num < cached;
    const bool busy = warp * (32 / LPT) < cached;        // warps without a tile to prepare stay out of the way
    const int tile = (int)blockIdx.x + (valid ? num : 0) * (int)gridDim.x;
    const int entry = valid ? num : 0;
    TileMeta m;
    MetaRaw<QDT, LPT> before;
    unsigned long long a[8];
    bool bad = false;
    int hv = 0, h = 0;
    if (busy) {
      split_tile(p, tile, m.n, hv, h);
      m.hv = hv;
      meta_load<QDT, LPT>(p, m.n, hv, h, sub, 0, 0, 0, before);
      m.slot = before.slot;
      bad = meta_addresses<RES, RSCALE, QDT>(p, m, hv, h, a);
      if (sub == 0 && valid && m.slot > 0) {
        l2_prefetch_line(reinterpret_cast<const void*>(a[D_V]));
        l2_prefetch_line(reinterpret_cast<const void*>(a[D_V] + kT * qes - 16));
        if (num < 2 * G) {                               // the state of the first two tiles of every group
          const long long d_codes = reinterpret_cast<const uint8_t*>(p.codes_in) - reinterpret_cast<const uint8_t*>(p.codes_out);
          const long long d_resid = reinterpret_cast<const uint8_t*>(p.resid_in) - reinterpret_cast<const uint8_t*>(p.resid_out);
          const long long d_sscale = reinterpret_cast<const uint8_t*>(p.sscale_in) - reinterpret_cast<const uint8_t*>(p.sscale_out);
          l2_prefetch_bulk(reinterpret_cast<const void*>(a[D_CODES] + d_codes), kT * kT);
          l2_prefetch_bulk(reinterpret_cast<const void*>(a[D_RESID] + d_resid), L::kResidBytes);
          l2_prefetch_bulk(reinterpret_cast<const void*>(a[D_SSCALE] + d_sscale), 512);
        }
      }
      meta_math<QDT, LPT>(p, before, m);
    }
    // nothing before this line hands on what it read from global memory, or writes it; everything after it
    // sees the results of the kernels that precede this one in the stream
    __syncthreads();
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (busy) {
      const bool same = meta_unchanged<QDT, LPT>(p, m.n, hv, h, sub, before);
      test_note_changed(p.status, same);
      const bool first = valid && sub == 0 && num < G;   // the lane that requests a group's first tile
      if (__all_sync(0xffffffffu, same && !test_inputs_changed(tile))) {
        if (first) {
          *reinterpret_cast<volatile int*>(&stage_tile[num]) = num;
          if (m.slot <= 0) mbar_arrive(&full_bar[num]);
          else issue_copies<LAYOUT, RES, RSCALE, QDT>(p, smem + (size_t)num * L::kBytes, &full_bar[num], a, tile);
        }
        if (valid) meta_put(p, m, a, bad, sub, &meta_cache[entry], &desc_cache[entry]);
      } else {
        tile_meta<RES, RSCALE, QDT, LPT>(p, tile, sub, valid, &meta_cache[entry], &desc_cache[entry]);
        __syncwarp();
        if (first) {
          *reinterpret_cast<volatile int*>(&stage_tile[num]) = num;
          issue_cached<LAYOUT, RES, RSCALE, QDT>(p, smem + (size_t)num * L::kBytes, &full_bar[num], &desc_cache[num],
                                                 meta_cache[num].slot, tile);
        }
      }
    }
  };
  static_assert(kThreads / 4 == kTileCache, "at four lanes per tile one pass covers the whole cache");
  if (cached <= G * kWarps) setup(LanesPerTile<32>{});
  else if (cached <= G * kWarps * 4) setup(LanesPerTile<8>{});
  else setup(LanesPerTile<4>{});
  __syncthreads();
  static_assert(S <= G * kWarps && S <= kTileCache, "one warp per stage issues the first requests, from the cache");

  // reciprocals rounded to nearest (div_qmax relies on it): a constant, and one that the host worked out --
  // the correctly rounded device routine is a subroutine call that, fetched cold right after the wait, was
  // seen to take up to a microsecond
  constexpr float rqmax = (RES == CARRY_RES_INT4) ? 7.0f : 127.0f;
  constexpr float rrqmax = 1.0f / rqmax;
  const float rqmax_state = p.inv_qmax;
  auto load_tile = [&](int num) {                   // one thread requests tile `num`
    uint8_t* dst_stage = smem + (size_t)(num % S) * L::kBytes;
    *reinterpret_cast<volatile int*>(&stage_tile[num % S]) = num;
    if (num < kCache) {
      issue_cached<LAYOUT, RES, RSCALE, QDT>(p, dst_stage, &full_bar[num % S], &desc_cache[num], meta_cache[num].slot,
                                             (int)blockIdx.x + num * (int)gridDim.x);
    } else {
      const int tile = (int)blockIdx.x + num * (int)gridDim.x;
      int tn, thv, th;
      split_tile(p, tile, tn, thv, th);
      const int tslot = p.packed ? p.slot_idx[(long long)tn * p.stride_idx] : 1;
      issue_tile<LAYOUT, RES, RSCALE, QDT>(p, dst_stage, &full_bar[num % S], tn, thv, th, tslot);
    }
  };
  if (lane == 0 && warp >= G && warp < S && warp < my_tiles) load_tile(warp);
  __syncwarp();
  // A group takes its tiles from the CTA's list as it goes (the two groups of an SM do not run at the
  // same pace).  Right before the last meeting of a tile, lane 0 of every warp calls claim_next(): the first
  // to arrive takes the next number for the whole group.  Right after that meeting every read of the tile's
  // stage is over, and that same warp -- the one with the most time in hand -- requests the tile that will
  // use the stage next while the others go on: 1 % faster than the warps taking turns.  (Measured
  // alternatives, both slower: the first warp to arrive requesting, before the meeting, the tile for the
  // stage of the group's previous tile; all eight warps requesting a part each.)
  bool refill_mine = false;                          // this warp was the first at the tile's last meeting
  auto claim_next = [&](int cnt) {
    refill_mine = atomicAdd(&first_cnt[grp][cnt & 1], 1) == 0;
    if (refill_mine) {
      first_cnt[grp][(cnt + 1) & 1] = 0;
      claimed[grp][cnt & 1] = atomicAdd(&next_seq, 1);
    }
  };
  auto refill_stage = [&](int num) {
    if (refill_mine && lane == 0 && num + S < my_tiles && !*poison) load_tile(num + S);
  };

  int it = grp;                                      // number of the tile in hand
  for (int cnt = 0; it < my_tiles; ++cnt) {
    const int s = it % S;
    const uint32_t parity = (uint32_t)(it / S) & 1u;
    uint8_t* sb = smem + (size_t)s * L::kBytes;
    const int entry = it < kCache ? it : kCache + warp;
    const TileMeta* tm = &meta_cache[entry];
    if (it >= kCache) {
      tile_meta<RES, RSCALE, QDT, 32>(p, (int)blockIdx.x + it * (int)gridDim.x, lane, true, &meta_cache[entry],
                                      &desc_cache[entry]);
      __syncwarp();
    }
    const uint4 tm0 = lds_v4(tm);
    const int n = (int)tm0.x, hv = (int)tm0.y;

    const bool healthy = tile_wait(&full_bar[s], parity, &stage_tile[s], it, poison, p.status);
    const int slot = (int)tm0.z;
    const int out_row = n * p.HV + hv;                // outputs of this tile start at element out_row * 128
    const bool live = slot > 0 && healthy;
    // where results go: read from the tile's cached addresses right before each use, not held in registers
    auto dst_of = [&](int which) -> unsigned long long {
      unsigned long long v;
      asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(smem_u32(&desc_cache[entry].a[which])));
      return v;
    };

    if (!live) {
      if (slot <= 0 && gtid < kT) store_from_float(p.out, (long long)out_row * kT + gtid, p.o_dtype, 0.f);
      if (LAYOUT == LAYOUT_KV) { warps_meet(bar0 + 1); warps_meet(bar0 + 2); }
      if (lane == 0) claim_next(cnt);
      warps_meet(bar0 + 3);
      refill_stage(it);
    } else {
      const uint4 tm1 = lds_v4(reinterpret_cast<const uint8_t*>(tm) + 16);
      const float alpha = __uint_as_float(tm0.w), beta = __uint_as_float(tm1.x), k_mul = __uint_as_float(tm1.y),
                  q_mul = __uint_as_float(tm1.z), kq = __uint_as_float(tm1.w);
      const float* sscale = reinterpret_cast<const float*>(sb + L::kSScale);
      const float* rscale = reinterpret_cast<const float*>(sb + L::kRScale);
      const float es_head = (RSCALE == CARRY_SCALE_PER_HEAD) ? rscale[hv & 3] : 0.f;
      const float2 alpha2 = splat(alpha);
      const float2 magic2 = splat(kMagicRound), nmagic2 = splat(-kMagicRound);

      if constexpr (LAYOUT == LAYOUT_VK) {
#define CARRY_SLOT_VEC_Q (sb + L::kQ)
#define CARRY_SLOT_VEC_K (sb + L::kK)
#define CARRY_SLOT_VEC_V (sb + L::kV)
#define CARRY_SLOT_OUT(idx, value) store_from_float(p.out, (long long)out_row * kT + (idx), p.o_dtype, (value))
#define CARRY_SLOT_PUT_SSCALE(r0_, v4_) stg_v4(dst_of(D_SSCALE) + (r0_) * 4, (v4_))
#define CARRY_SLOT_PUT_CODES(r0_, c0_, cw_)                                                   \
  {                                                                                           \
    const unsigned long long base = dst_of(D_CODES) + (r0_) * kT + (c0_);                     \
    stg_v4_at<0 * kT>(base, make_uint4(cw_[0][0], cw_[0][1], cw_[0][2], cw_[0][3]));          \
    stg_v4_at<1 * kT>(base, make_uint4(cw_[1][0], cw_[1][1], cw_[1][2], cw_[1][3]));          \
    stg_v4_at<2 * kT>(base, make_uint4(cw_[2][0], cw_[2][1], cw_[2][2], cw_[2][3]));          \
    stg_v4_at<3 * kT>(base, make_uint4(cw_[3][0], cw_[3][1], cw_[3][2], cw_[3][3]));          \
  }
#define CARRY_SLOT_HEAD_RED head_red[grp][cnt & 1]
#define CARRY_SLOT_MEET(statement)                \
  if (lane == 0) { statement; claim_next(cnt); }  \
  warps_meet(bar0 + 3);                           \
  refill_stage(it)
#define CARRY_SLOT_RESID_BEGIN() const unsigned long long dst_resid = dst_of(D_RESID)
#define CARRY_SLOT_PUT_RESID4(i_, r0_, c0_, w_)                                    \
  {                                                                                \
    const unsigned long long base = dst_resid + (r0_) * (kT / 2) + (c0_) / 2;      \
    if (i_ == 0) stg_v2_at<0 * (kT / 2)>(base, w_);                                \
    if (i_ == 1) stg_v2_at<1 * (kT / 2)>(base, w_);                                \
    if (i_ == 2) stg_v2_at<2 * (kT / 2)>(base, w_);                                \
    if (i_ == 3) stg_v2_at<3 * (kT / 2)>(base, w_);                                \
  }
#define CARRY_SLOT_PUT_RESID8(i_, r0_, c0_, w_)                                    \
  {                                                                                \
    const unsigned long long base = dst_resid + (r0_) * kT + (c0_);                \
    const uint4 pw = w_;                                                           \
    if (i_ == 0) stg_v4_at<0 * kT>(base, pw);                                      \
    if (i_ == 1) stg_v4_at<1 * kT>(base, pw);                                      \
    if (i_ == 2) stg_v4_at<2 * kT>(base, pw);                                      \
    if (i_ == 3) stg_v4_at<3 * kT>(base, pw);                                      \
  }
#define CARRY_SLOT_PUT_RSCALE_V(r0_, v4_) stg_v4(dst_of(D_RSCALE) + (r0_) * 4, (v4_))
#define CARRY_SLOT_PUT_RSCALE_HEAD(bits_) stg_b32(dst_of(D_RSCALE), (bits_))
#include "carry_gdn_slot_tile.inc"
#undef CARRY_SLOT_VEC_Q
#undef CARRY_SLOT_VEC_K
#undef CARRY_SLOT_VEC_V
#undef CARRY_SLOT_OUT
#undef CARRY_SLOT_PUT_SSCALE
#undef CARRY_SLOT_PUT_CODES
#undef CARRY_SLOT_HEAD_RED
#undef CARRY_SLOT_MEET
#undef CARRY_SLOT_RESID_BEGIN
#undef CARRY_SLOT_PUT_RESID4
#undef CARRY_SLOT_PUT_RESID8
#undef CARRY_SLOT_PUT_RSCALE_V
#undef CARRY_SLOT_PUT_RSCALE_HEAD
      } else {
        // ---------------- statequant layout [K][V]: lane = 4 columns x 16 rows ----
        // columns {c0, c0+1} are held as pair A, {c0+2, c0+3} as pair B
        const int r0 = 16 * gw, c0 = 4 * lane;
        float* red_dot = col_red;                       // [warp][col][2]
        float* red_max = col_red + kWarps * kT * 2;     // [warp][col]
        float* red_emax = red_max + kWarps * kT;        // [warp][col]
        // k and q of this warp's 16 rows are the same in every lane; they are read from the stage where they
        // are used (a broadcast load) instead of being held in 32 registers.  k_mul and q_mul are 1 in this
        // layout's callers but are applied all the same.
        auto k_of = [&](int i) { return act<QDT>(sb + L::kK, r0 + i) * k_mul; };
        auto q_of = [&](int i) { return act<QDT>(sb + L::kQ, r0 + i) * q_mul; };
        float scol[4];
        {
          const float4 s4 = *reinterpret_cast<const float4*>(sscale + c0);
          scol[0] = s4.x; scol[1] = s4.y; scol[2] = s4.z; scol[3] = s4.w;
        }
        const float2 sA = make_float2(scol[0], scol[1]), sB = make_float2(scol[2], scol[3]);
        float2 hA[16], hB[16];
        float2 dkA = make_float2(0.f, 0.f), dkB = dkA, dqA = dkA, dqB = dkA;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(sb + L::kCodes + (r0 + i) * kT + c0) ^ 0x80808080u;
          const float2 a = mul2(mul2(s8x2_to_float<0, 1>(w), sA), alpha2);
          const float2 b = mul2(mul2(s8x2_to_float<2, 3>(w), sB), alpha2);
          hA[i] = a; hB[i] = b;
          const float2 kr = splat(k_of(i)), qr = splat(q_of(i));
          dkA = fma2(a, kr, dkA); dkB = fma2(b, kr, dkB);
          dqA = fma2(a, qr, dqA); dqB = fma2(b, qr, dqB);
        }
        // finish the column sums across the 8 warps
        float dk[4], dq[4];
        {
          float4* dst = reinterpret_cast<float4*>(red_dot + ((size_t)gw * kT + c0) * 2);
          dst[0] = make_float4(dkA.x, dqA.x, dkA.y, dqA.y);
          dst[1] = make_float4(dkB.x, dqB.x, dkB.y, dqB.y);
          warps_meet(bar0 + 1);
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
        float dv[4], oval[4], es_col[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          dv[b] = __fmul_rn(beta, __fadd_rn(act<QDT>(sb + L::kV, c0 + b), -dk[b]));
          oval[b] = fmaf(dv[b], kq, dq[b]);
          es_col[b] = L::kFloatResid ? 0.f : (RSCALE == CARRY_SCALE_PER_V) ? rscale[c0 + b] : es_head;
        }
        const float2 dvA = make_float2(dv[0], dv[1]), dvB = make_float2(dv[2], dv[3]);
        float amax[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float2 eA, eB;
          if constexpr (RES == CARRY_RES_FP32) {
            const float4 e4 = *reinterpret_cast<const float4*>(sb + L::kResid + ((r0 + i) * kT + c0) * 4);
            eA = make_float2(e4.x, e4.y); eB = make_float2(e4.z, e4.w);
          } else if constexpr (RES == CARRY_RES_FP16) {
            const uint2 e2 = *reinterpret_cast<const uint2*>(sb + L::kResid + ((r0 + i) * kT + c0) * 2);
            eA = __half22float2(*reinterpret_cast<const __half2*>(&e2.x));
            eB = __half22float2(*reinterpret_cast<const __half2*>(&e2.y));
          } else if constexpr (RES == CARRY_RES_FP8) {
            e5m2x4_to_float(*reinterpret_cast<const uint32_t*>(sb + L::kResid + (r0 + i) * kT + c0), eA, eB);
          } else if constexpr (RES == CARRY_RES_INT4) {
            const uint32_t w =
                (uint32_t)(*reinterpret_cast<const uint16_t*>(sb + L::kResid + (r0 + i) * (kT / 2) + c0 / 2)) ^ 0x8888u;
            float2 lo, hi;                              // lo = cols {c0, c0+2}, hi = 16 * cols {c0+1, c0+3}
            s4x4_to_float<0, 1>(w, lo, hi);
            eA = mul2(make_float2(lo.x, hi.x), make_float2(es_col[0], es_col[1] * 0.0625f));
            eB = mul2(make_float2(lo.y, hi.y), make_float2(es_col[2], es_col[3] * 0.0625f));
          } else {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(sb + L::kResid + (r0 + i) * kT + c0) ^ 0x80808080u;
            eA = mul2(s8x2_to_float<0, 1>(w), make_float2(es_col[0], es_col[1]));
            eB = mul2(s8x2_to_float<2, 3>(w), make_float2(es_col[2], es_col[3]));
          }
          const float2 kr = splat(k_of(i));
          const float2 tA = add2(fma2(kr, dvA, hA[i]), eA);
          const float2 tB = add2(fma2(kr, dvB, hB[i]), eB);
          hA[i] = tA; hB[i] = tB;
          amax[0] = fmaxf(amax[0], fabsf(tA.x)); amax[1] = fmaxf(amax[1], fabsf(tA.y));
          amax[2] = fmaxf(amax[2], fabsf(tB.x)); amax[3] = fmaxf(amax[3], fabsf(tB.y));
        }
        if (gw == 0) {
#pragma unroll
          for (int b = 0; b < 4; ++b) store_from_float(p.out, (long long)out_row * kT + c0 + b, p.o_dtype, oval[b]);
        }
        *reinterpret_cast<float4*>(red_max + (size_t)gw * kT + c0) = make_float4(amax[0], amax[1], amax[2], amax[3]);
        warps_meet(bar0 + 2);
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          const float4 x = *reinterpret_cast<const float4*>(red_max + (size_t)w * kT + c0);
          amax[0] = fmaxf(amax[0], x.x); amax[1] = fmaxf(amax[1], x.y);
          amax[2] = fmaxf(amax[2], x.z); amax[3] = fmaxf(amax[3], x.w);
        }
        float snew[4], thr[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) { snew[b] = scale_fast(amax[b], p.qmax, rqmax_state, p.eps_mode); thr[b] = snew[b] * kTieGuard; }
        const float2 invA = make_float2(rcp_refined(snew[0]), rcp_refined(snew[1]));
        const float2 invB = make_float2(rcp_refined(snew[2]), rcp_refined(snew[3]));
        const float2 nsA = make_float2(-snew[0], -snew[1]), nsB = make_float2(-snew[2], -snew[3]);
        float eamax[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t cw[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 yA = fma2(hA[i], invA, magic2), yB = fma2(hB[i], invB, magic2);
          hA[i] = fma2(add2(yA, nmagic2), nsA, hA[i]);
          hB[i] = fma2(add2(yB, nmagic2), nsB, hB[i]);
          cw[i] = pack4(__float_as_uint(yA.x), __float_as_uint(yA.y), __float_as_uint(yB.x), __float_as_uint(yB.y));
          eamax[0] = fmaxf(eamax[0], fabsf(hA[i].x)); eamax[1] = fmaxf(eamax[1], fabsf(hA[i].y));
          eamax[2] = fmaxf(eamax[2], fabsf(hB[i].x)); eamax[3] = fmaxf(eamax[3], fabsf(hB[i].y));
        }
        if (fmaxf(fmaxf(eamax[0] - thr[0], eamax[1] - thr[1]), fmaxf(eamax[2] - thr[2], eamax[3] - thr[3])) > 0.f) {
          eamax[0] = eamax[1] = eamax[2] = eamax[3] = 0.f;      // rare: a quotient within the tie guard
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float2 yA = add2(s8x2_to_float<0, 1>(cw[i] ^ 0x80808080u), magic2);
            float2 yB = add2(s8x2_to_float<2, 3>(cw[i] ^ 0x80808080u), magic2);
            redecide_rec(hA[i].x, yA.x, snew[0], thr[0]); redecide_rec(hA[i].y, yA.y, snew[1], thr[1]);
            redecide_rec(hB[i].x, yB.x, snew[2], thr[2]); redecide_rec(hB[i].y, yB.y, snew[3], thr[3]);
            cw[i] = pack4(__float_as_uint(yA.x), __float_as_uint(yA.y), __float_as_uint(yB.x), __float_as_uint(yB.y));
            eamax[0] = fmaxf(eamax[0], fabsf(hA[i].x)); eamax[1] = fmaxf(eamax[1], fabsf(hA[i].y));
            eamax[2] = fmaxf(eamax[2], fabsf(hB[i].x)); eamax[3] = fmaxf(eamax[3], fabsf(hB[i].y));
          }
        }
        {
          const unsigned long long dst_codes = dst_of(D_CODES);
#pragma unroll
          for (int i = 0; i < 16; ++i) stg_b32(dst_codes + (r0 + i) * kT + c0, cw[i]);
        }
        if constexpr (L::kFloatResid) {
          // the new residual is stored as it is, in its format; the meeting only hands the stage on
          if (lane == 0) claim_next(cnt);
          warps_meet(bar0 + 3);
          refill_stage(it);
          const unsigned long long dst_resid = dst_of(D_RESID);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if constexpr (RES == CARRY_RES_FP32) {
              stg_v4(dst_resid + ((r0 + i) * kT + c0) * 4,
                     make_uint4(__float_as_uint(hA[i].x), __float_as_uint(hA[i].y), __float_as_uint(hB[i].x),
                                __float_as_uint(hB[i].y)));
            } else if constexpr (RES == CARRY_RES_FP16) {
              const __half2 a2 = __floats2half2_rn(hA[i].x, hA[i].y), b2 = __floats2half2_rn(hB[i].x, hB[i].y);
              stg_v2_at<0>(dst_resid + ((r0 + i) * kT + c0) * 2,
                           make_uint2(*reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&b2)));
            } else {
              stg_b32(dst_resid + (r0 + i) * kT + c0, float4_to_e5m2x4(hA[i], hB[i]));
            }
          }
          if ((lane >> 2) == gw)
            stg_v4(dst_of(D_SSCALE) + c0 * 4, make_uint4(__float_as_uint(snew[0]), __float_as_uint(snew[1]),
                                                         __float_as_uint(snew[2]), __float_as_uint(snew[3])));
        } else {
        float esn[4];
        if constexpr (RSCALE == CARRY_SCALE_PER_V) {
          *reinterpret_cast<float4*>(red_emax + (size_t)gw * kT + c0) =
              make_float4(eamax[0], eamax[1], eamax[2], eamax[3]);
          if (lane == 0) claim_next(cnt);
          warps_meet(bar0 + 3);
          refill_stage(it);
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const float4 x = *reinterpret_cast<const float4*>(red_emax + (size_t)w * kT + c0);
            eamax[0] = fmaxf(eamax[0], x.x); eamax[1] = fmaxf(eamax[1], x.y);
            eamax[2] = fmaxf(eamax[2], x.z); eamax[3] = fmaxf(eamax[3], x.w);
          }
#pragma unroll
          for (int b = 0; b < 4; ++b) esn[b] = scale_fast(eamax[b], rqmax, rrqmax, p.eps_mode);
        } else {
          float m = warp_max_nonneg(fmaxf(fmaxf(eamax[0], eamax[1]), fmaxf(eamax[2], eamax[3])));
          if (lane == 0) { head_red[grp][cnt & 1][gw] = m; claim_next(cnt); }
          warps_meet(bar0 + 3);
          refill_stage(it);
          m = head_red[grp][cnt & 1][0];
#pragma unroll
          for (int w = 1; w < kWarps; ++w) m = fmaxf(m, head_red[grp][cnt & 1][w]);
          esn[0] = esn[1] = esn[2] = esn[3] = scale_fast(m, rqmax, rrqmax, p.eps_mode);
        }
        const float2 ieA = make_float2(rcp_refined(esn[0]), rcp_refined(esn[1]));
        const float2 ieB = make_float2(rcp_refined(esn[2]), rcp_refined(esn[3]));
        const unsigned long long dst_resid = dst_of(D_RESID);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 rA = fma2(hA[i], ieA, magic2), rB = fma2(hB[i], ieB, magic2);
          const uint32_t y0 = __float_as_uint(rA.x), y1 = __float_as_uint(rA.y);
          const uint32_t y2 = __float_as_uint(rB.x), y3 = __float_as_uint(rB.y);
          if constexpr (RES == CARRY_RES_INT4) {
            const uint32_t v16 = (y0 & 0xFu) | ((y1 & 0xFu) << 4) | ((y2 & 0xFu) << 8) | ((y3 & 0xFu) << 12);
            stg_b16(dst_resid + (r0 + i) * (kT / 2) + c0 / 2, v16);
          } else {
            stg_b32(dst_resid + (r0 + i) * kT + c0, pack4(y0, y1, y2, y3));
          }
        }
        // scales: every warp holds all 128 of them; warp w publishes its 16-column share
        // (columns 16w..16w+15 are held by lanes 4w..4w+3)
        if ((lane >> 2) == gw) {
          stg_v4(dst_of(D_SSCALE) + c0 * 4, make_uint4(__float_as_uint(snew[0]), __float_as_uint(snew[1]),
                                                       __float_as_uint(snew[2]), __float_as_uint(snew[3])));
          if (RSCALE == CARRY_SCALE_PER_V)
            stg_v4(dst_of(D_RSCALE) + c0 * 4, make_uint4(__float_as_uint(esn[0]), __float_as_uint(esn[1]),
                                                   __float_as_uint(esn[2]), __float_as_uint(esn[3])));
        }
        if (RSCALE == CARRY_SCALE_PER_HEAD && gtid == 0) stg_b32(dst_of(D_RSCALE), __float_as_uint(esn[0]));
        }
      }
    }
    it = *reinterpret_cast<volatile int*>(&claimed[grp][cnt & 1]);   // written before this tile's last meeting
  }
  __syncthreads();
  // A CTA whose wait ran out has stopped requesting tiles, but copies it requested earlier may still be on
  // their way into its shared memory: give them a bounded while to land before the CTA leaves the SM.
  if (*poison) {
#pragma unroll 1
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

template <int LAYOUT, int RES, int RSCALE, int QDT>
int launch_variant(const KParams& p, cudaStream_t stream, int sms) {
  using L = StageLayout<RES, LAYOUT, QDT, RSCALE>;
  auto kern = gdn_tile128_kernel<LAYOUT, RES, RSCALE, QDT>;
  const size_t smem = (size_t)L::kBytes * L::kStages;
  static thread_local bool configured[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 64) return CARRY_GDN_ERR_NO_DEVICE;
  if (!configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
      cudaGetLastError();
      return CARRY_GDN_ERR_NO_DEVICE;
    }
    configured[dev] = true;
  }
  const long long tiles = (long long)p.B * p.HV;
  const long long per_cta = L::kGroups;               // a CTA works on that many tiles at a time
  const long long want = (tiles + per_cta - 1) / per_cta;
  const int grid = (int)(want < sms ? want : sms);
  // Programmatic dependent launch: when the kernel before this one in the stream lets its dependents go
  // early (this kernel does, at its top), the CTAs of this launch may take over SMs as that kernel's CTAs
  // leave them and set up their barriers; they touch global memory only after griddepcontrol.wait, i.e.
  // after the earlier kernel has completed and its writes are visible.  After any other kernel the
  // attribute changes nothing.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)(kThreads * L::kGroups));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, kern, p);
  if (err != cudaSuccess) cudaGetLastError();
  return err == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
}

template <int LAYOUT, int RES, int RSCALE>
int launch_dtype(const KParams& p, cudaStream_t stream, int sms) {
  if (p.qkv_dtype == CARRY_F32) return launch_variant<LAYOUT, RES, RSCALE, CARRY_F32>(p, stream, sms);
  if (p.qkv_dtype == CARRY_BF16) return launch_variant<LAYOUT, RES, RSCALE, CARRY_BF16>(p, stream, sms);
  return launch_variant<LAYOUT, RES, RSCALE, CARRY_F16>(p, stream, sms);
}

// all variants of one memory layout
template <int LAYOUT>
int launch_layout(const KParams& p, cudaStream_t stream, int sms) {
  if constexpr (LAYOUT == LAYOUT_KV) {     // the float residual formats exist on the statequant surfaces only
    if (p.res_fmt == CARRY_RES_FP32) return launch_dtype<LAYOUT, CARRY_RES_FP32, CARRY_SCALE_PER_V>(p, stream, sms);
    if (p.res_fmt == CARRY_RES_FP16) return launch_dtype<LAYOUT, CARRY_RES_FP16, CARRY_SCALE_PER_V>(p, stream, sms);
    if (p.res_fmt == CARRY_RES_FP8) return launch_dtype<LAYOUT, CARRY_RES_FP8, CARRY_SCALE_PER_V>(p, stream, sms);
  }
  const bool i4 = p.res_fmt == CARRY_RES_INT4, pv = p.rscale_mode == CARRY_SCALE_PER_V;
  if (i4) return pv ? launch_dtype<LAYOUT, CARRY_RES_INT4, CARRY_SCALE_PER_V>(p, stream, sms)
                    : launch_dtype<LAYOUT, CARRY_RES_INT4, CARRY_SCALE_PER_HEAD>(p, stream, sms);
  return pv ? launch_dtype<LAYOUT, CARRY_RES_INT8, CARRY_SCALE_PER_V>(p, stream, sms)
            : launch_dtype<LAYOUT, CARRY_RES_INT8, CARRY_SCALE_PER_HEAD>(p, stream, sms);
}

}  // namespace
}  // namespace carry
