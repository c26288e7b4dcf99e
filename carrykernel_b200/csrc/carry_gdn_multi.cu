// Multi-token variant of the slot-indexed decode step: T consecutive tokens of
// every request in one launch.  A (request, head) tile is fetched from the pool
// once, stays in shared memory while its T tokens are applied one after the
// other -- each token is the full step, requantisation and error feedback
// included, exactly as T single-token launches would do it -- and goes back to
// the pool once.  State traffic per token is 1/T of the single-token kernel's.
//
// One CTA (8 warps) per tile, two CTAs per SM.  The per-token arithmetic is the
// slot-layout tile body of the streaming kernel (carry_gdn_slot_tile.inc),
// with its stores pointed at the staged tile instead of global memory; a warp
// only ever reads and writes its own 16 rows of the tile, so tokens need no
// ordering between warps beyond the body's own meeting and one block barrier per
// token (for the per-head residual scale).  Activation vectors, gates and norms
// of up to 8 tokens are fetched together, one trip to global memory per chunk of
// tokens instead of one per token.
#include "carry_gdn_tile128.cuh"

namespace carry {

int launch_multi(const KParams& p, int T, long long stride_mixed_t, long long stride_a_t, long long stride_b_t,
                 cudaStream_t stream);

namespace {

struct MultiExtra {
  int T;
  long long stride_mixed_t, stride_a_t, stride_b_t;   // elements from one token of a request to the next
};

template <int RES, int RSCALE, int QDT>
__global__ void __launch_bounds__(kThreads, 2) gdn_multi_kernel(const __grid_constant__ KParams p,
                                                               const __grid_constant__ MultiExtra x) {
  using L = StageLayout<RES, LAYOUT_VK, QDT, RSCALE>;
  constexpr int qes = (QDT == CARRY_F32) ? 4 : 2;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t full_bar;
  __shared__ int poison_flag;
  __shared__ float head_red[2][kWarps];
  constexpr int kChunk = 8;                           // tokens whose activations and facts are fetched together
  __shared__ TileMeta meta_t[kChunk];
  __shared__ __align__(16) uint8_t vec_t[kChunk][3 * L::kVecBytes];   // raw q | k | v per token
  __shared__ __align__(16) float q_warp[kWarps * kT];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gw = warp, gtid = tid;
  uint8_t* sb = smem;
  volatile int* poison = &poison_flag;
  const int tile = (int)blockIdx.x;
  int n, hv, h;
  split_tile(p, tile, n, hv, h);
  long long slot = p.slot_idx[(long long)n * p.stride_idx];
  if (slot >= p.num_slots) {
    if (tid == 0 && p.status) atomicOr(p.status, CARRY_GDN_STATUS_BAD_SLOT);
    slot = 0;
  }
  const long long out_tok0 = ((long long)n * x.T * p.HV + hv) * kT;      // out is [B, T, HV, V]
  const long long out_tok_stride = (long long)p.HV * kT;
  if (slot <= 0) {                                   // padding request: zeros for every token, pool untouched
    for (int i = tid; i < x.T * kT; i += kThreads)
      store_from_float(p.out, out_tok0 + (long long)(i / kT) * out_tok_stride + (i % kT), p.o_dtype, 0.f);
    return;
  }

  __shared__ unsigned long long addr[8];            // where the tile and its activations live (see TileDesc)
  if (tid == 0) {
    unsigned long long a8[8];
    tile_addresses<RES, RSCALE, QDT>(p, n, hv, h, slot, a8);
#pragma unroll
    for (int i = 0; i < 8; ++i) addr[i] = a8[i];
    poison_flag = 0;
    mbar_init(&full_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // the state of the tile: codes, residual, state scales, residual scale(s)
    mbar_arrive_expect_tx(&full_bar, kT * kT + L::kResidBytes + 512 + L::kRScaleBytes + test_extra_tx(tile));
    bulk_load(sb + L::kCodes, reinterpret_cast<const void*>(a8[D_CODES]), kT * kT, &full_bar);
    bulk_load(sb + L::kResid, reinterpret_cast<const void*>(a8[D_RESID]), L::kResidBytes, &full_bar);
    bulk_load(sb + L::kSScale, reinterpret_cast<const void*>(a8[D_SSCALE]), 512, &full_bar);
    bulk_load(sb + L::kRScale, reinterpret_cast<const void*>(a8[D_RSCALE_IN]), L::kRScaleBytes, &full_bar);
  }
  constexpr float rqmax = (RES == CARRY_RES_INT4) ? 7.0f : 127.0f;
  constexpr float rrqmax = 1.0f / rqmax;             // rounded to nearest, like the host's p.inv_qmax
  const float rqmax_state = p.inv_qmax;
  bool healthy = true;

  for (int t = 0; t < x.T; ++t) {
    const int tc = t % kChunk;
    __syncthreads();                                 // everybody is done with the previous token (and chunk)
    if (tc == 0) {
      // the next chunk of tokens: q, k, v into shared memory (16 bytes per thread and step), gates and
      // norms by one warp per token
      const int nt = (x.T - t < kChunk) ? (x.T - t) : kChunk;
      constexpr int kVecChunks = 3 * L::kVecBytes / 16;
      for (int i = tid; i < nt * kVecChunks; i += kThreads) {
        const int tt = i / kVecChunks, c = i - tt * kVecChunks;
        const int which = c / (L::kVecBytes / 16), cc = c - which * (L::kVecBytes / 16);
        const uint8_t* src = reinterpret_cast<const uint8_t*>(addr[D_Q + which]) + (long long)(t + tt) * x.stride_mixed_t * qes;
        *reinterpret_cast<uint4*>(&vec_t[tt][16 * c]) = __ldg(reinterpret_cast<const uint4*>(src) + cc);
      }
      if (warp < nt)
        tile_meta<RES, RSCALE, QDT, 32>(p, tile, lane, true, &meta_t[warp], nullptr,
                                     (long long)(t + warp) * x.stride_mixed_t, (long long)(t + warp) * x.stride_a_t,
                                     (long long)(t + warp) * x.stride_b_t);
      __syncthreads();
    }
    if (t == 0) {                                    // the tile has to be there; the verdict is the CTA's, not a warp's
      mbar_wait(&full_bar, 0u, poison, p.status);
      __syncthreads();
      healthy = !*poison;
    }
    if (!healthy) break;

    const uint4 tm0 = lds_v4(&meta_t[tc]), tm1 = lds_v4(reinterpret_cast<const uint8_t*>(&meta_t[tc]) + 16);
    const float alpha = __uint_as_float(tm0.w), beta = __uint_as_float(tm1.x), k_mul = __uint_as_float(tm1.y),
                q_mul = __uint_as_float(tm1.z), kq = __uint_as_float(tm1.w);
    const float* sscale = reinterpret_cast<const float*>(sb + L::kSScale);
    const float* rscale = reinterpret_cast<const float*>(sb + L::kRScale);
    const float es_head = (RSCALE == CARRY_SCALE_PER_HEAD) ? rscale[hv & 3] : 0.f;
    const float2 alpha2 = splat(alpha);
    const float2 magic2 = splat(kMagicRound), nmagic2 = splat(-kMagicRound);
    const long long out_tok = out_tok0 + (long long)t * out_tok_stride;

#define CARRY_SLOT_VEC_Q (&vec_t[tc][0])
#define CARRY_SLOT_VEC_K (&vec_t[tc][L::kVecBytes])
#define CARRY_SLOT_VEC_V (&vec_t[tc][2 * L::kVecBytes])
#define CARRY_SLOT_OUT(idx, value) store_from_float(p.out, out_tok + (idx), p.o_dtype, (value))
#define CARRY_SLOT_PUT_SSCALE(r0_, v4_) *reinterpret_cast<uint4*>(sb + L::kSScale + (r0_) * 4) = (v4_)
#define CARRY_SLOT_PUT_CODES(r0_, c0_, cw_)                                                                        \
  {                                                                                                                \
    _Pragma("unroll") for (int i_ = 0; i_ < 4; ++i_)                                                               \
        *reinterpret_cast<uint4*>(sb + L::kCodes + ((r0_) + i_) * kT + (c0_)) =                                    \
        make_uint4(cw_[i_][0], cw_[i_][1], cw_[i_][2], cw_[i_][3]);                                                \
  }
#define CARRY_SLOT_HEAD_RED head_red[t & 1]
#define CARRY_SLOT_MEET(statement) \
  if (lane == 0) { statement; }    \
  warps_meet(3)
#define CARRY_SLOT_RESID_BEGIN()
#define CARRY_SLOT_PUT_RESID4(i_, r0_, c0_, w_) \
  *reinterpret_cast<uint2*>(sb + L::kResid + ((r0_) + (i_)) * (kT / 2) + (c0_) / 2) = (w_)
#define CARRY_SLOT_PUT_RESID8(i_, r0_, c0_, w_) *reinterpret_cast<uint4*>(sb + L::kResid + ((r0_) + (i_)) * kT + (c0_)) = (w_)
#define CARRY_SLOT_PUT_RSCALE_V(r0_, v4_) *reinterpret_cast<uint4*>(sb + L::kRScale + (r0_) * 4) = (v4_)
#define CARRY_SLOT_PUT_RSCALE_HEAD(bits_) reinterpret_cast<uint32_t*>(sb + L::kRScale)[hv & 3] = (bits_)
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
  }

  __syncthreads();
  if (!healthy || *poison) {                         // the copies never arrived: leave the pool as it was,
#pragma unroll 1
    for (int i = 0; i < 200; ++i) __nanosleep(1000);  // after a bounded while for whatever is still on its way
    return;
  }
  // the tile goes back to the pool: 16 bytes per thread and step, whole lines
  for (int i = tid; i < kT * kT / 16; i += kThreads)
    stg_v4(addr[D_CODES] + 16ull * i, *reinterpret_cast<const uint4*>(sb + L::kCodes + 16 * i));
  for (int i = tid; i < L::kResidBytes / 16; i += kThreads)
    stg_v4(addr[D_RESID] + 16ull * i, *reinterpret_cast<const uint4*>(sb + L::kResid + 16 * i));
  if (tid < 32) stg_v4(addr[D_SSCALE] + 16ull * tid, *reinterpret_cast<const uint4*>(sb + L::kSScale + 16 * tid));
  if (RSCALE == CARRY_SCALE_PER_V) {
    if (tid >= 32 && tid < 64)
      stg_v4(addr[D_RSCALE] + 16ull * (tid - 32), *reinterpret_cast<const uint4*>(sb + L::kRScale + 16 * (tid - 32)));
  } else if (tid == 64) {
    stg_b32(addr[D_RSCALE], reinterpret_cast<const uint32_t*>(sb + L::kRScale)[hv & 3]);
  }
}

template <int RES, int RSCALE, int QDT>
int launch_multi_variant(const KParams& p, const MultiExtra& x, cudaStream_t stream) {
  using L = StageLayout<RES, LAYOUT_VK, QDT, RSCALE>;
  auto kern = gdn_multi_kernel<RES, RSCALE, QDT>;
  const size_t smem = (size_t)L::kBytes;
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
  kern<<<(unsigned)((long long)p.B * p.HV), kThreads, smem, stream>>>(p, x);
  return cudaGetLastError() == cudaSuccess ? CARRY_GDN_OK : CARRY_GDN_ERR_LAUNCH;
}

template <int RES, int RSCALE>
int launch_multi_dtype(const KParams& p, const MultiExtra& x, cudaStream_t stream) {
  if (p.qkv_dtype == CARRY_F32) return launch_multi_variant<RES, RSCALE, CARRY_F32>(p, x, stream);
  if (p.qkv_dtype == CARRY_BF16) return launch_multi_variant<RES, RSCALE, CARRY_BF16>(p, x, stream);
  return launch_multi_variant<RES, RSCALE, CARRY_F16>(p, x, stream);
}

}  // namespace

// p describes token 0 of every request exactly as for the single-token call; the caller has checked
// tile128_eligible(p) and that the per-token strides keep every row 16-byte aligned.
int launch_multi(const KParams& p_in, int T, long long stride_mixed_t, long long stride_a_t, long long stride_b_t,
                 cudaStream_t stream) {
  KParams p = p_in;
  auto log2_or_minus1 = [](int v) { int s = 0; while ((1 << s) < v) ++s; return (1 << s) == v ? s : -1; };
  p.hv_shift = log2_or_minus1(p.HV);
  p.group = p.HV / p.H;
  p.group_shift = log2_or_minus1(p.group);
  MultiExtra x = {T, stride_mixed_t, stride_a_t, stride_b_t};
  const bool i4 = p.res_fmt == CARRY_RES_INT4, pv = p.rscale_mode == CARRY_SCALE_PER_V;
  if (i4) return pv ? launch_multi_dtype<CARRY_RES_INT4, CARRY_SCALE_PER_V>(p, x, stream)
                    : launch_multi_dtype<CARRY_RES_INT4, CARRY_SCALE_PER_HEAD>(p, x, stream);
  return pv ? launch_multi_dtype<CARRY_RES_INT8, CARRY_SCALE_PER_V>(p, x, stream)
            : launch_multi_dtype<CARRY_RES_INT8, CARRY_SCALE_PER_HEAD>(p, x, stream);
}

}  // namespace carry
