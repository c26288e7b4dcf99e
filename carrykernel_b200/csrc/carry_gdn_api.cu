// C ABI of libcarry_gdn.so: argument checks and kernel selection.  See
// include/carry_gdn.h for the contract of every entry point.
#include "carry_gdn_common.cuh"

namespace {

thread_local int g_last_kernel = 0;

bool dtype_ok(int d) { return d == CARRY_F32 || d == CARRY_BF16 || d == CARRY_F16; }
bool scale_mode_ok(int m) { return m == CARRY_SCALE_PER_V || m == CARRY_SCALE_PER_HEAD; }
bool eps_ok(int m) { return m == CARRY_EPS_ON_AMAX || m == CARRY_EPS_ON_SCALE; }

int dispatch(const carry::KParams& p, cudaStream_t stream) {
  if ((long long)p.B * p.HV == 0) return CARRY_GDN_OK;
  if (carry::tile128_eligible(p)) {
    const int rc = carry::launch_tile128(p, stream);
    if (rc == CARRY_GDN_OK) g_last_kernel = 2;
    return rc;
  }
  if (carry::noef128_eligible(p)) {
    const int rc = carry::launch_noef128(p, stream);
    if (rc == CARRY_GDN_OK) g_last_kernel = 5;
    return rc;
  }
  const int rc = carry::launch_generic(p, stream);
  if (rc == CARRY_GDN_OK) g_last_kernel = 1;
  return rc;
}

}  // namespace

namespace carry {
// Checks the arguments of the slot-indexed call and turns them into kernel parameters.
int packed_params(const CarryGdnPackedArgs* a, KParams& p) {
  if (!a) return CARRY_GDN_ERR_NULL;
  if (a->B < 0 || a->H <= 0 || a->HV <= 0 || a->K <= 0 || a->V <= 0 || a->num_slots < 0)
    return CARRY_GDN_ERR_SHAPE;
  if (a->HV % a->H != 0) return CARRY_GDN_ERR_SHAPE;
  if (!(a->qmax >= 1.0f && a->qmax <= 127.0f)) return CARRY_GDN_ERR_SHAPE;
  if (!dtype_ok(a->qkv_dtype) || !dtype_ok(a->out_dtype) || !dtype_ok(a->ab_dtype) ||
      !dtype_ok(a->A_log_dtype) || !dtype_ok(a->dt_bias_dtype))
    return CARRY_GDN_ERR_DTYPE;
  if (a->res_fmt != CARRY_RES_INT8 && a->res_fmt != CARRY_RES_INT4) return CARRY_GDN_ERR_FORMAT;
  if (!scale_mode_ok(a->resid_scale_mode) || !eps_ok(a->eps_mode)) return CARRY_GDN_ERR_FORMAT;
  if (a->res_fmt == CARRY_RES_INT4 && (a->K & 1)) return CARRY_GDN_ERR_FORMAT;
  if (a->B == 0) return CARRY_GDN_OK;   // nothing to do; p is not filled
  if (!a->mixed_qkv || !a->a || !a->b || !a->A_log || !a->dt_bias || !a->state_codes ||
      !a->state_scale || !a->resid_codes || !a->resid_scale || !a->out || !a->ssm_state_indices)
    return CARRY_GDN_ERR_NULL;

  p = carry::KParams{};
  p.packed = 1;
  p.B = a->B; p.H = a->H; p.HV = a->HV; p.K = a->K; p.V = a->V;
  p.qmax = a->qmax;
  p.inv_qmax = 1.0f / a->qmax;
  p.res_fmt = a->res_fmt; p.rscale_mode = a->resid_scale_mode; p.sscale_mode = CARRY_SCALE_PER_V;
  p.eps_mode = a->eps_mode;
  p.qkv_dtype = a->qkv_dtype; p.o_dtype = a->out_dtype;
  p.status = a->status;
  p.codes_in = a->state_codes; p.codes_out = a->state_codes;
  p.sscale_in = a->state_scale; p.sscale_out = a->state_scale;
  p.resid_in = a->resid_codes; p.resid_out = a->resid_codes;
  p.rscale_in = a->resid_scale; p.rscale_out = a->resid_scale;
  p.stride_state_slot = a->stride_state_slot; p.stride_resid_slot = a->stride_resid_slot;
  p.stride_sscale_slot = a->stride_sscale_slot; p.stride_rscale_slot = a->stride_rscale_slot;
  p.q = a->mixed_qkv; p.k = a->mixed_qkv; p.v = a->mixed_qkv;
  p.stride_mixed_tok = a->stride_mixed_tok;
  p.a = a->a; p.b = a->b; p.stride_a_tok = a->stride_a_tok; p.stride_b_tok = a->stride_b_tok;
  p.ab_dtype = a->ab_dtype;
  p.A_log = a->A_log; p.dt_bias = a->dt_bias;
  p.A_log_dtype = a->A_log_dtype; p.dt_bias_dtype = a->dt_bias_dtype;
  p.qscale = a->scale;
  p.l2norm = a->use_qk_l2norm;
  p.slot_idx = a->ssm_state_indices; p.stride_idx = a->stride_indices;
  p.num_slots = a->num_slots;
  p.out = a->out;
  return CARRY_GDN_OK;
}
}  // namespace carry

// The runtime keeps a per-thread "last error" until somebody reads it.  Every entry point reads it away
// first, so that a launch failure reported by this library is this call's and not a leftover of the host
// program's earlier CUDA calls (sticky errors, i.e. a lost context, come back on the next call anyway).
static inline void clear_stale_error() { (void)cudaGetLastError(); }

extern "C" {

int carry_gdn_abi_version(void) { return CARRY_GDN_ABI_VERSION; }

int carry_gdn_last_kernel(void) { return g_last_kernel; }

const char* carry_gdn_strerror(int code) {
  switch (code) {
    case CARRY_GDN_OK: return "ok";
    case CARRY_GDN_ERR_NULL: return "a required pointer is NULL";
    case CARRY_GDN_ERR_SHAPE: return "a dimension is non-positive or inconsistent";
    case CARRY_GDN_ERR_DTYPE: return "unknown element type";
    case CARRY_GDN_ERR_FORMAT: return "unknown residual format or scale mode, or odd contiguous length for int4";
    case CARRY_GDN_ERR_UNSUPPORTED: return "tile does not fit one SM's shared memory";
    case CARRY_GDN_ERR_LAUNCH: return "the CUDA runtime refused the launch";
    case CARRY_GDN_ERR_NO_DEVICE: return "no usable sm_100 device is current";
    case CARRY_GDN_ERR_TOO_LARGE: return "request exceeds a fixed capacity of this entry point";
    default: return "unknown error code";
  }
}

int carry_gdn_quant_step(const CarryGdnStepArgs* a, void* stream) {
  clear_stale_error();
  if (!a) return CARRY_GDN_ERR_NULL;
  if (a->B < 0 || a->HV < 0 || a->K <= 0 || a->V <= 0) return CARRY_GDN_ERR_SHAPE;
  if (!(a->qmax >= 1.0f && a->qmax <= 127.0f)) return CARRY_GDN_ERR_SHAPE;
  if (!dtype_ok(a->qkv_dtype) || !dtype_ok(a->o_dtype)) return CARRY_GDN_ERR_DTYPE;
  if (a->res_fmt < CARRY_RES_FP32 || a->res_fmt > CARRY_RES_NONE) return CARRY_GDN_ERR_FORMAT;
  if (!scale_mode_ok(a->resid_scale_mode) || !scale_mode_ok(a->state_scale_mode) || !eps_ok(a->eps_mode))
    return CARRY_GDN_ERR_FORMAT;
  if (a->res_fmt == CARRY_RES_INT4 && (a->V & 1)) return CARRY_GDN_ERR_FORMAT;
  if ((long long)a->B * a->HV == 0) return CARRY_GDN_OK;
  if (!a->h_in || !a->scale_in || !a->q || !a->k || !a->v || !a->alpha || !a->beta || !a->o ||
      !a->h_out || !a->scale_out)
    return CARRY_GDN_ERR_NULL;
  const bool int_resid = a->res_fmt == CARRY_RES_INT8 || a->res_fmt == CARRY_RES_INT4;
  if (a->res_fmt != CARRY_RES_NONE && (!a->e_in || !a->e_out)) return CARRY_GDN_ERR_NULL;
  if (int_resid && (!a->e_scale_in || !a->e_scale_out)) return CARRY_GDN_ERR_NULL;

  carry::KParams p = {};
  p.packed = 0;
  p.B = a->B; p.H = a->HV; p.HV = a->HV; p.K = a->K; p.V = a->V;
  p.qmax = a->qmax;
  p.inv_qmax = 1.0f / a->qmax;
  p.res_fmt = a->res_fmt; p.rscale_mode = a->resid_scale_mode; p.sscale_mode = a->state_scale_mode;
  p.eps_mode = a->eps_mode;
  p.qkv_dtype = a->qkv_dtype; p.o_dtype = a->o_dtype;
  p.status = a->status;
  p.codes_in = a->h_in; p.codes_out = a->h_out;
  p.sscale_in = a->scale_in; p.sscale_out = a->scale_out;
  p.resid_in = a->e_in; p.resid_out = a->e_out;
  p.rscale_in = a->e_scale_in; p.rscale_out = a->e_scale_out;
  p.q = a->q; p.k = a->k; p.v = a->v;
  p.alpha = a->alpha; p.beta = a->beta;
  p.qscale = 1.0f;
  p.out = a->o;
  return dispatch(p, static_cast<cudaStream_t>(stream));
}

int carry_gdn_fp32_step(const CarryGdnFp32Args* a, void* stream) {
  clear_stale_error();
  if (!a) return CARRY_GDN_ERR_NULL;
  if (a->B < 0 || a->HV < 0 || a->K <= 0 || a->V <= 0) return CARRY_GDN_ERR_SHAPE;
  if (!dtype_ok(a->qkv_dtype) || !dtype_ok(a->o_dtype)) return CARRY_GDN_ERR_DTYPE;
  if ((long long)a->B * a->HV == 0) return CARRY_GDN_OK;
  if (!a->h_in || !a->q || !a->k || !a->v || !a->alpha || !a->beta || !a->o || !a->h_out)
    return CARRY_GDN_ERR_NULL;
  const int rc = carry::launch_fp32(*a, static_cast<cudaStream_t>(stream));
  if (rc == CARRY_GDN_OK) g_last_kernel = 1;
  return rc;
}

int carry_gdn_packed_decode(const CarryGdnPackedArgs* a, void* stream) {
  clear_stale_error();
  carry::KParams p;
  const int rc = carry::packed_params(a, p);
  if (rc != CARRY_GDN_OK || a->B == 0) return rc;
  return dispatch(p, static_cast<cudaStream_t>(stream));
}

int carry_gdn_packed_decode_multi(const CarryGdnPackedMultiArgs* m, void* stream) {
  clear_stale_error();
  if (!m) return CARRY_GDN_ERR_NULL;
  if (m->T < 1) return CARRY_GDN_ERR_SHAPE;
  carry::KParams p;
  const int rc = carry::packed_params(&m->step, p);
  if (rc != CARRY_GDN_OK || m->step.B == 0) return rc;
  const int qes = p.qkv_dtype == CARRY_F32 ? 4 : 2;
  if (!carry::tile128_eligible(p) || (m->stride_mixed_t * qes) % 16) return CARRY_GDN_ERR_UNSUPPORTED;
  const int rc2 = carry::launch_multi(p, m->T, m->stride_mixed_t, m->stride_a_t, m->stride_b_t,
                                      static_cast<cudaStream_t>(stream));
  if (rc2 == CARRY_GDN_OK) g_last_kernel = 3;
  return rc2;
}

namespace {
int pool_ok(const CarryGdnPool& pool) {
  if (pool.HV <= 0 || pool.K <= 0 || pool.V <= 0 || pool.num_slots < 0) return CARRY_GDN_ERR_SHAPE;
  if (pool.res_fmt != CARRY_RES_INT8 && pool.res_fmt != CARRY_RES_INT4) return CARRY_GDN_ERR_FORMAT;
  if (!scale_mode_ok(pool.resid_scale_mode)) return CARRY_GDN_ERR_FORMAT;
  if (pool.res_fmt == CARRY_RES_INT4 && (pool.K & 1)) return CARRY_GDN_ERR_FORMAT;
  return CARRY_GDN_OK;
}
bool pool_has_pointers(const CarryGdnPool& pool) {
  return pool.state_codes && pool.state_scale && pool.resid_codes && pool.resid_scale;
}
}  // namespace

int carry_gdn_pool_store(const CarryGdnPoolStoreArgs* a, void* stream) {
  clear_stale_error();
  if (!a) return CARRY_GDN_ERR_NULL;
  if (a->B < 0) return CARRY_GDN_ERR_SHAPE;
  const int rc = pool_ok(a->pool);
  if (rc != CARRY_GDN_OK) return rc;
  if (!(a->qmax >= 1.0f && a->qmax <= 127.0f)) return CARRY_GDN_ERR_SHAPE;
  if (!dtype_ok(a->h_dtype)) return CARRY_GDN_ERR_DTYPE;
  if (a->B == 0) return CARRY_GDN_OK;
  if (!a->h || !a->slots || !pool_has_pointers(a->pool)) return CARRY_GDN_ERR_NULL;
  const int rc2 = carry::launch_pool_store(*a, static_cast<cudaStream_t>(stream));
  if (rc2 == CARRY_GDN_OK) g_last_kernel = 4;
  return rc2;
}

int carry_gdn_pool_load(const CarryGdnPoolLoadArgs* a, void* stream) {
  clear_stale_error();
  if (!a) return CARRY_GDN_ERR_NULL;
  if (a->B < 0) return CARRY_GDN_ERR_SHAPE;
  const int rc = pool_ok(a->pool);
  if (rc != CARRY_GDN_OK) return rc;
  if (!dtype_ok(a->h_dtype)) return CARRY_GDN_ERR_DTYPE;
  if (a->B == 0) return CARRY_GDN_OK;
  if (!a->h || !a->slots || !pool_has_pointers(a->pool)) return CARRY_GDN_ERR_NULL;
  const int rc2 = carry::launch_pool_load(*a, static_cast<cudaStream_t>(stream));
  if (rc2 == CARRY_GDN_OK) g_last_kernel = 4;
  return rc2;
}

int carry_gdn_pool_copy(const CarryGdnPoolCopyArgs* a, void* stream) {
  clear_stale_error();
  if (!a) return CARRY_GDN_ERR_NULL;
  if (a->B < 0) return CARRY_GDN_ERR_SHAPE;
  int rc = pool_ok(a->src);
  if (rc == CARRY_GDN_OK) rc = pool_ok(a->dst);
  if (rc != CARRY_GDN_OK) return rc;
  if (a->src.HV != a->dst.HV || a->src.K != a->dst.K || a->src.V != a->dst.V) return CARRY_GDN_ERR_SHAPE;
  if (a->src.res_fmt != a->dst.res_fmt || a->src.resid_scale_mode != a->dst.resid_scale_mode)
    return CARRY_GDN_ERR_FORMAT;
  if (a->B == 0) return CARRY_GDN_OK;
  if (!a->src_slots || !a->dst_slots || !pool_has_pointers(a->src) || !pool_has_pointers(a->dst))
    return CARRY_GDN_ERR_NULL;
  const int rc2 = carry::launch_pool_copy(*a, static_cast<cudaStream_t>(stream));
  if (rc2 == CARRY_GDN_OK) g_last_kernel = 4;
  return rc2;
}

}  // extern "C"
