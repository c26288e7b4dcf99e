/*
 * carry_gdn.h -- C ABI of libcarry_gdn.so: the fused Gated-DeltaNet decode step
 * on an INT8 recurrent state with an error-feedback residual, for NVIDIA B200
 * (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes and a CUDA stream
 * handle (a cudaStream_t passed as void*).  The library never allocates device
 * memory, never synchronises and never changes the current device: the caller
 * makes the right device current, owns every buffer and keeps it alive until
 * the stream has run the kernel.  Return value: 0 on success, a negative
 * CARRY_GDN_ERR_* otherwise; nothing throws across this boundary.  Every entry
 * point reads away the CUDA runtime's per-thread "last error" first, so that a
 * launch failure it reports is its own.
 *
 * What each entry point replaces in tomalmog/carrykernel (paths relative to
 * that project) is cited above it.
 */
#ifndef CARRY_GDN_H_
#define CARRY_GDN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CARRY_GDN_ABI_VERSION 3

/* element types of activations / outputs */
enum { CARRY_F32 = 0, CARRY_BF16 = 1, CARRY_F16 = 2 };

/* residual storage: ids 0..3 are statequant/kernel.py:59-63; 4 and 5 are new */
enum {
  CARRY_RES_FP32 = 0,
  CARRY_RES_FP16 = 1,
  CARRY_RES_FP8 = 2,  /* e5m2 */
  CARRY_RES_INT8 = 3, /* codes + scale */
  CARRY_RES_INT4 = 4, /* two codes per byte along the contiguous axis, even index low nibble */
  CARRY_RES_NONE = 5  /* no error feedback: plain re-quantisation */
};

/* granularity of a scale: one per V channel, or one per (slot, head) matrix */
enum { CARRY_SCALE_PER_V = 0, CARRY_SCALE_PER_HEAD = 1 };

/* scale floor: max(amax, 1e-12)/qmax (statequant/kernel.py:110,173) or
 * max(amax/qmax, 1e-12) (vllm_integration/quantized_packed_decode.py:206,213) */
enum { CARRY_EPS_ON_AMAX = 0, CARRY_EPS_ON_SCALE = 1 };

enum {
  CARRY_GDN_OK = 0,
  CARRY_GDN_ERR_NULL = -1,        /* a required pointer is NULL */
  CARRY_GDN_ERR_SHAPE = -2,       /* a dimension is non-positive or inconsistent */
  CARRY_GDN_ERR_DTYPE = -3,       /* unknown element type id */
  CARRY_GDN_ERR_FORMAT = -4,      /* unknown residual format / scale mode, or odd length for int4 */
  CARRY_GDN_ERR_UNSUPPORTED = -5, /* tile too large for one SM's shared memory */
  CARRY_GDN_ERR_LAUNCH = -6,      /* the CUDA runtime refused the launch */
  CARRY_GDN_ERR_NO_DEVICE = -7,   /* no usable sm_100 device is current */
  CARRY_GDN_ERR_TOO_LARGE = -8    /* beyond a stated fixed capacity */
};

/* bits of the optional device-side status word (OR-ed in by the kernels) */
enum {
  CARRY_GDN_STATUS_BAD_SLOT = 1,   /* a slot id was >= num_slots; that request was treated as padding */
  CARRY_GDN_STATUS_TIMEOUT = 2     /* an asynchronous copy did not complete within the wait limit: that CTA
                                      stopped loading and storing and left its remaining tiles untouched */
};

/*
 * One fused step in the statequant layout: state [B, HV, K, V], V contiguous.
 * Replaces ext.gdn_quant_step(14 tensors, qmax, res_fmt, block_v)
 * (cuda/gdn_state_kernel.cu:310-348, bound at :373-377) and the Triton launch in
 * statequant/kernel.py:379-408.  Output buffers may alias the matching inputs
 * (in-place update); they must not partially overlap anything else.
 */
typedef struct CarryGdnStepArgs {
  const int8_t* h_in;      /* [B,HV,K,V] state codes */
  const float* scale_in;   /* [B,HV,V] (PER_V) or [B,HV] (PER_HEAD) */
  const void* e_in;        /* residual, [B,HV,K,V] in res_fmt ([.., V/2] bytes for INT4); NULL for RES_NONE */
  const float* e_scale_in; /* [B,HV,V] or [B,HV]; INT8/INT4 only, else may be NULL */
  const void* q;           /* [B,HV,K] qkv_dtype */
  const void* k;           /* [B,HV,K] */
  const void* v;           /* [B,HV,V] */
  const float* alpha;      /* [B,HV] decay */
  const float* beta;       /* [B,HV] write strength */
  void* o;                 /* [B,HV,V] o_dtype */
  int8_t* h_out;
  float* scale_out;
  void* e_out;
  float* e_scale_out;
  int32_t B, HV, K, V;
  int32_t qkv_dtype;        /* CARRY_F32 | CARRY_BF16 | CARRY_F16 */
  int32_t o_dtype;
  float qmax;               /* 2^(bits-1) - 1 */
  int32_t res_fmt;          /* CARRY_RES_* */
  int32_t resid_scale_mode; /* CARRY_SCALE_* (INT8/INT4 residual) */
  int32_t state_scale_mode; /* CARRY_SCALE_* */
  int32_t eps_mode;         /* CARRY_EPS_* */
  int32_t* status;          /* optional device word, may be NULL */
} CarryGdnStepArgs;

int carry_gdn_quant_step(const CarryGdnStepArgs* args, void* stream);

/*
 * Unquantised fp32 step, state [B, HV, K, V] fp32.  Replaces
 * ext.gdn_fp32_step (cuda/gdn_state_kernel.cu:350-371) and
 * statequant/kernel.py:411-433.  h_out may alias h_in.
 */
typedef struct CarryGdnFp32Args {
  const float* h_in;
  const void* q;
  const void* k;
  const void* v;
  const float* alpha;
  const float* beta;
  void* o;
  float* h_out;
  int32_t B, HV, K, V;
  int32_t qkv_dtype;
  int32_t o_dtype;
} CarryGdnFp32Args;

int carry_gdn_fp32_step(const CarryGdnFp32Args* args, void* stream);

/*
 * One slot-indexed step, in place on a paged pool [slots, HV, V, K] (K
 * contiguous).  Replaces the Triton launch of _quant_int8_kernel
 * (vllm_integration/quantized_packed_decode.py:303-326; kernel :101-239).
 * Request n uses slot ssm_state_indices[n]; a slot id <= 0 is padding: zeros go
 * to out[n] and the pool is not touched.  Two requests must not name the same
 * slot.  Strides are in elements.
 */
typedef struct CarryGdnPackedArgs {
  const void* mixed_qkv;  /* [B, 2*H*K + HV*V], last stride 1: q | k | v */
  int64_t stride_mixed_tok;
  int32_t qkv_dtype;
  const void* a;          /* [B, HV] */
  int64_t stride_a_tok;
  const void* b;          /* [B, HV] */
  int64_t stride_b_tok;
  int32_t ab_dtype;
  const void* A_log;      /* [HV] */
  int32_t A_log_dtype;
  const void* dt_bias;    /* [HV] */
  int32_t dt_bias_dtype;
  float scale;            /* multiplies q after the optional L2 norm */
  int8_t* state_codes;    /* [slots, HV, V, K] */
  float* state_scale;     /* [slots, HV, V] */
  int8_t* resid_codes;    /* [slots, HV, V, K] (INT8) or [slots, HV, V, K/2] (INT4) */
  float* resid_scale;     /* [slots, HV, V] (PER_V) or [slots, HV] (PER_HEAD) */
  int64_t stride_state_slot;
  int64_t stride_resid_slot;
  int64_t stride_sscale_slot;
  int64_t stride_rscale_slot;
  void* out;              /* [B, 1, HV, V] contiguous */
  int32_t out_dtype;
  const int32_t* ssm_state_indices; /* [B] */
  int64_t stride_indices;
  int32_t B, H, HV, K, V;
  int32_t num_slots;
  int32_t use_qk_l2norm;
  int32_t res_fmt;          /* CARRY_RES_INT8 | CARRY_RES_INT4 */
  int32_t resid_scale_mode; /* CARRY_SCALE_* */
  int32_t eps_mode;         /* CARRY_EPS_* */
  float qmax;               /* state grid, 127 for 8 bits */
  int32_t* status;          /* optional device word, may be NULL */
} CarryGdnPackedArgs;

int carry_gdn_packed_decode(const CarryGdnPackedArgs* args, void* stream);

/*
 * T consecutive tokens of every request in one call: the same step applied T
 * times to each request's slot, with the slot's tile held on chip in between,
 * so the state crosses HBM once per call instead of once per token.  Results
 * are those of T calls of carry_gdn_packed_decode, bit for bit.  No such entry
 * exists in the reference; it is the multi-token decode that vLLM reaches
 * through its speculative-decoding path (the sibling of the call
 * vllm_integration/quantized_packed_decode.py:242 mirrors).
 *
 * `step` describes token 0 exactly as for carry_gdn_packed_decode, with
 * mixed_qkv [B, T, width], a and b [B, T, HV] and out [B, T, HV, V] contiguous:
 * stride_*_tok are the strides between requests, stride_*_t those between the
 * tokens of one request (in elements).  Only the shapes the streaming kernel
 * takes are supported (K = V = 128, 16-byte aligned rows); anything else
 * returns CARRY_GDN_ERR_UNSUPPORTED and the caller loops over tokens.
 */
typedef struct CarryGdnPackedMultiArgs {
  CarryGdnPackedArgs step;
  int32_t T;
  int64_t stride_mixed_t;
  int64_t stride_a_t;
  int64_t stride_b_t;
} CarryGdnPackedMultiArgs;

int carry_gdn_packed_decode_multi(const CarryGdnPackedMultiArgs* args, void* stream);

/*
 * The slot pool of one layer -- the four tensors carry_gdn_packed_decode
 * updates -- for the calls that move a request's state in and out of it.  The
 * reference keeps the pool as four torch tensors and seeds it with eager ops
 * (init_quantized_state, vllm_integration/quantized_packed_decode.py:330-352);
 * it names what a serving engine additionally needs of it -- the residual has
 * to survive paging, preemption, prefix-cache reuse and speculative-decode
 * rollback -- as work not done (same file :50-54).  Within a slot the tensors
 * are contiguous [HV, V, K]; strides between slots are in elements.
 */
typedef struct CarryGdnPool {
  int8_t* state_codes;    /* [slots, HV, V, K] */
  float* state_scale;     /* [slots, HV, V] */
  int8_t* resid_codes;    /* [slots, HV, V, K] (INT8) or [slots, HV, V, K/2] (INT4) */
  float* resid_scale;     /* [slots, HV, V] (PER_V) or [slots, HV] (PER_HEAD) */
  int64_t stride_state_slot;
  int64_t stride_resid_slot;
  int64_t stride_sscale_slot;
  int64_t stride_rscale_slot;
  int32_t num_slots, HV, V, K;
  int32_t res_fmt;          /* CARRY_RES_INT8 | CARRY_RES_INT4 */
  int32_t resid_scale_mode; /* CARRY_SCALE_* */
} CarryGdnPool;

/*
 * Prefill hand-off: quantise the floating-point state h[n] ([HV, V, K], K
 * contiguous -- the final state a prefill kernel returns) of request n into
 * slot slots[n].  State codes and scales are those of init_quantized_state
 * (quantized_packed_decode.py:346-350): scale = max(amax_K|h|, 1e-12) / qmax,
 * codes = round_half_even(h / scale).  keep_error == 0 zeroes the slot's
 * residual, as the reference does; keep_error != 0 stores the quantisation
 * error h - codes * scale as the residual instead (encoded like a decode step
 * encodes it), so the first decode step already feeds it back.  A slot id <= 0
 * is padding and skipped.  Two requests must not name the same slot.
 */
typedef struct CarryGdnPoolStoreArgs {
  CarryGdnPool pool;
  const void* h;          /* [B, HV, V, K] */
  int64_t stride_h_req;   /* elements between requests */
  int32_t h_dtype;        /* CARRY_F32 | CARRY_BF16 | CARRY_F16 */
  const int32_t* slots;   /* [B] */
  int64_t stride_slots;
  int32_t B;
  int32_t keep_error;
  float qmax;             /* state grid, 127 for 8 bits */
  int32_t* status;        /* optional device word, may be NULL */
} CarryGdnPoolStoreArgs;

int carry_gdn_pool_store(const CarryGdnPoolStoreArgs* args, void* stream);

/*
 * The reverse: h[n] = codes * scale (+ resid_codes * resid_scale when
 * with_residual != 0, which is the state the next decode step re-quantises)
 * for slot slots[n], each product rounded to fp32 before the sum.  Hands a
 * request back to a kernel that wants a floating-point state (a further prefill
 * chunk, a swap-out in an engine's own format).  A slot id <= 0 writes zeros.
 */
typedef struct CarryGdnPoolLoadArgs {
  CarryGdnPool pool;      /* read only */
  void* h;                /* [B, HV, V, K] */
  int64_t stride_h_req;
  int32_t h_dtype;
  const int32_t* slots;   /* [B] */
  int64_t stride_slots;
  int32_t B;
  int32_t with_residual;
  int32_t* status;
} CarryGdnPoolLoadArgs;

int carry_gdn_pool_load(const CarryGdnPoolLoadArgs* args, void* stream);

/*
 * Copy whole slots, residual included, bit for bit: slot src_slots[n] of `src`
 * to slot dst_slots[n] of `dst` (the same pool, or a second pool of the same
 * shape and formats: a spill pool for preempted requests, a checkpoint before
 * speculative tokens, a prefix-cache entry).  Pairs with either id <= 0 are
 * skipped.  No destination slot may be the source or destination of another
 * pair of the same call.
 */
typedef struct CarryGdnPoolCopyArgs {
  CarryGdnPool src;       /* read only */
  CarryGdnPool dst;
  const int32_t* src_slots; /* [B] */
  int64_t stride_src_slots;
  const int32_t* dst_slots; /* [B] */
  int64_t stride_dst_slots;
  int32_t B;
  int32_t* status;
} CarryGdnPoolCopyArgs;

int carry_gdn_pool_copy(const CarryGdnPoolCopyArgs* args, void* stream);

/* Human-readable text for a CARRY_GDN_ERR_* code (static storage). */
const char* carry_gdn_strerror(int code);

/* CARRY_GDN_ABI_VERSION the library was built with. */
int carry_gdn_abi_version(void);

/*
 * Which kernel the last successful call on this host thread selected:
 * 0 = none yet, 1 = generic tile kernel, 2 = 128x128 streaming kernel,
 * 3 = multi-token kernel, 4 = a pool store / load / copy kernel,
 * 5 = 128x128 kernel of the step without error feedback.
 * Diagnostic only (tests use it to prove which path ran).
 */
int carry_gdn_last_kernel(void);

#ifdef __cplusplus
}
#endif
#endif /* CARRY_GDN_H_ */
