/*
 * natten_b200 -- C ABI of the B200 neighbourhood-attention library.
 *
 * Plain C: device pointers, sizes and a CUDA stream handle.  No PyTorch types.
 * Every entry point is asynchronous on the given stream, allocates nothing,
 * never synchronises, and returns 0 on success, a negative NATTEN_E_* code for
 * a rejected argument, or a positive cudaError_t value.
 *
 * The reference (natten-mps) has no foreign-function interface: its backends
 * are Python modules that implement the nine-function protocol of
 * src/natten_mps/_core/ops.py:90-152.  Each function below names the protocol
 * function(s) it stands in for; the Python package in this repository binds
 * them with ctypes and re-creates that protocol on top.
 *
 * Tensor layout (heads last, same as the reference):
 *   q      [B, *L, Hq,  D ]   strided: batch / token / head strides in elements,
 *   k      [B, *L, Hkv, D ]            spatial axes collapsed to one token axis,
 *   v      [B, *L, Hkv, Dv]            innermost axis contiguous
 *   out    [B, *O, Hq,  Dv]   contiguous, O_a = ceil(L_a / stride_a)
 *   lse    [B, *O, Hq]        contiguous, float (double when dtype is F64)
 *   logits / attn [B, *O, Hq, prod(kernel)]  contiguous, slots row-major
 *   extra_k [B, Ne, Hkv, D], extra_v [B, Ne, Hkv, Dv]  contiguous
 *   gradients have the shape of what they differentiate and are contiguous.
 */
#ifndef NATTEN_B200_H
#define NATTEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { NATTEN_F32 = 0, NATTEN_F16 = 1, NATTEN_BF16 = 2, NATTEN_F64 = 3 };

enum {
    NATTEN_OK = 0,
    NATTEN_E_INVALID = -1,      /* malformed params (rank, sizes, null pointers)   */
    NATTEN_E_UNSUPPORTED = -2,  /* legal but outside what the kernels cover        */
    NATTEN_E_WORKSPACE = -3,    /* workspace missing or too small                  */
    NATTEN_E_DEVICE = -4,       /* a kernel reported a bounded-wait timeout        */
    NATTEN_E_TOO_LARGE = -5     /* exceeds the built-in scratch of the *_static entry */
};

enum {
    NATTEN_FLAG_FORCE_SIMT = 1, /* skip the tensor-core kernels (tests compare)    */
    NATTEN_FLAG_FORCE_TC = 2    /* fail with UNSUPPORTED instead of falling back   */
};

enum { NATTEN_OP_FUSED_FWD = 0, NATTEN_OP_FUSED_BWD = 1 };

/* Which kernel family served the last call on this thread. */
enum { NATTEN_PATH_NONE = 0, NATTEN_PATH_SIMT = 1, NATTEN_PATH_TCGEN05 = 2 };

typedef struct natten_params {
    int32_t rank;          /* 1, 2 or 3                                           */
    int32_t dtype;         /* NATTEN_F32 / F16 / BF16 / F64                       */
    int32_t batch, heads_q, heads_kv, dim, dim_v;
    int32_t extent[3];     /* padded spatial sizes L_a (unused axes = 1)          */
    int32_t kernel[3];     /* neighbourhood size per axis                         */
    int32_t dilation[3];
    int32_t stride[3];
    int32_t causal[3];     /* 0 / 1 per axis                                      */
    int32_t n_extra;       /* additional key/value tokens per sample (0 = none)   */
    int32_t has_scale;     /* split QK only: 0 = return unscaled dot products     */
    int32_t flags;         /* NATTEN_FLAG_*                                       */
    double scale;          /* resolved logit scale                                */
    int64_t q_stride[3];   /* batch, token, head strides of q (elements)          */
    int64_t k_stride[3];
    int64_t v_stride[3];
    const int32_t* extents;/* device [batch, rank] per-sample sizes, or NULL      */
} natten_params_t;

/* Fused forward: softmax(scale * q k_n^T) v_n over each query's neighbourhood
 * (plus the extra tokens, in the same softmax); writes out and lse.
 * Stands in for na{1,2,3}d_forward of the backend protocol
 * (src/natten_mps/_core/ops.py:90-96; oracle src/natten_mps/_core/pure.py:146-220,
 * 397-433), for the additional-token merge of src/natten_mps/functional.py:285-295
 * and for na{1,2,3}d_varlen_forward (src/natten_mps/_core/pure.py:573-673) when
 * params->extents is set.                                                        */
int natten_fused_fwd(const natten_params_t* params, const void* q, const void* k, const void* v,
                     const void* extra_k, const void* extra_v, void* out, void* lse, void* stream);

/* Fused backward: dq, dk, dv (and d_extra_k / d_extra_v) from dout and the
 * optional dlse, without materialising the attention matrix.  Stands in for
 * na{R}d_fused_backward of the accelerated backend
 * (src/natten_mps/autograd/_factory.py:55-74) and for autograd through the pure
 * backend (src/natten_mps/autograd/_factory.py:95-102).  `workspace` must hold
 * natten_workspace_bytes(params, NATTEN_OP_FUSED_BWD) bytes.                      */
int natten_fused_bwd(const natten_params_t* params, const void* q, const void* k, const void* v,
                     const void* extra_k, const void* extra_v, const void* out, const void* lse,
                     const void* dout, const void* dlse, void* dq, void* dk, void* dv,
                     void* dextra_k, void* dextra_v, void* workspace, size_t workspace_bytes,
                     void* stream);

/* Scratch bytes an op needs (0 when none). */
size_t natten_workspace_bytes(const natten_params_t* params, int op);

/* natten_fused_bwd for callers that cannot allocate device memory (no counterpart in
 * the reference, which always allocates through PyTorch).  Same arguments without the
 * workspace: the scratch is a fixed array of natten_static_scratch_bytes() (4 MiB) inside the
 * library.  A problem fits when natten_workspace_bytes(params, NATTEN_OP_FUSED_BWD) is at most
 * that size; larger problems return NATTEN_E_TOO_LARGE and launch nothing.  The workspace holds
 * one accumulator per (batch, query, head) -- 4 bytes, 8 for F64 -- plus, with additional
 * tokens, their partial gradient sums: e.g. batch * queries * heads_q <= 1 048 576 for
 * F32 / F16 / BF16 without additional tokens, half that for F64.
 * The first call on each device queries the array's device address (no allocation):
 * make it before any stream capture.  All calls on a device share the array, so calls
 * whose kernels can overlap (different streams) race; keep them on one stream.        */
int natten_fused_bwd_static(const natten_params_t* params, const void* q, const void* k, const void* v,
                            const void* extra_k, const void* extra_v, const void* out, const void* lse,
                            const void* dout, const void* dlse, void* dq, void* dk, void* dv,
                            void* dextra_k, void* dextra_v, void* stream);
size_t natten_static_scratch_bytes(void);

/* Split QK forward / backward: na{R}d_qk_forward / na{R}d_qk_backward
 * (src/natten_mps/_core/ops.py:98-110, 126-138; oracle _core/pure.py:223-254,
 * 294-332, 436-471).  Masked slots hold -inf (times scale when has_scale).       */
int natten_qk_fwd(const natten_params_t* params, const void* q, const void* k, void* logits,
                  void* stream);
int natten_qk_bwd(const natten_params_t* params, const void* q, const void* k,
                  const void* dlogits, void* dq, void* dk, void* stream);

/* Split QK with a relative position bias: logits += rpb[h, bias index of (position, slot)], rpb of
 * shape [Hq, 2*K_0-1, (2*K_1-1, (2*K_2-1))] in the tensors' dtype; the backward also returns
 * d_rpb (same shape, every entry written).  Stands in for natten1dqkrpb / natten2dqkrpb of
 * src/natten_mps/compat/v014.py:66-183 (bias window start: src/natten_mps/utils/window.py:119-135)
 * and their autograd.  Unit stride, non-causal, heads_q == heads_kv; anything else returns
 * NATTEN_E_UNSUPPORTED after the plain QK part has been computed.                               */
int natten_qk_rpb_fwd(const natten_params_t* params, const void* q, const void* k, const void* rpb,
                      void* logits, void* stream);
int natten_qk_rpb_bwd(const natten_params_t* params, const void* q, const void* k,
                      const void* dlogits, void* dq, void* dk, void* d_rpb, void* stream);

/* Split AV forward / backward: na{R}d_av_forward / na{R}d_av_backward
 * (src/natten_mps/_core/ops.py:112-124, 140-152; oracle _core/pure.py:257-291,
 * 520-565, 474-517).  heads_q/dim describe attn's head count; dim is unused.     */
int natten_av_fwd(const natten_params_t* params, const void* attn, const void* v, void* out,
                  void* stream);
int natten_av_bwd(const natten_params_t* params, const void* attn, const void* v,
                  const void* dout, void* dattn, void* dv, void* stream);

/* Diagnostics. */
const char* natten_strerror(int code);
int natten_abi_version(void);
int natten_last_path(void);              /* NATTEN_PATH_* of the last call, this thread */
unsigned long long natten_launch_count(void); /* kernels launched by this library so far */
/* Bounded waits.  Every barrier wait inside the tensor-core kernels has a cycle budget; a
 * kernel whose wait runs out raises a status word on its device, stops touching data, frees
 * what it holds and returns, and kernels launched afterwards on that device return at once
 * without computing until the word is cleared.  The three calls below act on the current device.
 *   natten_device_status  synchronises the device; NATTEN_OK or NATTEN_E_DEVICE.
 *   natten_clear_status   synchronises, resets the word; 0 or a cudaError_t value.
 *   natten_status_async   enqueues a 4-byte copy of the word into caller-owned pinned host
 *                         memory on `stream` (no synchronisation, no allocation): non-zero there
 *                         after the stream has passed that point means a kernel gave up.       */
int natten_device_status(void);
int natten_clear_status(void);
int natten_status_async(int32_t* pinned_host_word, void* stream);
/* Test hook: cycle budget of those waits (<= 0 restores the default of about two seconds) and a
 * host-side fault to inject into the following launches (0 = none; 1 = the fused forward's first
 * barrier expects more bytes than its loads deliver, so its wait runs out and the kernel
 * returns with the status word set).  Process-wide.                                            */
void natten_debug_wait(long long budget_cycles, int inject);

#ifdef __cplusplus
}
#endif
#endif /* NATTEN_B200_H */
