/* C ABI of the B200 window-attention library (libfwa2_b200.so).
 *
 * Plain pointers and sizes only; no torch types.  Every device buffer, including the
 * workspace, is owned by the caller; the library allocates no device memory.  The state it keeps
 * is: a per-thread "last CUDA error", a host-side table of how many thread-block clusters each
 * device holds at once, and -- for fwa2_backward_static_scratch only -- one fixed scratch array
 * in its device image with the per-device address of that array.  All entry points return 0 on
 * success and a negative code on error (see fwa2_strerror); every argument check and every
 * descriptor is done before the first launch, so a rejected call launches nothing and leaves
 * workspace and outputs untouched.  No entry point synchronises the host with the device.
 *
 * A kernel whose bounded device-side wait runs out writes the `status` block and returns with its
 * outputs incomplete; callers of this raw ABI must look at that block (for example by copying it
 * to the host after each step).
 *
 * The two compute entry points are what a binding for the reference project's kernel package
 * (flash_win_attn_v2/kernels/__init__.py:1-2) calls in place of its Triton launches.
 */
#ifndef FWA2_H_
#define FWA2_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FWA2_ABI_VERSION 2

enum fwa2_dtype { FWA2_F16 = 0, FWA2_BF16 = 1 };

enum fwa2_error {
  FWA2_OK = 0,
  FWA2_ERR_NULL = -1,          /* a required pointer is null */
  FWA2_ERR_DTYPE = -2,         /* dtype is not f16 / bf16 */
  FWA2_ERR_HEAD_DIM = -3,      /* head dimension other than 32 */
  FWA2_ERR_SHAPE = -4,         /* non-positive size, N > 640, heads > 192, BW not a multiple of nW */
  FWA2_ERR_STRIDE = -5,        /* a stride that TMA cannot express (not a multiple of 8 elements) */
  FWA2_ERR_ALIGN = -6,         /* a base pointer that is not 16-byte aligned */
  FWA2_ERR_WORKSPACE = -7,     /* workspace missing or too small */
  FWA2_ERR_DRIVER = -8,        /* the CUDA driver entry point for tensor maps is unavailable */
  FWA2_ERR_TENSOR_MAP = -9,    /* cuTensorMapEncodeTiled rejected a descriptor */
  FWA2_ERR_ABI = -10,          /* struct_size / abi_version mismatch */
  FWA2_ERR_LAUNCH = -11,       /* the CUDA runtime refused the launch (see fwa2_last_cuda_error) */
  FWA2_ERR_SCRATCH_LIMIT = -12 /* fwa2_backward_static_scratch: the problem needs more scratch than
                                  FWA2_STATIC_SCRATCH_BYTES */
};

/* Bits of fwa2_fwd_args.variant / fwa2_bwd_args.variant (0 = normal operation). */
#define FWA2_FWD_P_IN_SMEM 1     /* forward: stage P through shared memory instead of TMEM */
#define FWA2_BWD_SKIP_TABLES 2   /* backward: the workspace still holds the transposed tables of an
                                    identical earlier call (used to time the main kernel alone) */
#define FWA2_BWD_SKIP_REDUCE 4   /* backward: leave the per-CTA partials in the workspace */
#define FWA2_BWD_GENERAL_KERNEL 16 /* backward: windows of 65 to 256 tokens normally run on the
                                    cluster kernel (one 128 x 128 score tile per CTA); this bit
                                    selects the general kernel for them instead */
#define FWA2_FWD_GENERAL_KERNEL 32 /* forward: windows of 129 to 256 tokens normally run on the
                                    kernel with two softmax warpgroups per CTA (one per 128-row
                                    tile of the unit); this bit selects the general kernel */
#define FWA2_FWD_COMBINE_TABLES 64 /* forward, bias AND mask, windows of 129 to 256 tokens: add the
                                    two tables once per call into one fp32 table per (window type,
                                    head) in the workspace and let the kernel read that (it then
                                    walks the units table by table).  Without this bit the library
                                    does so only when the batch holds enough images per window type
                                    to pay for the extra pass (fwa2_fwd_workspace_bytes tells), and
                                    falls back to separate tables if the workspace is missing;
                                    with this bit a missing workspace is FWA2_ERR_WORKSPACE */
#define FWA2_FWD_SEPARATE_TABLES 128 /* forward: never combine the tables */

/* A (BW, H, N, 32) tensor of 16-bit elements with unit stride along the last axis.
 * Strides are in elements. */
typedef struct fwa2_tensor4 {
  void* ptr;
  int64_t stride_bw, stride_h, stride_n;
} fwa2_tensor4;

/* Arguments of the forward pass.
 * Replaces `_flash_attn_forward` (flash_win_attn_v2/kernels/attn_kernel_forward.py:261-345). */
typedef struct fwa2_fwd_args {
  uint32_t struct_size;     /* sizeof(fwa2_fwd_args) */
  uint32_t abi_version;     /* FWA2_ABI_VERSION */
  int32_t dtype;            /* fwa2_dtype of q, k, v, o, bias, mask and (tensor mode) logit_scale */
  int32_t bw, heads, n, head_dim;
  int32_t n_windows;        /* mask.shape[0]; the mask of row b of BW is b mod n_windows; 0 if no mask */
  fwa2_tensor4 q, k, v;     /* inputs */
  fwa2_tensor4 o;           /* output, same dtype */
  float* lse;               /* (BW, H, lse_stride_h) fp32: natural-log sum-exp per query row */
  int64_t lse_stride_bw, lse_stride_h;
  const void* logit_scale;  /* tensor mode: H values of `dtype` (the log-domain parameter);
                               scalar mode: one fp32 multiplier */
  int32_t scale_is_tensor;  /* 1 = tensor mode: scale_h = exp(min(g_h, ln 100)) */
  const void* bias;         /* (H, N, bias_row_stride) or NULL */
  const void* mask;         /* (n_windows, N, mask_row_stride) or NULL */
  int64_t bias_row_stride, mask_row_stride;  /* elements; multiples of 8 */
  void* workspace;          /* optional scratch of fwa2_fwd_workspace_bytes() bytes, 256-byte aligned;
                               NULL (or too small) = the kernel reads bias and mask separately */
  size_t workspace_bytes;
  void* status;             /* optional 16-byte device word block written only on a device-side
                               timeout (must be zero-initialised by the caller); may be NULL */
  int32_t variant;          /* FWA2_FWD_* bits */
  int32_t max_ctas;         /* 0 = default (fill the device); otherwise an upper bound on the grid */
  uint64_t* developer0;     /* must be NULL (read only by development builds of the library) */
  int32_t developer1;       /* must be 0 */
  int32_t reserved0;
} fwa2_fwd_args;

/* Arguments of the backward pass.
 * Replaces `_flash_attn_backward` (flash_win_attn_v2/kernels/attn_kernel_backward.py:567-711),
 * including its delta pre-pass (:6-51), the fp32 accumulators and the final casts (:703-711). */
typedef struct fwa2_bwd_args {
  uint32_t struct_size;
  uint32_t abi_version;
  int32_t dtype;
  int32_t bw, heads, n, head_dim;
  int32_t n_windows;
  fwa2_tensor4 q, k, v, o, dout;      /* inputs */
  fwa2_tensor4 dq, dk, dv;            /* outputs, fully overwritten */
  const float* lse;
  int64_t lse_stride_bw, lse_stride_h;
  const void* logit_scale;
  int32_t scale_is_tensor;
  const void* bias;
  const void* mask;
  int64_t bias_row_stride, mask_row_stride;
  void* dbias;              /* (H, N, N) contiguous, `dtype`; NULL when there is no bias */
  void* dscale;             /* H values of `dtype`; NULL in scalar mode */
  float* partial_out;       /* optional (H*N*N + H) fp32: if non-NULL the window-summed dBias and
                               dLogitScale are written here in fp32 (before the clamp gate and
                               the cast) and dbias / dscale are left untouched, so that several
                               GPUs can sum their shards before fwa2_finalize_grads */
  void* workspace;          /* at least fwa2_bwd_workspace_bytes() bytes, 256-byte aligned */
  size_t workspace_bytes;
  void* status;
  int32_t variant;          /* FWA2_BWD_* bits */
  int32_t max_ctas;
  uint64_t* developer0;     /* must be NULL (read only by development builds of the library) */
  int32_t developer1;       /* must be 0 */
  int32_t reserved0;
} fwa2_bwd_args;

int fwa2_abi_version(void);
const char* fwa2_strerror(int code);
/* cudaError_t value of the most recent failed runtime / driver call on this thread (0 if none). */
int fwa2_last_cuda_error(void);

/* Forward pass on `stream` (a cudaStream_t). */
int fwa2_forward(const fwa2_fwd_args* args, void* stream);

/* Bytes of workspace the forward pass would USE for this problem and these variant bits; 0 when it
 * has no use for one (no bias or no mask, other window sizes, too few images per window type and
 * FWA2_FWD_COMBINE_TABLES not set).  The forward never requires a workspace: without one it reads
 * the two tables separately, with the same results up to the rounding of (bias + mask) in fp32. */
size_t fwa2_fwd_workspace_bytes(int32_t bw, int32_t heads, int32_t n, int32_t n_windows,
                                int32_t has_bias, int32_t has_mask, int32_t variant);

/* Scratch bytes the backward pass needs for the given problem (0 on invalid sizes). */
size_t fwa2_bwd_workspace_bytes(int32_t bw, int32_t heads, int32_t n, int32_t n_windows,
                                int32_t has_bias, int32_t has_mask);
/* Backward pass on `stream`. */
int fwa2_backward(const fwa2_bwd_args* args, void* stream);

/* Cast a (possibly all-reduced) fp32 partial buffer [H*N*N dBias | H dLogitScale] to the output
 * dtype; dLogitScale is multiplied by 1[g_h <= ln 100] first
 * (attn_kernel_backward.py:703-711).  dbias / dscale may be NULL. */
int fwa2_finalize_grads(const float* partial, int32_t dtype, int32_t heads, int32_t n,
                        const void* logit_scale, void* dbias, void* dscale, void* stream);

/* The exchange step of the window-sharded backward (one process per GPU, windows split over the
 * GPUs) as one kernel per GPU over peer memory: sums every rank's fp32 [H*N*N dBias | H
 * dLogitScale] buffer in ascending rank order and applies fwa2_finalize_grads' gate and cast.
 * Stands where the reference would need an all-reduce of its fp32 accumulators followed by the
 * casts of attn_kernel_backward.py:703-711 (the reference itself has no multi-GPU path).
 * partials[r] / flags[r]: rank r's buffer and rank r's flag array (at least 8 zero-initialised
 * uint32, written only by this call) as mapped into THIS process (symmetric / peer memory).
 * epoch: 1, 2, 3, ... the same sequence on every rank; consecutive epochs must use different
 * `partials` buffers (two sets, alternating).  Waits for the peers are bounded (about a second);
 * on expiry `status` is written, the outputs are not.  Every rank must make the matching call. */
int fwa2_peer_reduce_finalize(const float* const* partials, uint32_t* const* flags, int32_t rank,
                              int32_t world, uint32_t epoch, int32_t dtype, int32_t heads, int32_t n,
                              const void* logit_scale, void* dbias, void* dscale, void* status,
                              void* stream);

/* The step in front of the operator in Swin-V2 (swin_transformer_v2.py:283-287), fused into one
 * kernel:  bias[h, i, j] = 16 * sigmoid(table[index[i, j], h]).
 * table: (rows, heads), fp32 when table_is_f32 else `dtype`; index: (n, n) int32 with values in
 * [0, rows); bias: (heads, n, n) contiguous, `dtype`. */
int fwa2_cpb_bias_forward(const void* table, int32_t table_is_f32, const int32_t* index, int32_t dtype,
                          int32_t n, int32_t heads, int32_t rows, void* bias, void* stream);

/* Its backward, fed with the fp32 window-summed dBias that fwa2_backward leaves in `partial_out`
 * (so the gradient never passes through a 16-bit (heads, n, n) tensor):
 *   dtable[r, h] = 16 s (1 - s) * sum_{index[i, j] = r} dbias[h, i, j],  s = sigmoid(table[r, h]).
 * row_offsets (rows + 1) / positions (n * n): the inverse of `index` in CSR form (positions of
 * row r are positions[row_offsets[r] .. row_offsets[r + 1]), flat i * n + j, ascending); the
 * summation order is fixed, the result bitwise reproducible.  dtable: (rows, heads) fp32. */
int fwa2_cpb_bias_backward(const float* dbias_f32, const void* table, int32_t table_is_f32, int32_t dtype,
                           const int32_t* row_offsets, const int32_t* positions, int32_t n, int32_t heads,
                           int32_t rows, float* dtable_f32, void* stream);

/* Backward pass that allocates nothing and takes no workspace.  (No counterpart in the reference
 * project, which allocates its fp32 accumulators with torch on every call.)
 *
 * For callers that cannot provide scratch memory: a plugin inside a framework that keeps the
 * device allocator to itself; a serving loop that bans allocator calls once it is warm; code in a
 * context where cudaMalloc is not allowed.
 * Same arguments and results as fwa2_backward, except that `workspace` / `workspace_bytes` are
 * ignored: the scratch is a fixed array of FWA2_STATIC_SCRATCH_BYTES inside the library's
 * device image, present on every GPU that loads the library until the process exits.
 *
 *  - Problems whose fwa2_bwd_workspace_bytes() exceeds FWA2_STATIC_SCRATCH_BYTES are refused
 *    with FWA2_ERR_SCRATCH_LIMIT and nothing is launched.
 *  - The first call on each device looks up the array's device address (the device must be
 *    current); make that first call outside any stream capture.
 *  - All calls on a device share the one array.  Nothing in it has to be cleared between calls,
 *    but two calls that can overlap on the GPU (different streams, no dependency) race on it:
 *    keep them on one stream or order them with events.
 *  - No cudaMalloc / cudaFree or any other allocating routine is called. */
#define FWA2_STATIC_SCRATCH_BYTES (48u << 20)
int fwa2_backward_static_scratch(const fwa2_bwd_args* args, void* stream);

/* Device self-checks of the tensor-core building blocks (used by the test-suite). */
int fwa2_selftest_mma(int mode, int dtype, const void* a, const void* b, float* d, void* status,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FWA2_H_ */
