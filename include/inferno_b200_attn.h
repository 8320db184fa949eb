/* inferno_b200_attn.h -- C ABI of the B200 (sm_100a) causal-attention kernels.
 *
 * Drop-in boundary for the attention sub-path of K9Megahertz/Inferno.  The
 * reference has no plugin or FFI mechanism; its operator API is source level
 * (dtype-dispatch lambda -> raw pointers -> switch on device -> cuda_* launcher,
 * e.g. src/inferno/core/ops.cpp:204-270), and its CUDA launchers are declared in
 * src/inferno/cuda/cudaops.h:14-236 as plain functions over raw device pointers.
 * The entry points below are what such a launcher for a fused attention op binds:
 * raw device pointers, sizes and a stream; no C++ types, no exceptions, no exit().
 *
 * Layout of every tensor: dense row-major [B, H, T, D] (element strides
 * H*T*D, T*D, D, 1), base address 16-byte aligned.  lse is dense [B, H, T] fp32.
 * dtype selects the element type of q, k, v, o, dO, dq, dk, dv.
 *
 * All calls are asynchronous with respect to the host on `stream` and use the
 * caller's current device; the library never calls cudaSetDevice and keeps no
 * global handles.  Every function returns an ib200_status (0 = success).
 */
#ifndef INFERNO_B200_ATTN_H_
#define INFERNO_B200_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Forward-declared so that the header needs no CUDA include; identical to the
 * runtime's cudaStream_t. */
typedef struct CUstream_st* ib200_stream_t;

typedef enum {
    IB200_OK = 0,
    IB200_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive size, bad enum */
    IB200_ERR_UNSUPPORTED = 2,      /* head dim / dtype / mode the kernels do not implement */
    IB200_ERR_MISALIGNED = 3,       /* a base pointer is not 16-byte aligned */
    IB200_ERR_WORKSPACE = 4,        /* workspace missing or smaller than ib200_attn_workspace_bytes */
    IB200_ERR_CUDA = 5,             /* a CUDA runtime/driver call failed (see ib200_last_cuda_error) */
    IB200_ERR_DEVICE_TIMEOUT = 6,   /* a bounded device-side wait expired; outputs are invalid */
    IB200_ERR_NO_DEVICE = 7,        /* no sm_100 device is current */
    IB200_ERR_TOO_LARGE = 8         /* problem needs more scratch than the built-in static buffer holds */
} ib200_status;

enum { IB200_DTYPE_F32 = 0, IB200_DTYPE_BF16 = 1 };
/* Arithmetic of the fp32-I/O path (ignored for bf16 I/O).  One mode exists: every fp32 operand x is carried as the
 * bf16 pair (hi = bf16(x), lo = bf16(x - hi)) and every product is hi*hi + lo*hi + hi*lo on the bf16 tensor pipe with
 * fp32 accumulation -- the accuracy class of a 3xTF32 scheme (measured normwise error <= 1e-5 against float64) at the
 * cost of 1.5 single TF32 passes.  A single-pass TF32 mode is not implemented; values other than
 * IB200_MATH_SPLIT_BF16 are refused with IB200_ERR_UNSUPPORTED. */
enum { IB200_MATH_SPLIT_BF16 = 0 };
enum { IB200_PASS_FWD = 0, IB200_PASS_BWD = 1 };

/* Bytes of device scratch the forward (pass 0) or backward (pass 1) needs for
 * this problem.  The caller owns the allocation; the library never allocates or
 * frees device memory.  The first 256 bytes are a header (device status word, work counter); the
 * workspace need not be initialised.
 * Replaces nothing one-to-one: the reference's launchers cudaMalloc their own
 * scratch per call (e.g. src/inferno/cuda/cudamaskedfill.cu:86-164). */
int ib200_attn_workspace_bytes(int B, int H, int T, int D, int dtype, int pass, size_t* out_bytes);

/* O = softmax(mask(Q K^T * scale)) V and lse = log-sum-exp of the masked, scaled
 * scores of each row.  Replaces InfernoApp/main.cpp:737-754, i.e. the launch
 * sequence cublas_mm_strided_batched_row_major (src/inferno/cuda/cudamatmul.cu:1114-1179),
 * multiply_kernel_broadcast (cudamultiply.cu:16-47), cuda_triu_kernel (cudatri.cu:8-47),
 * masked_fill_kernel (cudamaskedfill.cu:23-73), softmax_strided_kernel
 * (cudasoftmax.cu:52-97) and a second batched GEMM.  causal must be 0 or 1
 * (the reference path is always causal). */
int ib200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                   int B, int H, int T, int D, float scale, int causal, int dtype, int math_mode,
                   void* workspace, size_t workspace_bytes, ib200_stream_t stream);

/* dQ, dK, dV from dO, recomputing P from q, k and the saved lse.  Replaces the
 * reference's backward node chain MMBackward (src/inferno/gradfn/mmbackward.cpp:36-98)
 * -> SoftmaxBackward (softmaxbackward.cpp:36-128, kernel cudasoftmax.cu:222-280)
 * -> MultiplyBackward (multiplybackward.cpp:34-57) -> MMBackward, including the
 * masked_fill backward the reference lacks (ops.cpp:1235-1289). */
int ib200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dO,
                   const float* lse, void* dq, void* dk, void* dv,
                   int B, int H, int T, int D, float scale, int causal, int dtype, int math_mode,
                   void* workspace, size_t workspace_bytes, ib200_stream_t stream);

/* Strided operands.  Element strides of the batch, head and token axes of one [B, H, T, D] operand; the D
 * elements of a row must be contiguous, every stride a multiple of 16 bytes, the base 16-byte aligned.
 * Dense row-major is {H*T*D, T*D, D}.  A q / k / v slice of the packed projection output [B, T, 3, H, D]
 * (the reference's qkv = Wqkv(x), InfernoApp/main.cpp:712) is {T*3*H*D, D, 3*H*D}; an output written straight
 * into [B, T, H, D] (what main.cpp:758-761 obtains with transpose + contiguous + reshape) is {T*H*D, D, H*D}. */
typedef struct {
    int64_t stride_b, stride_h, stride_t;
} ib200_layout;

/* ib200_attn_fwd / ib200_attn_bwd for operands that live inside larger buffers: same semantics, workspace and
 * statuses; each tensor carries its own layout (NULL = dense).  lse stays dense [B, H, T].  These take the
 * place of the reference's layout plumbing around attention -- slice + contiguous (x3), reshape,
 * transpose(1,2).contiguous() (x3), k^T contiguous, and transpose + contiguous on the way out
 * (InfernoApp/main.cpp:716-737, 758-761; SliceBackward's scatter-adds, src/inferno/gradfn/slicebackward.cpp:35-53,
 * on the way back): the TMA descriptors absorb the strides, so no copy kernel runs. */
int ib200_attn_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse,
                           const ib200_layout* lq, const ib200_layout* lk, const ib200_layout* lv, const ib200_layout* lo,
                           int B, int H, int T, int D, float scale, int causal, int dtype, int math_mode,
                           void* workspace, size_t workspace_bytes, ib200_stream_t stream);
int ib200_attn_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* dO, const float* lse,
                           void* dq, void* dk, void* dv,
                           const ib200_layout* lq, const ib200_layout* lk, const ib200_layout* lv, const ib200_layout* lo,
                           const ib200_layout* ldo, const ib200_layout* ldq, const ib200_layout* ldk, const ib200_layout* ldv,
                           int B, int H, int T, int D, float scale, int causal, int dtype, int math_mode,
                           void* workspace, size_t workspace_bytes, ib200_stream_t stream);

/* The projections either side of attention.  C[M,N] = A[M,K] B[K,N] (+ bias[N]), bf16 operands and output, fp32
 * accumulation on the tensor cores, fp32 bias.  a_transposed = 0: A stored [M rows, K contiguous]; 1: stored
 * [K rows, M contiguous].  b_transposed = 0: B stored [K rows, N contiguous]; 1: stored [N rows, K contiguous].
 * M, N, K multiples of 8; bases 16-byte aligned.  Replaces cublas_mm_row_major + the broadcast add of the reference's
 * Linear::forward (src/inferno/modules/linear.cpp:99-106, src/inferno/cuda/cudamatmul.cu:1058-1112,
 * src/inferno/cuda/cudaadd.cu:20-142); a transposed operand costs a descriptor, not the copy the reference makes
 * (src/inferno/gradfn/mmbackward.cpp:77-80).  An expired device-side wait of these kernels is recorded in the status
 * word of the library's built-in buffer (ib200_attn_check_static); the first call on a device looks that buffer's
 * address up once, so make it outside any stream capture. */
int ib200_gemm_bf16(const void* a, const void* b, void* c, const float* bias, int M, int N, int K,
                    int a_transposed, int b_transposed, ib200_stream_t stream);

/* y[M,N] = x[M,K] w[K,N] + bias[N]  (Linear::forward, weight stored [in, out] as in the reference). */
int ib200_linear_fwd(const void* x, const void* w, const float* bias, void* y, int M, int K, int N, ib200_stream_t stream);

/* dx[M,K] = dy w^T, dw[K,N] = x^T dy, db[N] = column sums of dy (fp32); any of dx / dw / db may be NULL.
 * Replaces MMBackward (src/inferno/gradfn/mmbackward.cpp:36-98) and the bias gradient's sum_to_shape for a Linear. */
int ib200_linear_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw, float* db,
                     int M, int K, int N, ib200_stream_t stream);

/* Capacity in bytes of the scratch buffer that is compiled into the library for
 * ib200_attn_bwd_static (one copy lives in the memory of every GPU that loads the library,
 * from load until the process exits). */
#define IB200_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)

/* Backward pass for callers that have no way to hand over scratch memory at call time: code that
 * runs where device allocation is off limits (a latency-critical loop that must never touch the
 * allocator, a host application whose memory pool already owns the whole GPU and offers no hook to
 * borrow from it), so that even the caller-owned workspace of ib200_attn_bwd cannot be provided.
 * Same arguments, results and tolerances as ib200_attn_bwd minus the workspace pair: the dQ
 * accumulator, the per-row vectors and (fp32 I/O) the operand copies live in a fixed buffer of
 * IB200_STATIC_SCRATCH_BYTES inside the library, and the call allocates nothing on host or device.
 *   - A problem whose scratch (what ib200_attn_workspace_bytes reports for IB200_PASS_BWD) exceeds
 *     the buffer is refused with IB200_ERR_TOO_LARGE; nothing is launched.
 *   - The first call on each device looks up the buffer's device address (a one-time set-up step);
 *     make that first call outside any stream capture.
 *   - All calls on a device share the one buffer, which still holds the previous call's contents
 *     when the next begins; the parts that must start from zero are cleared on `stream` by each
 *     call.  Two calls whose kernels may overlap on the GPU (different streams without an ordering
 *     between them) race on it: serialise them.
 *   - An expired device-side wait is reported by ib200_attn_check_static (the buffer is not
 *     caller-visible, so ib200_attn_check cannot read its status word).
 * This entry point has no counterpart in the reference. */
int ib200_attn_bwd_static(const void* q, const void* k, const void* v, const void* o, const void* dO,
                          const float* lse, void* dq, void* dk, void* dv,
                          int B, int H, int T, int D, float scale, int causal, int dtype, int math_mode,
                          ib200_stream_t stream);

/* Synchronises `stream`, then reads the device status word in the header of `workspace`.  The
 * word is sticky: it keeps the site code of the FIRST bounded wait that expired in any forward
 * or backward call that used this workspace since the last check, so one check after a
 * forward + backward pair (or after a whole step) sees a failure of any of them; a failure is
 * reported once and the word is cleared.  Returns IB200_OK, IB200_ERR_DEVICE_TIMEOUT
 * (*device_code receives the site code) or IB200_ERR_CUDA.
 * The reference's counterpart is check_cuda() -> log + exit
 * (src/inferno/cuda/cudaops.h:198-210); this library reports instead of exiting. */
int ib200_attn_check(const void* workspace, ib200_stream_t stream, int* device_code);

/* The same check for the calls that have no caller workspace: ib200_attn_bwd_static and the
 * projection entry points (ib200_gemm_bf16, ib200_linear_fwd, ib200_linear_bwd) record an expired
 * wait in the header of the library's built-in buffer on the current device; this reads and clears
 * it after synchronising `stream`.  Same return values as ib200_attn_check.  Replaces the same
 * check_cuda() convention (src/inferno/cuda/cudaops.h:198-210). */
int ib200_attn_check_static(ib200_stream_t stream, int* device_code);

/* Self-test of the bounded-wait machinery, for test suites: launches one small CTA that allocates
 * tensor memory and waits on a barrier nothing ever signals; after `limit_us` microseconds
 * (1 .. 100000) the wait gives up, the CTA records site code 190 in the header of `workspace`
 * (at least 256 bytes), releases its tensor memory and exits normally -- no fault, no trap; the
 * context stays usable.  ib200_attn_check on the workspace then returns
 * IB200_ERR_DEVICE_TIMEOUT with *device_code == 190.  The reference has no counterpart (its
 * kernels never wait on each other). */
int ib200_selftest_wait_expiry(void* workspace, size_t workspace_bytes, unsigned limit_us, ib200_stream_t stream);

/* Observability hook: CUDA events (cudaEvent_t handles, or NULL) that the following calls on this
 * host thread record on their stream immediately before and after the forward main kernel and the
 * backward main kernel, so a caller can time those kernels apart from the helper passes around
 * them.  Pass four NULLs to switch it off (the default).  The reference's counterpart is its
 * wall-clock lap timer around ops (InfernoApp/timer.h:10-40, laps at InfernoApp/main.cpp:713-765). */
typedef struct CUevent_st* ib200_event_t;
int ib200_attn_set_timing_events(ib200_event_t fwd_start, ib200_event_t fwd_stop,
                                 ib200_event_t bwd_start, ib200_event_t bwd_stop);

/* Dense casts between fp32 and bf16 (round to nearest even) for callers whose tensors are fp32 but who want the bf16
 * kernels: the reference has no 16-bit DType (include/inferno/core/dtype.h:17-26; dispatch tags
 * src/inferno/core/dtype_dispatch.h:43-102), so its tensors reach the bf16 path through these.  n elements, a multiple
 * of 8; both bases 16-byte aligned.  Asynchronous on `stream`. */
int ib200_cast_f32_to_bf16(const float* src, void* dst, size_t n, ib200_stream_t stream);
int ib200_cast_bf16_to_f32(const void* src, float* dst, size_t n, ib200_stream_t stream);

/* Diagnostic, host only (no device needed): the work-item list the persistent bf16 kernels walk for a problem on a GPU with
 * `sm_count` SMs.  Item i of the list is unit `units[i]` (forward: pair of 128-row query tiles, backward: 128-row key tile) of
 * head `heads[i]` (0 <= head < B*H); units are numbered as the tensor is (unit 0 = first rows).  The list runs over groups of
 * consecutive heads; `*n_groups` receives their number.  At most `capacity` entries are written; the return value is the
 * number of items of the list, or a negative IB200_ERR_* value.  The reference has no counterpart (it launches one thread
 * per score row, src/inferno/cuda/cudasoftmax.cu:52-97). */
int ib200_attn_item_order(int pass, int B, int H, int T, int D, int sm_count, int* heads, int* units, int capacity, int* n_groups);

/* Human-readable name of a status value; never NULL. */
const char* ib200_status_string(int status);

/* cudaError_t value of the most recent failing CUDA call on this host thread (0 if none). */
int ib200_last_cuda_error(void);

/* ABI version: major * 1000 + minor. */
int ib200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* INFERNO_B200_ATTN_H_ */
