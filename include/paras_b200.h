/*
 * paras_b200.h -- C ABI of the B200 (sm_100a) hot-path library `libparas_b200.so`.
 *
 * This is the lower boundary that replaces the reference's compat layer for the
 * transformer hot path.  In the reference that boundary is a C++ template over a device
 * lambda compiled by the ParaS compiler (csrc/compat/paras_compat.h:143-202,
 * `compat::Queue::{alloc,dealloc,copy,memset,synchronize,parallel_for<F>}`); here it is a
 * plain C ABI over hand-written CUDA kernels: `extern "C"`, plain pointers and sizes,
 * `int` status codes, no C++ or torch type in any signature.
 *
 * Conventions
 *   - Every function returns 0 on success and a negative PARAS_E_* code on failure and
 *     never throws; `paras_b200_last_error()` returns the calling thread's last message.
 *     (The reference throws std::runtime_error("ptsycl: ...") from compat::fail,
 *     csrc/compat/paras_compat.cpp:35-37; the operator layer above this ABI turns a
 *     non-zero status back into an exception.)
 *   - `gpu` is a CUDA ordinal 0..count-1.  (The `paras:N` device index of the operator
 *     layer is gpu+1; index 0 is the host engine, csrc/compat/paras_compat.cpp:87-135.)
 *   - `stream` is a `cudaStream_t` passed as `void*`; NULL means the library's own
 *     non-blocking stream of that GPU (the reference creates one per GPU,
 *     csrc/compat/paras_compat.cpp:230-254).
 *   - All device pointers must belong to `gpu`.  Kernels only borrow pointers; outputs
 *     are allocated by the caller.
 *   - There is no CPU fallback: without a usable GPU every compute entry point fails
 *     with PARAS_E_NODEVICE.
 */
#ifndef PARAS_B200_H_
#define PARAS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PARAS_B200_ABI_VERSION 2

enum {
    PARAS_OK = 0,
    PARAS_E_INVALID = -1,     /* bad argument (null pointer, bad shape, misalignment)  */
    PARAS_E_UNSUPPORTED = -2, /* valid request this build has no kernel for            */
    PARAS_E_CUDA = -3,        /* a CUDA runtime/driver call failed                      */
    PARAS_E_NODEVICE = -4,    /* no usable GPU                                          */
    PARAS_E_NOMEM = -5,       /* device or pinned allocation failed                     */
    PARAS_E_TIMEOUT = -6      /* a bounded device-side wait ran out (status word set)   */
};

typedef enum { PARAS_F32 = 0, PARAS_BF16 = 1, PARAS_F16 = 2 } paras_dtype;

/* ---- runtime: replaces compat::enumerate_devices / Queue (paras_compat.h:74-218) ---- */

int paras_b200_abi_version(void);
/* compat::backend_name() (paras_compat.h:221) */
const char* paras_b200_backend_name(void);
const char* paras_b200_last_error(void);
/* Number of CUDA GPUs (0 when there is none; never an error).  enumerate_devices,
 * csrc/compat/paras_compat.cpp:87-135. */
int paras_b200_device_count(void);
int paras_b200_device_name(int gpu, char* buf, size_t buflen);
int paras_b200_device_sm_count(int gpu, int* sms);
/* The library's stream of `gpu` (Queue::init, paras_compat.cpp:230-254). */
int paras_b200_stream(int gpu, void** stream);
/* Queue::synchronize (paras_compat.cpp:354-364): waits for the library stream. */
int paras_b200_synchronize(int gpu);

/* Stream-ordered device memory (replaces Queue::alloc = cudaMallocManaged,
 * paras_compat.cpp:270-307, and core/allocator.cpp's MemoryPool): cudaMallocAsync /
 * cudaFreeAsync on a per-GPU pool with a high release threshold. */
int paras_b200_malloc_async(int gpu, size_t bytes, void* stream, void** ptr);
int paras_b200_free_async(int gpu, void* ptr, void* stream);
/* Bytes handed out and bytes reserved by the pool (MemoryPool::allocated_bytes /
 * cached_bytes, core/allocator.h:43-44). */
int paras_b200_pool_stats(int gpu, uint64_t* used_bytes, uint64_t* reserved_bytes);
/* MemoryPool::clear (core/allocator.cpp): returns cached memory to the driver. */
int paras_b200_pool_trim(int gpu);
/* Caps the bytes the pool of `gpu` may have handed out at any time (0 = no cap; the environment
 * variable PARAS_POOL_LIMIT_MB sets the initial value): an allocation that would pass the cap
 * returns PARAS_E_NOMEM without a CUDA call, as Queue::alloc fails when the device is out of
 * memory (paras_compat.cpp:270-307).  For sharing a GPU and for testing out-of-memory handling. */
int paras_b200_pool_set_limit(int gpu, size_t bytes);

/* Queue::copy / Queue::memset (paras_compat.cpp:326-352).  Host<->device copies of
 * pageable memory go through the library's pinned staging buffers; `blocking` != 0
 * returns only when the bytes have landed (device->host always blocks). */
int paras_b200_memcpy_h2d(int gpu, void* dst, const void* src, size_t bytes, void* stream,
                          int blocking);
int paras_b200_memcpy_d2h(int gpu, void* dst, const void* src, size_t bytes, void* stream);
int paras_b200_memcpy_d2d(int gpu, void* dst, const void* src, size_t bytes, void* stream);
int paras_b200_memcpy_peer(int dst_gpu, void* dst, int src_gpu, const void* src, size_t bytes);
int paras_b200_memset(int gpu, void* dst, int value, size_t bytes, void* stream);
/* Pinned host memory for callers that stage their own transfers. */
int paras_b200_host_alloc(size_t bytes, void** ptr);
int paras_b200_host_free(void* ptr);
/* 1 when `ptr` points into pinned (page-locked) host memory known to CUDA, else 0. */
int paras_b200_host_is_pinned(const void* ptr);

/* Strided copy with element conversion between f32/bf16/f16/f64/i64/i32/i16/i8/u8/bool
 * (the device<->device branch of _copy_from, csrc/ops/tensor_ops.cpp:252-330, and
 * launch_strided_store, core/kernels.h).  `code` values are PARAS_SC_*; sizes/strides in
 * elements, ndim <= 8. */
enum { PARAS_SC_F32 = 0, PARAS_SC_BF16 = 1, PARAS_SC_F16 = 2, PARAS_SC_F64 = 3, PARAS_SC_I64 = 4,
       PARAS_SC_I32 = 5, PARAS_SC_I16 = 6, PARAS_SC_I8 = 7, PARAS_SC_U8 = 8, PARAS_SC_BOOL = 9 };
int paras_b200_strided_copy(int gpu, void* dst, int dst_code, const int64_t* dst_strides,
                            const void* src, int src_code, const int64_t* src_strides,
                            const int64_t* sizes, int ndim, void* stream);
/* fill_.Scalar (tensor_ops.cpp): contiguous fill of n elements with a value given as double. */
int paras_b200_fill(int gpu, void* dst, int code, double value, int64_t n, void* stream);

/* ---- scaled dot product attention forward ----
 * Replaces sdpa_math (csrc/ops/attention_ops.cpp:71-136) together with everything it
 * composes: repeat_interleave (tensor_ops.cpp:687-729), bmm.out (vision_ops.cpp:398-406),
 * mul.out (pointwise_ops.cpp:280-284), ones/tril/masked_fill (creation_ops.cpp:45-51,
 * indexing_ops.cpp:533-596, scatter_ops.cpp:43-71) and _softmax (pointwise_ops.cpp:926-981).
 *
 * q   [B, Hq,  Lq, D]   k, v [B, Hkv, Lk, D]   out [B, Hq, Lq, D]; the last dim is
 * contiguous, the other three have element strides *_strides[3] = {B, H, L}.
 * Hq must be a multiple of Hkv (GQA; query head h reads kv head h / (Hq/Hkv), which is
 * what repeat_interleave produces).  `causal` uses the reference's TOP-LEFT alignment:
 * query i attends keys 0..i whatever Lk-Lq is (attention_ops.cpp:103-116).
 * `mask` (optional, exclusive with causal) is [B, Hq, Lq, Lk] with element strides
 * mask_strides[4] (0 = broadcast); kind 1 = bool (true = attend), 2 = additive in `dtype`,
 * 3 = additive f32 (attention_ops.cpp:117-126).
 * `lse` (optional) receives log-sum-exp of the scaled scores, f32 [B, Hq, Lq].
 * `flags`: PARAS_SDPA_REF_SCALE rounds `scale` to `dtype` first, as the reference's
 * scalar wrapping does (pointwise_ops.cpp:54-59).
 * `workspace` (optional): device scratch for split-KV partial results; when NULL and the
 * chosen kernel needs scratch, it is taken from the GPU's pool and freed stream-ordered.
 * Query it with paras_b200_sdpa_workspace_bytes().
 */
enum { PARAS_SDPA_REF_SCALE = 1, PARAS_SDPA_FORCE_SIMT = 2, PARAS_SDPA_FORCE_TENSOR = 4 };

typedef struct paras_sdpa_args {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    float* lse;
    const void* mask;
    int32_t mask_kind;
    int32_t dtype; /* paras_dtype */
    int32_t B, Hq, Hkv, Lq, Lk, D;
    int64_t q_strides[3];
    int64_t k_strides[3];
    int64_t v_strides[3];
    int64_t o_strides[3];
    int64_t mask_strides[4];
    int32_t causal;
    int32_t flags;
    double scale;
    void* workspace;
    size_t workspace_bytes;
    int32_t gpu;
    int32_t reserved;
    void* stream;
    /* Dropout on the attention weights and the weights themselves (attention_ops.cpp:128-135).  Any
     * of the three below sends the call to a CUDA-core kernel that forms each row of weights twice
     * (statistics, then values) -- the reference's O(Lq*Lk) result cannot come out of a flash kernel:
     *   dropout_p > 0, no dropout_mask: weight i (flat index into the contiguous [B,Hq,Lq,Lk] weights)
     *     is kept when Philox2x32-10(rng_seed, rng_sequence, i).r0 >> 8, as a fraction of 2^24, is below
     *     1 - p, and scaled by 1 / (1 - p) in fp32 -- native_dropout, csrc/ops/random_ops.cpp:27-59,140-176;
     *   dropout_mask: weights * dropout_mask / (1 - p) instead of drawing (kind as for `mask`);
     *   attn_out: receives the weights after dropout, contiguous [B,Hq,Lq,Lk] in `dtype`.
     * All zero / NULL = the fused kernels above. */
    double dropout_p;
    uint64_t rng_seed;
    uint64_t rng_sequence;
    const void* dropout_mask;
    int64_t dropout_mask_strides[4];
    int32_t dropout_mask_kind;
    int32_t reserved2;
    void* attn_out;
} paras_sdpa_args;

int paras_b200_sdpa_fwd(const paras_sdpa_args* args);
int paras_b200_sdpa_workspace_bytes(const paras_sdpa_args* args, size_t* bytes);
/* Is the [Lq, Lk] mask (mask_kind as in paras_sdpa_args, `dtype` the tensors' dtype, rows `row_stride` elements
 * apart) the causal mask written out -- visible exactly where key <= query, i.e. what the reference builds from
 * is_causal (attention_ops.cpp:100-116) -- so that the call may be made with causal = 1 and no mask?  Looks at
 * the mask on the device and WAITS for the answer (*result = 1 or 0): for callers that pick a route by it, such
 * as a backward that takes no mask tensor.  paras_b200_sdpa_fwd itself recognises such masks without waiting. */
int paras_b200_sdpa_mask_is_causal(int gpu, const void* mask, int mask_kind, int dtype, int64_t row_stride, int32_t Lq,
                                   int32_t Lk, double scale, void* stream, int* result);
/* Name of the kernel the last successful paras_b200_sdpa_fwd call of this thread used; for tests and
 * logs.  "tcgen05" (tensor-core tiles), "tcgen05_split" (few query blocks against a long key range: the
 * key range runs in pieces that a second kernel merges; scratch from `workspace` or the pool, size from
 * paras_b200_sdpa_workspace_bytes), "tcgen05_packed" / "tcgen05_packed_split" (2, 4 or 8 query heads per
 * kv head and at most 256 / that many query positions: the group's heads share one pass over K/V),
 * "tcgen05_rope", "decode_mma", "simt", "simt_splitkv", "simt_splitkv_static", "weights". */
const char* paras_b200_sdpa_last_kernel(void);

/* Attention with the rotary position embedding applied to q and k first:
 *     q' = q * cos + rotate_half(q) * sin      (rows q_pos0 .. q_pos0+Lq-1 of the tables)
 *     k' = k * cos + rotate_half(k) * sin      (rows 0 .. Lk-1)
 *     out = sdpa(q', k', v)
 * i.e. what a model composes from paras::rotate_half (csrc/ops/fused_ops.cpp:234-267), two mul and an
 * add (pointwise_ops.cpp:62-85, each rounding to the dtype) in front of sdpa_math
 * (attention_ops.cpp:71-136).  cos, sin: [table_rows, D] contiguous in `dtype`.  With 16-bit tensors
 * and D = 128 the queries are rotated inside the tensor-core kernel, between their TMA load and the
 * first QK^T; the keys -- which every query block re-reads -- are rotated once into pool scratch.
 * No mask tensor, dropout or weights output. */
int paras_b200_sdpa_rope_fwd(const paras_sdpa_args* args, const void* cos, const void* sin,
                             int64_t table_rows, int64_t q_pos0);
/* The rotation alone, out dense [B, H, L, D]; x with element strides {B, H, L} and unit stride on D. */
int paras_b200_rope(int gpu, const void* x, const int64_t* x_strides, const void* cos, const void* sin,
                    void* out, int B, int H, int L, int D, int64_t pos0, int dtype, void* stream);

/* Layout of the split-KV scratch for `splits` > 1 partial results over `rows` = B*Hq*Lq query
 * rows of D elements: byte offsets of the {max, sum} pairs (8-byte entries) and of the fp32
 * partial outputs inside the scratch, and its total size (what paras_b200_sdpa_workspace_bytes
 * reports once the kernel and the number of splits are chosen).  Host arithmetic only; needs no
 * GPU.  Both offsets are multiples of 16 for every rows, D and splits.  (The reference has no
 * split-KV path; its scratch is the [B,H,Lq,Lk] score tensor of attention_ops.cpp:101.) */
int paras_b200_sdpa_split_layout(int64_t rows, int32_t D, int32_t splits, size_t* ml_offset,
                                 size_t* o_offset, size_t* bytes);

/* The same attention on HOST-resident operands: q, k, v and out are host pointers ([B,H,L,D],
 * every batch element a dense [H,L,D] block; strides[0] may be larger).  The call moves batch
 * chunks (about 64 MB of operands each: batch elements, or head groups of one) through the GPU as a three-stage pipeline on three
 * streams -- host-to-device copy of chunk i+1, attention on chunk i, device-to-host copy of
 * chunk i-1 -- so that both directions of the link and the kernel overlap, and returns when the
 * result is in `out`.  Page-locked buffers (paras_b200_host_alloc, or registered with CUDA) are
 * copied directly; pageable ones go through the library's staging ring and lose most of the
 * overlap.  mask, lse and workspace must be NULL.  This is what the reference does implicitly on
 * every call when tensors live on the host (its attention copies operands to the device engine
 * and results back, csrc/ops/vision_ops.cpp:35-37, tensor_ops.cpp:270-322), as one call. */
int paras_b200_sdpa_fwd_host(const paras_sdpa_args* args);

/* No counterpart in the reference.  The same attention, for callers that cannot allocate
 * device memory when they call -- for example a server whose memory manager claimed the whole
 * GPU at start-up, or a latency-bound decode loop: this entry point calls no cudaMalloc /
 * cudaFree and creates no pool, stream or event.  It always runs the CUDA-core (split-KV)
 * kernel; the split-KV partial results live in a fixed device array inside the library
 * (paras_b200_sdpa_static_scratch_bytes() = 4 MiB, resident on every GPU that loaded the
 * library until the process exits).  A problem whose partials do not fit is rejected with
 * PARAS_E_INVALID.  `workspace` is ignored; a NULL `stream` means the legacy default stream.
 * The first call on each GPU looks up the array's device address; make that call outside
 * any stream capture.  All calls share the array: calls that overlap on the GPU race. */
int paras_b200_sdpa_fwd_static_scratch(const paras_sdpa_args* args);
int paras_b200_sdpa_static_scratch_bytes(void);

/* ---- RMSNorm ----
 * mode PARAS_ROUND_ONCE  = paras::rms_norm (csrc/ops/fused_ops.cpp:43-88): wide
 *      accumulation, one rounding of the result; `rstd` (optional, f32[rows]) receives
 *      1/sqrt(mean(x^2)+eps).
 * mode PARAS_ROUND_PER_OP = aten::rms_norm on the reference (csrc/ops/rms_swiglu_ops.cpp:
 *      43-75): emulates its rounding to `dtype` after pow, sum, *1/N, +eps, rsqrt, *inv and
 *      *weight (pointwise_ops.cpp:33-85,246-249), so 16-bit results match it.
 * x, y: [rows, H] contiguous rows with a row stride of H; weight: [H] or NULL.
 */
enum { PARAS_ROUND_ONCE = 0, PARAS_ROUND_PER_OP = 1 };
int paras_b200_rmsnorm_fwd(int gpu, const void* x, const void* weight, void* y, float* rstd,
                           int64_t rows, int64_t H, double eps, int dtype, int mode,
                           void* stream);
/* paras::rms_norm_backward (csrc/ops/fused_ops.cpp:90-157). grad_weight has `dtype`. */
int paras_b200_rmsnorm_bwd(int gpu, const void* grad_out, const void* x, const void* weight,
                           const float* rstd, void* grad_x, void* grad_weight, int64_t rows,
                           int64_t H, int dtype, void* stream);

/* ---- SwiGLU ----
 * mode PARAS_ROUND_ONCE  = paras::swiglu(gate, up) (csrc/ops/fused_ops.cpp:162-194):
 *      out = gate/(1+exp(-gate)) * up, one rounding.
 * mode PARAS_ROUND_PER_OP = torch_paras::swiglu(x, gate) = x * silu(gate)
 *      (csrc/ops/rms_swiglu_ops.cpp:83-86): silu is rounded to `dtype` before the multiply.
 *      Pass x as `up`.
 * Contiguous, n elements.
 */
int paras_b200_swiglu_fwd(int gpu, const void* gate, const void* up, void* out, int64_t n,
                          int dtype, int mode, void* stream);
/* paras::swiglu_backward (csrc/ops/fused_ops.cpp:196-229). */
int paras_b200_swiglu_bwd(int gpu, const void* grad_out, const void* gate, const void* up,
                          void* grad_gate, void* grad_up, int64_t n, int dtype, void* stream);

/* paras::rotate_half / rotate_half_backward (csrc/ops/fused_ops.cpp:234-302): rows of D
 * contiguous elements, out = cat(-x2, x1) (forward) or cat(g2, -g1) (backward). */
int paras_b200_rotate_half(int gpu, const void* x, void* out, int64_t rows, int64_t D, int dtype,
                           int backward, void* stream);

/* ---- attention backward ----
 * The gradient the reference obtains by autograd through sdpa_math (csrc/ops/attention_ops.cpp:
 * 71-136) and its softmax backward (csrc/ops/pointwise_ops.cpp:994-1062).  q, out, dout, dq:
 * dense [B,Hq,Lq,D]; k, v, dk, dv: dense [B,Hkv,Lk,D]; lse: f32 [B,Hq,Lq] as returned by
 * paras_b200_sdpa_fwd (args->lse) for the same inputs, causal flag and scale.  dtype BF16 or F16;
 * D a multiple of 8 (the composite path: Lk too), all pointers 16-byte aligned (else PARAS_E_UNSUPPORTED).
 * D = 128 or 64: two fused tcgen05 kernels (dK/dV, then dQ) that rebuild the probabilities tile by
 * tile in TMEM; deterministic, no atomics, scratch = one fp32 per query row.  Other head dims, or
 * `reserved` = PARAS_SDPA_BWD_COMPOSITE: five batched GEMMs over two [rows, Lk] matrices
 * materialised per chunk of kv-head groups (about 1 GB each at most).  Scratch comes from the
 * GPU's pool, stream-ordered.  No mask tensor, no dropout. */
enum { PARAS_SDPA_BWD_COMPOSITE = 1 };
typedef struct paras_sdpa_bwd_args {
    const void* q;
    const void* k;
    const void* v;
    const void* out;
    const void* dout;
    const float* lse;
    void* dq;
    void* dk;
    void* dv;
    int32_t B, Hq, Hkv, Lq, Lk, D;
    int32_t dtype;
    int32_t causal;
    double scale;
    int32_t gpu;
    int32_t reserved; /* flags: PARAS_SDPA_BWD_COMPOSITE */
    void* stream;
} paras_sdpa_bwd_args;
int paras_b200_sdpa_bwd(const paras_sdpa_bwd_args* args);

/* Attention gradients for the cases the reference reaches by autograd through its composite
 * (attention_ops.cpp:71-136: mask, softmax, dropout, product with V) and paras_b200_sdpa_bwd does not
 * take: an explicit attn_mask, dropout (the same rng_seed / rng_sequence or dropout_mask as the forward
 * call), fp32 tensors, any head dim up to 256, strided q / k / v.  `fwd` is the argument block of the
 * forward call (its `out`, `lse`, `attn_out` and workspace fields are ignored); `dout` is [B, Hq, Lq, D]
 * with element strides dout_strides[3] and unit stride on D; dq, dk, dv are dense [B, H, L, D] in the
 * tensors' dtype.  A CUDA-core path that accumulates dk and dv with atomic adds in fp32: slow, and not
 * bit-reproducible run to run. */
int paras_b200_sdpa_bwd_general(const paras_sdpa_args* fwd, const void* dout, const int64_t* dout_strides,
                                void* dq, void* dk, void* dv);

/* ---- 16-bit GEMM (the projections either side of the path) ----
 * Replaces the host round trip of mm / bmm / addmm / linear (csrc/ops/vision_ops.cpp:248-309,
 * 388-423: both operands copied to the host, at::mm / at::bmm / at::addmm / at::linear in
 * libtorch's CPU library, result copied back).  fp32 accumulation, one rounding of the result.
 *   C[i][M,N] = A[i][M,K] * B[i]  for i < batch
 *   a_layout PARAS_GEMM_A_MK (0, default): A is [M,K], rows of K elements, row stride lda
 *            PARAS_GEMM_A_KM: A is [K,M], rows of M elements (C = A^T B; no epilogue)
 *   b_layout PARAS_GEMM_B_NK: B is [N,K], rows of K elements (a Linear weight; C = A B^T)
 *            PARAS_GEMM_B_KN: B is [K,N], rows of N elements (mm / bmm; C = A B)
 *   epilogue PARAS_GEMM_EPI_NONE
 *            PARAS_GEMM_EPI_BIAS:   C += bias[N] (same dtype), added in fp32 before the rounding
 *            PARAS_GEMM_EPI_SWIGLU: b = gate weight [N,K], b2 = up weight [N,K] (layout NK only);
 *                C[M,N] = swiglu(A b^T, A b2^T) with both projections rounded to `dtype` first,
 *                i.e. what linear, linear, paras::swiglu (csrc/ops/fused_ops.cpp:162-194) give.
 *            PARAS_GEMM_EPI_ROWSCALE: C[m, :] *= row_scale[m] (fp32 [batch * M]) before the rounding.
 *                With b = W o w (paras_b200_scale_columns) and row_scale = rstd (paras_b200_rms_rstd)
 *                this is linear(rms_norm(A, w), W) -- csrc/ops/rms_swiglu_ops.cpp:43-75 feeding
 *                vision_ops.cpp:248-309 -- without the normalised activations ever being written.
 * All leading dimensions and batch strides are in elements and must be multiples of 8 (16
 * bytes), all base pointers 16-byte aligned; otherwise PARAS_E_UNSUPPORTED (the caller keeps
 * its own path for such operands).  dtype: PARAS_BF16 or PARAS_F16. */
enum { PARAS_GEMM_B_NK = 0, PARAS_GEMM_B_KN = 1 };
enum { PARAS_GEMM_A_MK = 0, PARAS_GEMM_A_KM = 1 };
enum { PARAS_GEMM_EPI_NONE = 0, PARAS_GEMM_EPI_BIAS = 1, PARAS_GEMM_EPI_SWIGLU = 2, PARAS_GEMM_EPI_ROWSCALE = 5 };
typedef struct paras_gemm_args {
    const void* a;
    const void* b;
    const void* b2;     /* up weight, SwiGLU epilogue only */
    const void* bias;   /* [N], bias epilogue only */
    void* c;
    int64_t M, N, K;
    int64_t lda, ldb, ldc;
    int64_t batch;      /* >= 1 */
    int64_t stride_a, stride_b, stride_c;  /* elements between consecutive matrices (batch > 1) */
    int32_t dtype;
    int32_t b_layout;
    int32_t epilogue;
    int32_t gpu;
    void* stream;
    int32_t a_layout;
    int32_t reserved;
    const float* row_scale; /* [batch * M], row-scale epilogue only */
} paras_gemm_args;
int paras_b200_gemm(const paras_gemm_args* args);

/* The two small passes that fold RMSNorm (csrc/ops/fused_ops.cpp:43-88) into the projection after it:
 *   rstd[r] = 1 / sqrt(mean(x[r, :]^2) + eps)        fp32 [rows]; x [rows, H] contiguous (one read of x)
 *   out[n, k] = weight[n, k] * scale[k]               [N, K] contiguous rows, one rounding; done once per
 *                                                     weight when the caller keeps the result */
int paras_b200_rms_rstd(int gpu, const void* x, float* rstd, int64_t rows, int64_t H, double eps, int dtype,
                        void* stream);
int paras_b200_scale_columns(int gpu, const void* weight, const void* scale, void* out, int64_t N, int64_t K,
                             int dtype, void* stream);

/* ---- failure path self-test ----
 * No counterpart in the reference (its kernels have no device-side waits; a stuck queue there
 * hangs the process in Queue::synchronize, csrc/compat/paras_compat.cpp:354-364).  Launches a
 * one-warp kernel on the library's stream of `gpu` whose single bounded wait -- the same
 * primitive every tensor-core kernel here waits with -- is on a barrier nobody arrives at, with
 * a limit of `limit_us` microseconds (1..1000000).  The wait gives up, the kernel returns by
 * itself and the call returns what any later call would after a production kernel gave up:
 * PARAS_E_TIMEOUT, once; `status_word` (optional) receives the raw word the kernel wrote
 * (0x40000000 | 1 << 27).  The GPU and the library stay usable afterwards. */
int paras_b200_selftest_bounded_wait(int gpu, uint32_t limit_us, int* status_word);

#ifdef __cplusplus
}
#endif
#endif /* PARAS_B200_H_ */
