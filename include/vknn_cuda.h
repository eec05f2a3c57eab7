/* libvknn_cuda — C-ABI of the B200 (sm_100a) attention/encoder kernels that sit behind VKNN's pluggable
 * Backend/Segment interface.
 *
 * Conventions
 *   - every entry point returns an int status: VKC_OK (0) or a negative VKC_ERR_* code; nothing throws;
 *     vkc_last_error(ctx) gives the message of the last failure on that context;
 *   - handles are opaque; buffers are plain pointers + sizes; a context is bound to one CUDA device and is
 *     driven by one host thread at a time (the reference's Session has the same rule, src/core/session.cpp:649);
 *   - `stream` is a cudaStream_t passed as void*; NULL selects the context's own stream;
 *   - device tensors are row-major, exactly like the reference's host tensors (include/vknn/rt_tensor.h:15-43);
 *     storage types: VKC_F32 (Precision::High), VKC_F16 (Precision::Low/Normal), VKC_BF16; accumulation,
 *     softmax and LayerNorm statistics are always fp32 (include/vknn/precision.h:7-11);
 *   - there is no CPU fallback: when no usable device or kernel exists the call fails with an error.
 *
 * Each entry point names the reference interface it stands in for (file:line inside the reference tree).
 */
#ifndef VKNN_CUDA_H
#define VKNN_CUDA_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define VKC_API __attribute__((visibility("default")))

typedef struct vkc_ctx vkc_ctx;
typedef void          *vkc_stream;

enum { VKC_F32 = 0, VKC_F16 = 1, VKC_BF16 = 2, VKC_I32 = 3 };

enum {
    VKC_OK              = 0,
    VKC_ERR_INVALID     = -1, /* bad argument (maps to vknn::Status::InvalidArgument, include/vknn/status.h:7-15) */
    VKC_ERR_UNSUPPORTED = -2, /* shape/dtype the kernels do not cover (Status::Unsupported) */
    VKC_ERR_CUDA        = -3, /* a CUDA runtime/driver call failed (Status::RuntimeError) */
    VKC_ERR_OOM         = -4, /* device allocation failed (Status::RuntimeError) */
    VKC_ERR_DEVICE      = -5, /* a kernel reported a device-side error, e.g. a bounded wait ran out (Status::DeviceLost) */
    VKC_ERR_NO_DEVICE   = -6  /* no CUDA device / not an sm_100 part (Backend::available() == false) */
};

/* GEMM epilogue, applied in this order on the fp32 accumulator: +bias[n], GELU(erf), +residual[m,n]. */
enum { VKC_EPI_NONE = 0, VKC_EPI_BIAS = 1, VKC_EPI_GELU_ERF = 2, VKC_EPI_RESIDUAL = 4 };
/* Layout of the B operand: row-major [K,N] (the reference's MatMul B, and what an initializer holds after the
 * weight Transpose is const-folded, src/import/const_fold.cpp:30-60) or row-major [N,K] (Q.K^T without a Transpose). */
enum { VKC_B_KN = 0, VKC_B_NK = 1 };
/* Kernel family selection, for tests and A/B measurements. AUTO is what the backend uses. */
enum { VKC_IMPL_AUTO = 0, VKC_IMPL_SIMT = 1, VKC_IMPL_TCGEN05 = 2 };

/* ---- context: stands in for the device half of a Backend instance. Reference: Backend::available/configure,
 * include/vknn/backend_class.h:15-31; VulkanContext creation in src/backend/vulkan/vk_backend.cpp:152-188. ---- */
VKC_API int         vkc_device_count(int *count);
VKC_API int         vkc_ctx_create(int device_ordinal, vkc_ctx **out);
VKC_API int         vkc_ctx_destroy(vkc_ctx *ctx);
/* Name, SM count and maximum SM clock (MHz) of the context's device: what a measured table has to be keyed by
 * (the reference keys its caches by the Vulkan device identity, src/backend/vulkan/vk_backend.cpp:445-470). */
VKC_API int         vkc_device_info(const vkc_ctx *ctx, char *name, size_t name_cap, int *sm_count, int *sm_clock_mhz);
VKC_API const char *vkc_last_error(const vkc_ctx *ctx);
VKC_API int         vkc_ctx_set_impl(vkc_ctx *ctx, int impl);
/* Blocks until `stream` is idle, then reports (and clears) any device-side error word the kernels wrote. */
VKC_API int vkc_sync(vkc_ctx *ctx, vkc_stream stream);
/* Number of kernels of this library launched through `ctx` since it was created. */
VKC_API int64_t vkc_launch_count(const vkc_ctx *ctx);

/* ---- memory and boundary transfers. Reference: boundary pack/unpack of a device segment, host fp32 <->
 * device storage precision, src/backend/vulkan/vk_backend.cpp:558-696,1324-1382; weight upload helpers
 * src/backend/vulkan/ops/vk_op_common.h:82-196. Conversion runs on the device. ---- */
VKC_API int vkc_alloc(vkc_ctx *ctx, size_t bytes, void **dptr);
VKC_API int vkc_free(vkc_ctx *ctx, void *dptr);
VKC_API int vkc_upload(vkc_ctx *ctx, void *dst_dev, int dst_dtype, const void *src_host, int src_dtype, int64_t n, vkc_stream stream);
VKC_API int vkc_download(vkc_ctx *ctx, void *dst_host, int dst_dtype, const void *src_dev, int src_dtype, int64_t n, vkc_stream stream);
VKC_API int vkc_convert(vkc_ctx *ctx, void *dst_dev, int dst_dtype, const void *src_dev, int src_dtype, int64_t n, vkc_stream stream);

/* ---- device-resident inputs and outputs. Reference: IOTensor::dmaBufFd / Tensor::fromDmaBuf / toDmaBuf
 * (include/vknn/io_tensor.h:11-23, include/vknn/tensor_class.h:17-29) — the caller names a device buffer by an integer
 * that Session::run passes through untouched (src/core/session.cpp:688-696,715-728) and the device segment binds it as
 * the boundary buffer (src/backend/vulkan/vk_backend.cpp:1218-1260,1339-1382). A CUDA pointer has no file descriptor, so
 * the caller registers it here and hands the returned handle (>= 0x40000000, never a valid fd) to fromDmaBuf/toDmaBuf;
 * the CUDA segment resolves it and converts on the device, with no host staging. The table is process-wide like the
 * fd namespace; the caller keeps ownership of the memory and unregisters before freeing it. ---- */
VKC_API int vkc_extbuf_register(void *dptr, size_t bytes, int *handle);
VKC_API int vkc_extbuf_unregister(int handle);
VKC_API int vkc_extbuf_lookup(int handle, void **dptr, size_t *bytes);

/* ---- K1: batched GEMM with fused epilogue. Reference: MatMulCpu::run src/backend/cpu/ops/matmul.cpp:14-116
 * (oracle), shaders/matmul_tiled.comp:13-95 and matmul_tiled_bias.comp:8-87 with host MatMulOp
 * src/backend/vulkan/ops/matmul.cpp:22-181 (device path replaced); the GELU tail Div/Erf/Add/FusedPointwise
 * (src/backend/cpu/ops/unary.cpp:44, fused_pointwise.cpp:107-167) and the residual Add (ops/add.cpp:66-84).
 *   D[b,m,n] = epi( sum_k A[b,m,k] * B[b,k,n] ),  A: lda-strided rows [M,K]; B per b_layout with row stride ldb;
 *   D and residual: rows of stride ldd; bias: fp32 [N]; batch strides in elements (0 broadcasts an operand). ---- */
VKC_API int vkc_gemm(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                     int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb,
                     int64_t ldd, int b_layout, int epilogue, int dtype, vkc_stream stream);
/* The same with the tensor-core kernel's configuration (tile width, ring depth, CTAs per SM, split-K) chosen by the
 * caller: config in [0, vkc_gemm_config_count()), or -1 for the built-in choice. VKC_ERR_UNSUPPORTED when that
 * configuration cannot run the problem. Reference counterpart: the per-shape kernel autotune behind Hint::Tuning
 * (include/vknn/hint.h:8-22; timing loop and table src/backend/vulkan/ops/vk_op_common.h, WeightCache tuning section
 * src/backend/vulkan/vk_backend.cpp:507-517) — the plug-in times the configurations once per GEMM shape and keeps the
 * table in the session's cache file. */
VKC_API int vkc_gemm_config_count(void);
VKC_API int vkc_gemm_ex(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                        int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb,
                        int64_t ldd, int b_layout, int epilogue, int dtype, int config, vkc_stream stream);

/* ---- K2: fused prefill attention O = softmax(Q.K^T * scale + mask) . V, never materialising the scores.
 * Reference: the node run Transpose(K) -> MatMul -> Binary Mul / FusedPointwise{Mul,Add mask} -> Softmax -> MatMul
 * executed by CpuSegment::run src/backend/cpu/cpu_backend.cpp:94-144 with ops/matmul.cpp:14-116, ops/binary.cpp:31-140,
 * ops/softmax.cpp:9-47; device path replaced: matmul_tiled.comp + flat_softmax.comp:9-50.
 *   Q [B,Hq,Sq,D], K/V [B,Hkv,Skv,D], O [B,Hq,Sq,D]; query head h uses kv head h / (Hq/Hkv);
 *   *_strides = element strides {batch, head, seq} with D contiguous, or NULL for the dense layout (this is how
 *   the head split/merge Reshape/Transpose/Gather nodes are absorbed: ops/transpose.cpp:8-63, ops/gather.cpp:12-63);
 *   causal masks key j > i + (Skv - Sq); kv_len (device int32 [B] or NULL) masks keys >= kv_len[b];
 *   mask (device fp32 [Sq,Skv] additive, or NULL). ---- */
VKC_API int vkc_attn_prefill(vkc_ctx *ctx, const void *Q, const void *K, const void *V, void *O, int64_t B, int64_t Hq, int64_t Hkv,
                             int64_t Sq, int64_t Skv, int64_t D, const int64_t *q_strides, const int64_t *k_strides,
                             const int64_t *v_strides, const int64_t *o_strides, float scale, int causal, const float *mask,
                             const int32_t *kv_len, int dtype, vkc_stream stream);

/* How vkc_attn_prefill's tensor-core kernel (16-bit storage, D in {64,128}, no additive mask) spreads a shape over a GPU
 * with sm_count SMs. Host arithmetic only: no device, no context; the launcher runs the same code. The reference's
 * counterpart is the fixed group count of its dispatches (one workgroup per output tile / per row:
 * src/backend/vulkan/ops/matmul.cpp:172, softmax.cpp:36); here the grid is planned, so the plan can be inspected.
 *   plan[0] form: 0 = one CTA per unit on a (query groups, Hq, B) grid, 1 = persistent CTAs that each run a list of items
 *   plan[1] query tiles of 128 rows a CTA works on at a time (1 or 2)
 *   plan[2] CTAs launched
 *   plan[3] rounds of whole blocks a CTA takes before the left-over blocks (form 1)
 *   plan[4] left-over blocks, cut into plan[5] pieces each of at most plan[6] key tiles of 128 keys
 *   plan[7] key tiles per block
 * A block is one unit (a query group of one batch and head) or, with a causal mask in form 1, the pair of query groups
 * (nq-1-k, k) of one batch and head. vkc_attn_prefill_items lists the items CTA `cta` runs, in order, eight numbers each:
 * batch, head, query group, first key tile, key tiles of query tile 0, of query tile 1, partial-result slot (0 or 1; -1
 * when the item is a whole unit and writes O directly), 1 on the CTA's final item. It returns the number of items (which
 * may exceed max_items; only max_items are written) or a negative VKC_ERR code. has_kv_len: per-sequence lengths will be
 * passed (they rule out form 1; the listed key-tile counts are those of full-length sequences). ---- */
VKC_API int vkc_attn_prefill_plan(int sm_count, int64_t B, int64_t Hq, int64_t Sq, int64_t Skv, int64_t D, int causal, int has_kv_len,
                                  int32_t *plan);
VKC_API int vkc_attn_prefill_items(int sm_count, int64_t B, int64_t Hq, int64_t Sq, int64_t Skv, int64_t D, int causal, int has_kv_len, int cta,
                                   int32_t *items, int max_items);

/* ---- prefill attention with its output fanned out to several GPUs (the all-gather at the attention-output boundary of a
 * head-sharded encoder, done by the kernel that produces the tiles instead of a collective after it). The reference has no
 * multi-device path (docs/LIMITATIONS.md:15-32); the arithmetic is vkc_attn_prefill's (MatMulCpu / SoftmaxCpu chain,
 * src/backend/cpu/ops/matmul.cpp:14-116, softmax.cpp:9-51).
 *   dest[0..n_dest): output buffers addressed with o_strides, all mapped on THIS GPU: its own gather buffer and the peers'
 *     (vkc_peer_open); the kernel stores every output row into each of them (plain peer stores over NVLink).
 *   flag[p]: a 32-bit word in destination p's memory that belongs to this rank. When the last block has stored its rows the
 *     kernel publishes (release, system scope) the number of fan-outs this rank has completed so far. NULL: no signal.
 *   state: two zero-initialised 32-bit words in this GPU's memory (block counter, completed fan-outs); the caller keeps
 *     them for the lifetime of the flags.
 * The consumer calls vkc_peer_wait on its own flag array before reading its buffer. Needs the tensor-core kernel
 * (16-bit storage, D in {64,128}, no additive mask): VKC_ERR_UNSUPPORTED otherwise. ---- */
typedef struct vkc_fanout {
    int       n_dest;
    void     *dest[8];
    uint32_t *flag[8];
    uint32_t *state;
    void     *mcast; /* NULL, or the address of the same output buffer in an NVSwitch multicast mapping that covers all n_dest
                        GPUs (cuMulticast* / a symmetric-memory allocator): the kernel then issues ONE multimem store per 16
                        bytes, which the switch replicates to every destination, instead of n_dest peer stores. dest[] and
                        flag[] are still needed (flags are written per destination). */
} vkc_fanout;
VKC_API int vkc_attn_prefill_fanout(vkc_ctx *ctx, const void *Q, const void *K, const void *V, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                                    int64_t Skv, int64_t D, const int64_t *q_strides, const int64_t *k_strides, const int64_t *v_strides,
                                    const int64_t *o_strides, float scale, int causal, const int32_t *kv_len, int dtype, const vkc_fanout *fan,
                                    vkc_stream stream);
/* LayerNorm whose output rows go to every destination of `fan` (same description as above; dest[d] points at the first of
 * the `rows` rows in destination d): the all-gather of a token-sharded activation done by the kernel that produces it.
 * Arithmetic of vkc_layernorm (LayerNormCpu::run src/backend/cpu/ops/layernorm.cpp:12-79). Rows must be 16-byte aligned
 * and at most 8 * 32 * (16 / element size) elements long: VKC_ERR_UNSUPPORTED otherwise. */
VKC_API int vkc_layernorm_fanout(vkc_ctx *ctx, const void *X, const float *gamma, const float *beta, int64_t rows, int64_t norm, float eps,
                                 int dtype, const vkc_fanout *fan, vkc_stream stream);
/* Waits (on the stream, in a one-block kernel) until each of the n flags has reached *expected + 1, then stores that value
 * to *expected (a 32-bit device word, zero-initialised once). The wait is bounded (about two seconds): on expiry the
 * kernel sets the context's device error word, which the next vkc_sync reports as VKC_ERR_DEVICE, leaves *expected as it
 * was and returns, so a missing peer never hangs the GPU. While the error word is set, later waits on the same context
 * return at once without polling (a captured forward with dozens of waits does not spend the limit dozens of times). */
VKC_API int vkc_peer_wait(vkc_ctx *ctx, const uint32_t *flags, int n, uint32_t *expected, vkc_stream stream);
/* The same wait folded into the consuming GEMM (no separate launch between the producers' signal and the consumer): the
 * kernel's TMA-producer thread of every CTA polls the gate's flags, bounded like vkc_peer_wait (device error 3 on expiry; the
 * kernel then leaves through its own bounded barrier waits without reading A), before its first load. state: two 32-bit
 * device words, zero-initialised once, {expected count, CTAs that have passed}; the last CTA to pass advances the count.
 * A gate state is used either by vkc_peer_wait (its first word) or by gated kernels, not by both in one step. The
 * arithmetic is vkc_gemm_ex's. The reference has no multi-device path (docs/LIMITATIONS.md:15-32). */
typedef struct vkc_gate {
    const uint32_t *flags;
    int             n;
    uint32_t       *state;
} vkc_gate;
VKC_API int vkc_gemm_gated(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                           int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb,
                           int64_t ldd, int b_layout, int epilogue, int dtype, int config, const vkc_gate *gate, vkc_stream stream);
/* Sharing a vkc_alloc'ed buffer with the other processes of the node: export gives 64 opaque bytes to hand to a peer
 * process (any transport), open maps that buffer into this process (peer access over NVLink), close unmaps it. */
#define VKC_PEER_HANDLE_BYTES 64
VKC_API int vkc_peer_export(vkc_ctx *ctx, void *dptr, unsigned char *handle);
VKC_API int vkc_peer_open(vkc_ctx *ctx, const unsigned char *handle, void **dptr);
VKC_API int vkc_peer_close(vkc_ctx *ctx, void *dptr);

/* ---- K3: single-query (decode) attention over a KV cache, split along the cache length. Reference: the same
 * node run as K2 in its decode shape, which the reference executes as naive MatMul (M < 32 path,
 * src/backend/vulkan/ops/matmul.cpp:137-141, shaders/matmul.comp:15-29) -> scale+mask -> flat_softmax -> MatMul.
 *   Q [B,Hq,D], Kc/Vc [B,Hkv,Lmax,D], O [B,Hq,D]; kv_len device int32 [B] (NULL = Lmax for all).
 *   workspace: device scratch of at least vkc_attn_decode_workspace_bytes(...) bytes holding the per-split
 *   partial (max, sum, o) triples; NULL lets the context keep (and grow) its own. ---- */
VKC_API size_t vkc_attn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D);
/* The split kernel's work distribution for a set of sequence lengths, walked on the host (no device, no context):
 * kv_len_host = HOST array of B lengths or NULL for Lmax everywhere. Lists the items of CTA `cta`, six numbers each:
 * sequence, kv head, first key, end key, slot pair (the item's partials are slots 2*pair and 2*pair+1 of its query
 * heads), 1 when the item holds the unit's final key tile. plan (3 numbers or NULL) receives the grid size, the partial
 * slots the workspace holds per (sequence, query head), and the least number of 128-key tiles a CTA takes. Returns the
 * number of items (which may exceed max_items), VKC_ERR_UNSUPPORTED for a shape the tensor-core form does not take,
 * VKC_ERR_INVALID for bad arguments. Used by the CPU test that checks exact coverage and the slot bound. */
VKC_API int vkc_attn_decode_items(int sm_count, int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D, const int32_t *kv_len_host, int cta,
                                  int32_t *items, int max_items, int32_t *plan);
VKC_API int    vkc_attn_decode(vkc_ctx *ctx, const void *Q, const void *Kc, const void *Vc, void *O, int64_t B, int64_t Hq, int64_t Hkv,
                               int64_t Lmax, int64_t D, const int32_t *kv_len, float scale, void *workspace, size_t workspace_bytes,
                               int dtype, vkc_stream stream);

/* ---- K3, allocation-free form. It has no counterpart in the reference. Some hosts may not allocate device memory
 * at the moment they need a decode step: a serving loop that runs inside a memory budget fixed at start-up, a
 * plug-in loaded into a process whose allocator owns the whole device, or a call made from a context where
 * cudaMalloc is forbidden or would stall the device (allocation synchronises). This entry point does the same
 * work as vkc_attn_decode but keeps the per-split partial results in a fixed area compiled into the library
 * (vkc_attn_decode_noalloc_max_bytes() = 16 MiB, resident on every GPU that loads the library until the process
 * ends) and calls no cudaMalloc / cudaFree or any other allocating routine. The caller still passes Q, the cache
 * and O. Shapes whose partials need more than the fixed area (the figure vkc_attn_decode_workspace_bytes returns
 * for the shape) are refused with VKC_ERR_INVALID and a message; nothing is launched.
 * The first call on a device resolves the area's device address (cudaGetSymbolAddress, with that device made
 * current for the lookup); under CUDA's lazy module loading that is also when the driver places the library's code
 * and the area itself on the device, so make that first call at start-up and before any stream capture: only
 * calls after it are free of driver-side allocation. All calls on a device share
 * the one area and it keeps whatever the last call left there: nothing in it needs clearing between calls, but
 * two calls that run concurrently on the same GPU (different streams or contexts) race on it. ---- */
VKC_API size_t vkc_attn_decode_noalloc_max_bytes(void);
VKC_API int    vkc_attn_decode_noalloc(vkc_ctx *ctx, const void *Q, const void *Kc, const void *Vc, void *O, int64_t B, int64_t Hq,
                                       int64_t Hkv, int64_t Lmax, int64_t D, const int32_t *kv_len, float scale, int dtype,
                                       vkc_stream stream);

/* ---- K4: LayerNorm over the trailing `norm` elements. Reference: LayerNormCpu::run
 * src/backend/cpu/ops/layernorm.cpp:12-75 (oracle), shaders/flat_layernorm.comp:8-50 + LayerNormOp
 * src/backend/vulkan/ops/layernorm.cpp:19-76 (device path replaced). gamma/beta fp32 [norm]; beta may be NULL. ---- */
VKC_API int vkc_layernorm(vkc_ctx *ctx, const void *X, const float *gamma, const float *beta, void *Y, int64_t rows, int64_t norm,
                          float eps, int dtype, vkc_stream stream);

/* ---- K5: generic per-element step program. Reference: applyPwEpilogue / FusedPointwiseCpu
 * src/backend/cpu/ops/fused_pointwise.cpp:107-185, BinaryCpu ops/binary.cpp:31-140, UnaryCpu ops/unary.cpp:10-69,
 * AddCpu ops/add.cpp:14-125; device path replaced: shaders/fused_pw_flat.comp + pw_epilogue.glsl:10-39.
 *   Y = program(X); steps: 4 ints per step {kind 0 binary/1 unary/2 act/3 select, code, operand index (1-based into
 *   operands[]), unused}; binary codes 16/17/18 are Equal/Greater/GreaterEqual (1.0 / 0.0 results, EqualCpu ops/equal.cpp,
 *   ops/greater.cpp, ops/greaterequal.cpp); a select step (WhereCpu ops/where.cpp:17-80) treats the running value as the
 *   condition and replaces it by operand[index] when non-zero, else by operand[code]; params: 2 floats per step; operand i has element strides op_strides[i*rank .. +rank)
 *   against the output shape (0 on broadcast dims). At most 8 steps, 6 operands, rank 8
 *   (include/vknn/op_type.h:65-67). Operands share the storage dtype. ---- */
VKC_API int vkc_pointwise(vkc_ctx *ctx, const void *X, void *Y, const int64_t *shape, int rank, int nsteps, const int32_t *steps,
                          const float *params, int noperands, const void *const *operands, const int64_t *op_strides, int dtype,
                          vkc_stream stream);

/* ---- standalone Softmax over rows of `inner` contiguous elements, for Softmax nodes outside an attention
 * pattern. Reference: SoftmaxCpu::run src/backend/cpu/ops/softmax.cpp:9-47; shaders/flat_softmax.comp:9-50. ---- */
VKC_API int vkc_softmax(vkc_ctx *ctx, const void *X, void *Y, int64_t outer, int64_t inner, int dtype, vkc_stream stream);

/* ---- Reduce family over the trailing `n` contiguous elements of each of `rows` rows (the caller moves the reduced axes
 * last): op 0 mean, 1 sum, 2 max, 3 min, 4 product, 5 L2 norm; fp32 accumulation. Reference: ReduceCpu::run
 * src/backend/cpu/ops/reduce.cpp:11-108 (ReduceType include/vknn/reduce_type.h:8). ---- */
VKC_API int vkc_reduce_rows(vkc_ctx *ctx, const void *X, void *Y, int64_t rows, int64_t n, int op, int dtype, vkc_stream stream);

/* ---- strided gather copy Y[i] = X[sum_d idx_d(i) * in_strides[d]] over an output of `shape`, for Transpose /
 * Gather / Slice nodes that cannot be absorbed as strides. Reference: TransposeCpu::run ops/transpose.cpp:8-63;
 * shaders/flat_gather.comp:11-21. ---- */
VKC_API int vkc_strided_copy(vkc_ctx *ctx, const void *X, void *Y, const int64_t *shape, const int64_t *in_strides, int rank,
                             int64_t in_offset, int dtype, vkc_stream stream);
/* The same with a strided destination, Y[sum_d idx_d(i) * out_strides[d]] = X[...]: writes one input of a Concat node
 * into its slab of the output. Reference: ConcatCpu::run src/backend/cpu/ops/concat.cpp:9-66. */
VKC_API int vkc_strided_copy2(vkc_ctx *ctx, const void *X, void *Y, const int64_t *shape, const int64_t *in_strides, const int64_t *out_strides,
                              int rank, int64_t in_offset, int dtype, vkc_stream stream);

/* ---- row moves through offset tables: for r in [0, nrows) copy row_elems contiguous elements from src + src_off[r] to
 * dst + dst_off[r] (offsets in elements, int64 arrays in DEVICE memory; a null table stands for r * row_elems).
 * Destination rows must not overlap. Serves Gather with a constant index list (GatherCpu::run
 * src/backend/cpu/ops/gather.cpp:12-99: the table holds (o * axisSize + idx[k]) * inner) and the update loop of ScatterND
 * (ScatterNDCpu::run src/backend/cpu/ops/scatternd.cpp:49-84; later rows win there, so the caller drops every row whose
 * destination a later row overwrites). ---- */
VKC_API int vkc_copy_rows(vkc_ctx *ctx, const void *src, void *dst, const int64_t *src_off, const int64_t *dst_off, int64_t nrows,
                          int64_t row_elems, int dtype, vkc_stream stream);
/* Gather along an axis with indices produced at run time: out[o, k, :] = data[o, index[k], :] for data
 * [outer, axis_size, inner]. `index` is a device tensor of nidx values of index_dtype: a floating type is truncated toward
 * zero like the reference's cast (gather.cpp:27-30; exact integers reach 2048 in fp16 and 256 in bf16), VKC_I32 is read
 * as is. Negative values count from the end; a value outside the axis is clamped to it. */
VKC_API int vkc_gather_rows(vkc_ctx *ctx, const void *data, const void *index, void *out, int64_t outer, int64_t axis_size, int64_t nidx,
                            int64_t inner, int dtype, int index_dtype, vkc_stream stream);

/* ---- K6: 3D Gaussian-splatting rasterizer, the step after the encoder. Reference: the renderer specified by
 * scripts/yonosplat/ref_rasterizer.py:22-75 (render_view) and implemented for the reference's device by
 * shaders/raster_{preprocess,duplicate,bitonic,ranges,composite,fill}.comp with the host driver examples/yonosplat.cpp.
 *   means [n,3], covs [n,3,3], colors [n,3], opacities [n]: fp32 device arrays (world space; colors already RGB);
 *   w2c: host 4x4 row-major world-to-camera matrix; K: host 3x3 pixel intrinsics; znear: near plane (reference 0.2);
 *   rgb [H,W,3] and alpha [H,W] (may be NULL): fp32 device outputs; precise != 0 computes in double like the float64
 *   specification (bit-comparable decisions), 0 in float. workspace: device memory of vkc_raster_workspace_bytes(n,
 *   H, W, precise) bytes, 256-byte aligned. ---- */
VKC_API size_t vkc_raster_workspace_bytes(int64_t n, int H, int W, int precise);
VKC_API int    vkc_raster_gaussians(vkc_ctx *ctx, const float *means, const float *covs, const float *colors, const float *opacities, int64_t n,
                                    const double *w2c, const double *K, int H, int W, double znear, int precise, float *rgb, float *alpha,
                                    void *workspace, size_t workspace_bytes, vkc_stream stream);

/* ---- segment replay. Reference: the pre-recorded command buffer of a device segment,
 * src/backend/vulkan/vk_backend.cpp:1009-1210 (record) and :1353-1357 (submit). Calls made between begin and
 * end on the context's own stream are captured into a CUDA graph; launch replays it. ---- */
typedef struct vkc_graph vkc_graph;
VKC_API int vkc_graph_begin(vkc_ctx *ctx);
VKC_API int vkc_graph_end(vkc_ctx *ctx, vkc_graph **out);
VKC_API int vkc_graph_launch(vkc_ctx *ctx, vkc_graph *g);
VKC_API int vkc_graph_destroy(vkc_ctx *ctx, vkc_graph *g);

/* ---- profiling. Reference: per-segment timestamps, src/backend/vulkan/vk_backend.cpp:1437-1457. ---- */
VKC_API int vkc_timer_start(vkc_ctx *ctx, vkc_stream stream);
VKC_API int vkc_timer_stop(vkc_ctx *ctx, vkc_stream stream, float *ms);

#ifdef __cplusplus
}
#endif
#endif
