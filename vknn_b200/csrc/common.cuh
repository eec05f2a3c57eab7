// Shared host/device helpers of libvknn_cuda: the context object, status plumbing and storage-type traits.
#pragma once
#include "vknn_cuda.h"
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <set>
#include <string>
#include <vector>
#include <utility>
#include <type_traits>

// Device-side error codes written to vkc_ctx::dev_err (first writer wins).
enum : int {
    VKC_DEVERR_NONE         = 0,
    VKC_DEVERR_WAIT_TIMEOUT = 1, // a bounded mbarrier wait ran out
    VKC_DEVERR_TMEM_ALLOC   = 2,
};

struct vkc_ctx {
    int          device     = 0;
    int          sm_count   = 0;
    size_t       l2_bytes   = 0;
    int          cc_major   = 0;
    int          impl       = VKC_IMPL_AUTO;
    cudaStream_t stream     = nullptr;
    int         *dev_err    = nullptr; // device word; 0 = ok
    void        *scratch    = nullptr; // grown on demand: decode and prefill partials, boundary staging
    size_t       scratch_sz = 0;
    std::vector<void *> retired_scratch;      // outgrown blocks, kept until the context is destroyed (graphs may point at them)
    cudaStream_t scratch_user = nullptr;      // stream of the last launch that used the scratch
    cudaEvent_t  scratch_ev   = nullptr;
    cudaEvent_t  ev0 = nullptr, ev1 = nullptr;
    int64_t      launches = 0;
    bool         capturing = false;
    bool         dep_launch = true; // programmatic dependent launch between consecutive kernels (VKNN_PDL=0 turns it off)
    std::string  err;
    // driver entry point for tensor-map encoding (resolved once; no link-time dependency on libcuda)
    void *encode_tiled = nullptr;
    // kernels whose dynamic shared-memory limit has been raised on this context's device
    std::set<const void *> smem_configured;
};

struct vkc_graph {
    cudaGraph_t     graph = nullptr;
    cudaGraphExec_t exec  = nullptr;
};

inline int vkc_fail(vkc_ctx *ctx, int code, const char *fmt, ...) {
    char    buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->err = buf;
    return code;
}

#define VKC_CUDA(ctx, expr)                                                                                  \
    do {                                                                                                     \
        cudaError_t e_ = (expr);                                                                             \
        if (e_ != cudaSuccess) return vkc_fail(ctx, VKC_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

#define VKC_REQUIRE(ctx, cond, ...)                                  \
    do {                                                             \
        if (!(cond)) return vkc_fail(ctx, VKC_ERR_INVALID, __VA_ARGS__); \
    } while (0)

inline cudaStream_t vkc_pick_stream(vkc_ctx *ctx, vkc_stream s) { return s ? (cudaStream_t) s : ctx->stream; }

inline int vkc_post_launch(vkc_ctx *ctx, const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return vkc_fail(ctx, VKC_ERR_CUDA, "launch %s: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return VKC_OK;
}

// Launch with programmatic stream serialization — ONLY for kernels that execute vkc_grid_dep_wait(): the kernel may start (set up shared memory, barriers, tensor
// memory) while the previous kernel of the stream is still draining; it must execute griddepcontrol.wait
// (vkc_grid_dep_wait) before its first access to global memory, which returns once the previous kernel has completed
// and its writes are visible. Inside a stream capture the dependency becomes a programmatic graph edge.
// `cluster_x` > 1 launches thread-block clusters of that many consecutive CTAs along x.
template <typename... KArgs, typename... Args>
inline void vkc_launch_cluster(vkc_ctx *ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, unsigned cluster_x,
                               Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim            = grid;
    cfg.blockDim           = block;
    cfg.dynamicSmemBytes   = smem;
    cfg.stream             = st;
    cudaLaunchAttribute at[2];
    unsigned            n = 0;
    if (ctx->dep_launch) {
        at[n].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        at[n].id               = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = cluster_x;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs    = at;
    cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...); // errors surface in vkc_post_launch
}
template <typename... KArgs, typename... Args>
inline void vkc_launch(vkc_ctx *ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    vkc_launch_cluster(ctx, kern, grid, block, smem, st, 1u, std::forward<Args>(args)...);
}

#ifdef __CUDACC__
// Device side of the above. Both are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void vkc_grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void vkc_grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

inline size_t vkc_dtype_size(int dt) { return dt == VKC_F32 || dt == VKC_I32 ? 4 : 2; }

int vkc_ensure_scratch(vkc_ctx *ctx, size_t bytes, cudaStream_t st);

// Opt a kernel into more than 48 KB of dynamic shared memory, once per context (the attribute is per device).
template <typename Kernel> inline int vkc_configure_smem(vkc_ctx *ctx, Kernel kern, int bytes) {
    const void *key = reinterpret_cast<const void *>(kern);
    if (ctx->smem_configured.count(key)) return VKC_OK;
    VKC_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    ctx->smem_configured.insert(key);
    return VKC_OK;
}

// ---- storage-type traits ------------------------------------------------------------------------------------
template <typename T> struct St;
template <> struct St<float> {
    static __device__ __forceinline__ float ld(const float *p) { return *p; }
    static __device__ __forceinline__ void  st(float *p, float v) { *p = v; }
};
template <> struct St<__half> {
    static __device__ __forceinline__ float ld(const __half *p) { return __half2float(*p); }
    static __device__ __forceinline__ void  st(__half *p, float v) { *p = __float2half_rn(v); }
};
template <> struct St<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void  st(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};

// GELU in the exact operation order of the reference's node chain Div(sqrt2) -> Erf -> Add(1) -> Mul(h) -> Mul(0.5).
__device__ __forceinline__ float vkc_gelu_erf(float h) {
    float t = h / 1.41421356237f;
    t       = erff(t);
    t       = t + 1.0f;
    t       = t * h;
    return t * 0.5f;
}

// GELU for 16-bit storage: same operation order, with erf evaluated by the Abramowitz-Stegun 7.1.26 rational form
// (absolute error < 1.5e-7, far below half-precision output rounding). The reference's own device kernels evaluate
// Erf with this formula (shaders/common.glsl:44-50); fp32 storage keeps erff.
__device__ __forceinline__ float vkc_erf_as(float x) {
    const float ax = fabsf(x);
    const float t  = __fdividef(1.0f, fmaf(0.3275911f, ax, 1.0f));
    float       p  = fmaf(1.061405429f, t, -1.453152027f);
    p              = fmaf(p, t, 1.421413741f);
    p              = fmaf(p, t, -0.284496736f);
    p              = fmaf(p, t, 0.254829592f);
    const float e  = __expf(-ax * ax);
    const float r  = fmaf(-p * t, e, 1.0f);
    return copysignf(r, x);
}
__device__ __forceinline__ float vkc_gelu_erf_fast(float h) {
    float t = h * 0.70710678118f;
    t       = vkc_erf_as(t);
    t       = t + 1.0f;
    t       = t * h;
    return t * 0.5f;
}

#define VKC_DISPATCH_DTYPE(dtype, T, ...)                  \
    switch (dtype) {                                       \
        case VKC_F32: { using T = float; __VA_ARGS__; } break;         \
        case VKC_F16: { using T = __half; __VA_ARGS__; } break;        \
        case VKC_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
        default: break;                                    \
    }

// Output fan-out to several GPUs (device-side copy of vkc_fanout): a kernel stores each output row into dest[0..n_dest) and,
// when the grid's last block has stored, publishes this rank's count of completed fan-outs in flag[d] (a word in
// destination d's memory).
struct VkcFanDev {
    int       n_dest;
    void     *dest[8];
    unsigned *flag[8];
    unsigned *state; // [0] blocks that have stored, [1] fan-outs completed
    void     *mcast; // multicast mapping of the destinations' buffers, or null
};
#ifdef __CUDACC__
// One 16-byte store to every destination of a fan-out: through the multicast mapping (one multimem store, replicated by the
// NVSwitch) when there is one, else one peer store per destination. `off` in elements of T.
template <typename T> __device__ __forceinline__ void vkc_fanout_store16(const VkcFanDev &f, int64_t off, const uint4 &v) {
    if (f.mcast) {
        asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"((T *) f.mcast + off), "f"(__uint_as_float(v.x)),
                     "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                     : "memory");
    } else {
        for (int d = 0; d < f.n_dest; ++d) *reinterpret_cast<uint4 *>((T *) f.dest[d] + off) = v;
    }
}
// Called by every thread of a block after its last output store; `total` blocks take part. The stores of all blocks are
// ordered before the flag values by the barrier, the fences around the block counter and the release stores (the last block
// to arrive publishes).
__device__ __forceinline__ void vkc_fanout_signal(const VkcFanDev &f, unsigned total) {
    // The block's stores are ordered before thread 0's device-scope fence by the barrier, the blocks' fences before the last
    // block's system-scope fence by the counter, and that fence before the flag stores (fence + relaxed store = release): causality order is
    // transitive over the scopes, and only ONE system-scope fence runs per kernel (they serialise GPU-wide: one per block
    // cost 10 us per kernel).
    __syncthreads();
    if (threadIdx.x == 0 && f.state) {
        __threadfence();
        if (atomicAdd(f.state, 1u) == total - 1) {
            __threadfence_system();
            f.state[0]       = 0;
            const unsigned e = f.state[1] + 1;
            f.state[1]       = e;
            for (int d = 0; d < f.n_dest; ++d)
                if (f.flag[d]) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(f.flag[d]), "r"(e) : "memory"); // released by the fence above
        }
    }
}
#endif
#ifdef __CUDACC__
// Gate of a kernel whose input other GPUs produce (the consumer side of the fan-out above, folded into the consuming kernel
// instead of a separate wait kernel). ONE thread per CTA calls this before the CTA's first load of the gated data: it polls
// the `n` flag words (system-scope acquire loads) until each has reached state[0] + 1, for at most about half a second —
// shorter than the kernels' own barrier waits, so that a missing peer is reported as such. On expiry, or when the context's
// error word is already set, it records device error 3 and returns false; the caller then raises the CTA's abort flag so
// that the other roles leave through their bounded waits. The last of `total_ctas` callers advances state[0] (only when no
// error is pending, so that flags and count stay in step) and clears the caller counter state[1]. The cross-proxy fence
// orders the acquire before the CTA's bulk-tensor loads of what the peers wrote.
__device__ __forceinline__ bool vkc_gate_wait(const unsigned *flags, int n, unsigned *state, unsigned total_ctas, int *dev_err) {
    const unsigned  want = *reinterpret_cast<volatile unsigned *>(state) + 1;
    bool            ok   = *reinterpret_cast<volatile int *>(dev_err) == 0;
    const long long t0   = clock64();
    for (int f = 0; f < n && ok; ++f) {
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + f) : "memory");
            if ((int) (v - want) >= 0) break;
            if (clock64() - t0 > 1000000000LL) {
                ok = false;
                atomicCAS(dev_err, 0, 3);
                break;
            }
            __nanosleep(64);
        }
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");
    __threadfence();
    if (atomicAdd(state + 1, 1u) == total_ctas - 1) {
        state[1] = 0;
        if (ok && *reinterpret_cast<volatile int *>(dev_err) == 0) state[0] = want;
        __threadfence();
    }
    return ok;
}
#endif
// Validates a caller's fan-out description (destinations 16-byte aligned) and copies it; returns VKC_OK or fails the context.
inline int vkc_fan_to_dev(vkc_ctx *ctx, const vkc_fanout *fan, VkcFanDev *out, const char *who) {
    memset(out, 0, sizeof *out);
    if (!fan) return VKC_OK;
    if (fan->n_dest < 1 || fan->n_dest > 8 || !fan->state) return vkc_fail(ctx, VKC_ERR_INVALID, "%s: 1..8 destinations and a state buffer are required", who);
    out->n_dest = fan->n_dest;
    out->state  = fan->state;
    for (int d = 0; d < fan->n_dest; ++d) {
        if (!fan->dest[d] || ((uintptr_t) fan->dest[d] & 15)) return vkc_fail(ctx, VKC_ERR_INVALID, "%s: destination %d is null or not 16-byte aligned", who, d);
        out->dest[d] = fan->dest[d];
        out->flag[d] = fan->flag[d];
    }
    if (fan->mcast && ((uintptr_t) fan->mcast & 15)) return vkc_fail(ctx, VKC_ERR_INVALID, "%s: the multicast address is not 16-byte aligned", who);
    out->mcast = fan->mcast;
    return VKC_OK;
}
