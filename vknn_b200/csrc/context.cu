// Context, memory, boundary transfers, graph capture and timers of libvknn_cuda.
#include "common.cuh"
#include <climits>
#include <map>
#include <mutex>
#include <cstdlib>
#include "tensormap.cuh"

namespace {

    template <typename TS, typename TD> __global__ void convert_kernel(const TS *__restrict__ src, TD *__restrict__ dst, int64_t n) {
        int64_t i      = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        int64_t stride = (int64_t) gridDim.x * blockDim.x;
        for (; i < n; i += stride) St<TD>::st(dst + i, St<TS>::ld(src + i));
    }

    template <typename TS> int convert_from(vkc_ctx *ctx, const void *src, void *dst, int dst_dtype, int64_t n, cudaStream_t st) {
        int     threads = 256;
        int64_t blocks  = (n + threads - 1) / threads;
        int     cap     = ctx->sm_count * 16;
        int     grid    = (int) (blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
        switch (dst_dtype) {
            case VKC_F32: convert_kernel<TS, float><<<grid, threads, 0, st>>>((const TS *) src, (float *) dst, n); break;
            case VKC_F16: convert_kernel<TS, __half><<<grid, threads, 0, st>>>((const TS *) src, (__half *) dst, n); break;
            case VKC_BF16: convert_kernel<TS, __nv_bfloat16><<<grid, threads, 0, st>>>((const TS *) src, (__nv_bfloat16 *) dst, n); break;
            default: return vkc_fail(ctx, VKC_ERR_INVALID, "convert: bad dst dtype %d", dst_dtype);
        }
        return vkc_post_launch(ctx, "convert");
    }

} // namespace

// The context's scratch block only ever grows, and a block that has been handed out is never freed before the context is
// destroyed: its address may be baked into CUDA graphs the caller captured (key-range partials of prefill attention, decode
// partials, boundary staging), and those graphs must stay replayable after a later, larger call. A block that is outgrown is
// retired to a list that vkc_ctx_destroy frees. Growth is refused while `st` (or the context's own stream) is being
// captured, because an allocation is not a capturable operation: run the shape once outside the capture first.
// All users of the scratch are expected on one stream; when the using stream changes, the new stream is made to wait for
// everything enqueued so far on the previous one (not possible, and skipped, while either is being captured).
int vkc_ensure_scratch(vkc_ctx *ctx, size_t bytes, cudaStream_t st) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
        cudaGetLastError();
        cap = cudaStreamCaptureStatusActive; // the stream is in a broken capture: do nothing that could make it worse
    }
    const bool capturing = ctx->capturing || cap != cudaStreamCaptureStatusNone;
    if (bytes > ctx->scratch_sz) {
        if (capturing)
            return vkc_fail(ctx, VKC_ERR_INVALID, "context scratch cannot grow to %zu bytes during graph capture; run the shape once outside the capture first", bytes);
        size_t want = (bytes + ((size_t) 1 << 20) - 1) & ~(((size_t) 1 << 20) - 1);
        void  *blk  = nullptr;
        if (cudaMalloc(&blk, want) != cudaSuccess) {
            cudaGetLastError();
            return vkc_fail(ctx, VKC_ERR_OOM, "scratch allocation of %zu bytes failed", want);
        }
        if (ctx->scratch) ctx->retired_scratch.push_back(ctx->scratch); // still referenced by earlier launches and graphs
        ctx->scratch    = blk;
        ctx->scratch_sz = want;
    }
    if (ctx->scratch_user && ctx->scratch_user != st && !capturing) {
        cudaStreamCaptureStatus prev = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(ctx->scratch_user, &prev) == cudaSuccess && prev == cudaStreamCaptureStatusNone) {
            VKC_CUDA(ctx, cudaEventRecord(ctx->scratch_ev, ctx->scratch_user));
            VKC_CUDA(ctx, cudaStreamWaitEvent(st, ctx->scratch_ev, 0));
        } else {
            cudaGetLastError();
        }
    }
    if (!capturing) ctx->scratch_user = st;
    return VKC_OK;
}

extern "C" {

int vkc_device_count(int *count) {
    if (!count) return VKC_ERR_INVALID;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        *count = 0;
        return VKC_ERR_NO_DEVICE;
    }
    *count = n;
    return VKC_OK;
}

int vkc_ctx_create(int device_ordinal, vkc_ctx **out) {
    if (!out) return VKC_ERR_INVALID;
    *out  = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        return VKC_ERR_NO_DEVICE;
    }
    if (device_ordinal < 0 || device_ordinal >= n) return VKC_ERR_INVALID;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) return VKC_ERR_CUDA;
    if (prop.major != 10) return VKC_ERR_NO_DEVICE; // kernels are built for sm_100a only
    vkc_ctx *ctx  = new vkc_ctx();
    ctx->device   = device_ordinal;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->l2_bytes = (size_t) prop.l2CacheSize;
    if (const char *e = getenv("VKNN_PDL")) ctx->dep_launch = atoi(e) != 0;
    ctx->cc_major = prop.major;
    if (cudaSetDevice(device_ordinal) != cudaSuccess || cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(&ctx->dev_err, sizeof(int)) != cudaSuccess || cudaMemset(ctx->dev_err, 0, sizeof(int)) != cudaSuccess ||
        cudaEventCreate(&ctx->ev0) != cudaSuccess || cudaEventCreate(&ctx->ev1) != cudaSuccess ||
        cudaEventCreateWithFlags(&ctx->scratch_ev, cudaEventDisableTiming) != cudaSuccess) {
        delete ctx;
        return VKC_ERR_CUDA;
    }
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->encode_tiled, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
        ctx->encode_tiled = nullptr; // tcgen05 paths report an error when asked; SIMT paths still work
        cudaGetLastError();
    }
    *out = ctx;
    return VKC_OK;
}

int vkc_ctx_destroy(vkc_ctx *ctx) {
    if (!ctx) return VKC_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    for (void *blk : ctx->retired_scratch) cudaFree(blk);
    if (ctx->scratch_ev) cudaEventDestroy(ctx->scratch_ev);
    if (ctx->dev_err) cudaFree(ctx->dev_err);
    if (ctx->ev0) cudaEventDestroy(ctx->ev0);
    if (ctx->ev1) cudaEventDestroy(ctx->ev1);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return VKC_OK;
}

int vkc_device_info(const vkc_ctx *ctx, char *name, size_t name_cap, int *sm_count, int *sm_clock_mhz) {
    if (!ctx) return VKC_ERR_INVALID;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ctx->device) != cudaSuccess) {
        cudaGetLastError();
        return VKC_ERR_CUDA;
    }
    if (name && name_cap) snprintf(name, name_cap, "%s", prop.name);
    if (sm_count) *sm_count = prop.multiProcessorCount;
    if (sm_clock_mhz) {
        int khz = 0;
        if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device) != cudaSuccess) cudaGetLastError();
        *sm_clock_mhz = khz / 1000;
    }
    return VKC_OK;
}

const char *vkc_last_error(const vkc_ctx *ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int vkc_ctx_set_impl(vkc_ctx *ctx, int impl) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, impl >= VKC_IMPL_AUTO && impl <= VKC_IMPL_TCGEN05, "bad impl %d", impl);
    ctx->impl = impl;
    return VKC_OK;
}

int vkc_sync(vkc_ctx *ctx, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    VKC_CUDA(ctx, cudaStreamSynchronize(st));
    int code = 0;
    VKC_CUDA(ctx, cudaMemcpy(&code, ctx->dev_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (code != 0) {
        cudaMemset(ctx->dev_err, 0, sizeof(int));
        return vkc_fail(ctx, VKC_ERR_DEVICE, "device-side error word %d (1 = bounded wait ran out, 2 = tensor-memory allocation, 3 = a peer's flag did not arrive)", code);
    }
    return VKC_OK;
}

int64_t vkc_launch_count(const vkc_ctx *ctx) { return ctx ? ctx->launches : 0; }

int vkc_alloc(vkc_ctx *ctx, size_t bytes, void **dptr) {
    if (!ctx || !dptr) return VKC_ERR_INVALID;
    *dptr = nullptr;
    if (bytes == 0) return VKC_OK;
    if (cudaMalloc(dptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        return vkc_fail(ctx, VKC_ERR_OOM, "cudaMalloc(%zu) failed", bytes);
    }
    return VKC_OK;
}

int vkc_free(vkc_ctx *ctx, void *dptr) {
    if (!ctx) return VKC_ERR_INVALID;
    if (dptr) VKC_CUDA(ctx, cudaFree(dptr));
    return VKC_OK;
}

int vkc_convert(vkc_ctx *ctx, void *dst, int dst_dtype, const void *src, int src_dtype, int64_t n, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, n >= 0 && (n == 0 || (dst && src)), "convert: null buffer");
    if (n == 0) return VKC_OK;
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    if (src_dtype == dst_dtype) {
        VKC_CUDA(ctx, cudaMemcpyAsync(dst, src, (size_t) n * vkc_dtype_size(src_dtype), cudaMemcpyDeviceToDevice, st));
        return VKC_OK;
    }
    switch (src_dtype) {
        case VKC_F32: return convert_from<float>(ctx, src, dst, dst_dtype, n, st);
        case VKC_F16: return convert_from<__half>(ctx, src, dst, dst_dtype, n, st);
        case VKC_BF16: return convert_from<__nv_bfloat16>(ctx, src, dst, dst_dtype, n, st);
        default: return vkc_fail(ctx, VKC_ERR_INVALID, "convert: bad src dtype %d", src_dtype);
    }
}

// ---- registry of caller-owned device buffers used as segment inputs / outputs ------------------------------------
namespace {
    struct ExtBuf {
        void  *ptr;
        size_t bytes;
    };
    std::mutex            g_ext_mu;
    std::map<int, ExtBuf> g_ext;
    int                   g_ext_next = 0x40000000;
} // namespace

int vkc_extbuf_register(void *dptr, size_t bytes, int *handle) {
    if (!dptr || !handle || bytes == 0) return VKC_ERR_INVALID;
    std::lock_guard<std::mutex> lk(g_ext_mu);
    if (g_ext_next == INT32_MAX) return VKC_ERR_INVALID;
    *handle        = g_ext_next++;
    g_ext[*handle] = {dptr, bytes};
    return VKC_OK;
}
int vkc_extbuf_unregister(int handle) {
    std::lock_guard<std::mutex> lk(g_ext_mu);
    return g_ext.erase(handle) ? VKC_OK : VKC_ERR_INVALID;
}
int vkc_extbuf_lookup(int handle, void **dptr, size_t *bytes) {
    std::lock_guard<std::mutex> lk(g_ext_mu);
    auto                        it = g_ext.find(handle);
    if (it == g_ext.end()) return VKC_ERR_INVALID;
    if (dptr) *dptr = it->second.ptr;
    if (bytes) *bytes = it->second.bytes;
    return VKC_OK;
}

int vkc_upload(vkc_ctx *ctx, void *dst_dev, int dst_dtype, const void *src_host, int src_dtype, int64_t n, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, n >= 0 && (n == 0 || (dst_dev && src_host)), "upload: null buffer");
    if (n == 0) return VKC_OK;
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    if (src_dtype == dst_dtype) {
        VKC_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, (size_t) n * vkc_dtype_size(src_dtype), cudaMemcpyHostToDevice, st));
        return VKC_OK;
    }
    // stage in the source type on the device, then convert there (the reference converts on the host)
    size_t bytes = (size_t) n * vkc_dtype_size(src_dtype);
    int    rc    = vkc_ensure_scratch(ctx, bytes, st);
    if (rc) return rc;
    VKC_CUDA(ctx, cudaMemcpyAsync(ctx->scratch, src_host, bytes, cudaMemcpyHostToDevice, st));
    return vkc_convert(ctx, dst_dev, dst_dtype, ctx->scratch, src_dtype, n, stream);
}

int vkc_download(vkc_ctx *ctx, void *dst_host, int dst_dtype, const void *src_dev, int src_dtype, int64_t n, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, n >= 0 && (n == 0 || (dst_host && src_dev)), "download: null buffer");
    if (n == 0) return VKC_OK;
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    if (src_dtype == dst_dtype) {
        VKC_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, (size_t) n * vkc_dtype_size(src_dtype), cudaMemcpyDeviceToHost, st));
        return VKC_OK;
    }
    size_t bytes = (size_t) n * vkc_dtype_size(dst_dtype);
    int    rc    = vkc_ensure_scratch(ctx, bytes, st);
    if (rc) return rc;
    rc = vkc_convert(ctx, ctx->scratch, dst_dtype, src_dev, src_dtype, n, stream);
    if (rc) return rc;
    VKC_CUDA(ctx, cudaMemcpyAsync(dst_host, ctx->scratch, bytes, cudaMemcpyDeviceToHost, st));
    return VKC_OK;
}

int vkc_graph_begin(vkc_ctx *ctx) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, !ctx->capturing, "graph capture already active");
    VKC_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    return VKC_OK;
}

int vkc_graph_end(vkc_ctx *ctx, vkc_graph **out) {
    if (!ctx || !out) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, ctx->capturing, "no graph capture active");
    ctx->capturing = false;
    cudaGraph_t g  = nullptr;
    VKC_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &g));
    cudaGraphExec_t ex = nullptr;
    cudaError_t     e  = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        return vkc_fail(ctx, VKC_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    }
    vkc_graph *vg = new vkc_graph();
    vg->graph     = g;
    vg->exec      = ex;
    *out          = vg;
    return VKC_OK;
}

int vkc_graph_launch(vkc_ctx *ctx, vkc_graph *g) {
    if (!ctx || !g) return VKC_ERR_INVALID;
    VKC_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    return VKC_OK;
}

int vkc_graph_destroy(vkc_ctx *ctx, vkc_graph *g) {
    if (!g) return VKC_OK;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    (void) ctx;
    return VKC_OK;
}

int vkc_timer_start(vkc_ctx *ctx, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_CUDA(ctx, cudaEventRecord(ctx->ev0, vkc_pick_stream(ctx, stream)));
    return VKC_OK;
}

int vkc_timer_stop(vkc_ctx *ctx, vkc_stream stream, float *ms) {
    if (!ctx || !ms) return VKC_ERR_INVALID;
    VKC_CUDA(ctx, cudaEventRecord(ctx->ev1, vkc_pick_stream(ctx, stream)));
    VKC_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    VKC_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
    return VKC_OK;
}

} // extern "C"

// ---------------------------------------------------------------------------------------------------------------------
// Peer memory: buffers shared between the processes of one node, and the bounded wait on flags that peers write.
namespace {
    // One warp; lane i polls flag i. A context whose device error word is already set (an earlier wait ran out, a peer is gone)
    // returns at once instead of spinning through its own limit again, and the expected count only advances when every flag
    // arrived, so that flags and count stay in step for a retry.
    __global__ void peer_wait_kernel(const uint32_t *flags, int n, uint32_t *expected, int *dev_err) {
        const uint32_t want = *expected + 1;
        bool           ok   = *reinterpret_cast<volatile int *>(dev_err) == 0;
        if (ok && (int) threadIdx.x < n) {
            const long long t0 = clock64();
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
                if ((int32_t) (v - want) >= 0) break;
                if (clock64() - t0 > 4000000000LL) { // about two seconds: the peer is not coming
                    ok = false;
                    atomicCAS(dev_err, 0, 3);
                    break;
                }
                __nanosleep(200);
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok && threadIdx.x == 0) *expected = want;
    }
} // namespace

extern "C" int vkc_peer_wait(vkc_ctx *ctx, const uint32_t *flags, int n, uint32_t *expected, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, flags && expected && n >= 1 && n <= 32, "peer_wait: 1..32 flags and an expected-count word are required");
    peer_wait_kernel<<<1, 32, 0, vkc_pick_stream(ctx, stream)>>>(flags, n, expected, ctx->dev_err);
    return vkc_post_launch(ctx, "peer_wait");
}

extern "C" int vkc_peer_export(vkc_ctx *ctx, void *dptr, unsigned char *handle) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, dptr && handle, "peer_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == VKC_PEER_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    VKC_CUDA(ctx, cudaIpcGetMemHandle(&h, dptr));
    memcpy(handle, &h, sizeof h);
    return VKC_OK;
}

extern "C" int vkc_peer_open(vkc_ctx *ctx, const unsigned char *handle, void **dptr) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, dptr && handle, "peer_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    *dptr = nullptr;
    VKC_CUDA(ctx, cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess));
    return VKC_OK;
}

extern "C" int vkc_peer_close(vkc_ctx *ctx, void *dptr) {
    if (!ctx) return VKC_ERR_INVALID;
    if (dptr) VKC_CUDA(ctx, cudaIpcCloseMemHandle(dptr));
    return VKC_OK;
}
