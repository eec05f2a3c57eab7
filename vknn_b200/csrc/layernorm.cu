// K4 — LayerNorm over the trailing `norm` elements, HBM-bound: one warp per row, 128-bit loads, the row held in
// registers between the two statistics passes (mean first, then the centred second moment, the same two-pass
// form as the CPU reference) and the normalise/scale/shift pass, warp-shuffle reductions only. Each row is
// read once and written once: algorithmic bytes = rows * norm * 2 * sizeof(T) + 8 * norm.
#include "common.cuh"
#include <algorithm>

namespace {

    template <typename T> struct Vec16 {
        static constexpr int N = 16 / sizeof(T);
    };

    __device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        return v;
    }

    // CHUNKS = 16-byte vectors per lane; covers norm <= 32 * CHUNKS * (16/sizeof(T)). Warps are persistent: each
    // walks rows warp_id, warp_id + total_warps, ... with its slice of gamma / beta held in registers for the whole
    // kernel, so the only memory instructions per row are the 128-bit loads of x and stores of y. For 16-bit
    // storage the next row's loads are issued before the current row is reduced (more bytes in flight per SM).
    template <typename T, int CHUNKS>
    __global__ void __launch_bounds__(256, 2) layernorm_kernel(const T *__restrict__ X, const float *__restrict__ gamma,
                                                               const float *__restrict__ beta, T *__restrict__ Y, int64_t rows, int norm, float eps,
                                                               const VkcFanDev fan) {
        constexpr int  VN       = Vec16<T>::N;
        constexpr bool PREFETCH = sizeof(T) == 2;
        const int      lane     = threadIdx.x & 31;
        const int64_t  nwarps   = (int64_t) gridDim.x * (blockDim.x >> 5);
        int64_t        row      = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        if (row >= rows && fan.n_dest == 0) return;
        vkc_grid_dep_wait();
        vkc_grid_dep_launch();
        if (row < rows) {

        float g[CHUNKS][VN], bt[CHUNKS][VN];
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int e = (c * 32 + lane) * VN;
#pragma unroll
            for (int j = 0; j < VN; j += 4) {
                float4 gv = make_float4(0.f, 0.f, 0.f, 0.f), bv = gv;
                if (e < norm) {
                    gv = __ldg(reinterpret_cast<const float4 *>(gamma + e + j));
                    if (beta) bv = __ldg(reinterpret_cast<const float4 *>(beta + e + j));
                }
                g[c][j] = gv.x, g[c][j + 1] = gv.y, g[c][j + 2] = gv.z, g[c][j + 3] = gv.w;
                bt[c][j] = bv.x, bt[c][j + 1] = bv.y, bt[c][j + 2] = bv.z, bt[c][j + 3] = bv.w;
            }
        }
        auto load_row = [&](int64_t r, uint4(&raw)[CHUNKS]) {
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const int e = (c * 32 + lane) * VN;
                raw[c]      = (e < norm && r < rows) ? *reinterpret_cast<const uint4 *>(X + r * norm + e) : make_uint4(0, 0, 0, 0);
            }
        };
        uint4 cur[CHUNKS], nxt[CHUNKS];
        load_row(row, cur);
        for (; row < rows; row += nwarps) {
            if (PREFETCH) load_row(row + nwarps, nxt);
            float v[CHUNKS][VN];
            float s = 0.f;
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const T *t = reinterpret_cast<const T *>(&cur[c]);
#pragma unroll
                for (int j = 0; j < VN; ++j) {
                    v[c][j] = St<T>::ld(t + j);
                    s += v[c][j];
                }
            }
            const float mean = warp_sum(s) / (float) norm;
            float       q    = 0.f;
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const int e = (c * 32 + lane) * VN;
                if (e < norm) {
#pragma unroll
                    for (int j = 0; j < VN; ++j) {
                        const float d = v[c][j] - mean;
                        q += d * d;
                    }
                }
            }
            const float var = warp_sum(q) / (float) norm;
            const float inv = 1.0f / sqrtf(var + eps);
            T          *yr  = Y + row * norm;
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                const int e = (c * 32 + lane) * VN;
                if (e < norm) {
                    uint4 out;
                    T    *t = reinterpret_cast<T *>(&out);
#pragma unroll
                    for (int j = 0; j < VN; ++j) {
                        float o = (v[c][j] - mean) * inv * g[c][j];
                        if (beta) o += bt[c][j];
                        St<T>::st(t + j, o);
                    }
                    if (fan.n_dest == 0) {
                        *reinterpret_cast<uint4 *>(yr + e) = out;
                    } else { // the row goes to every destination (this GPU's and the peers' buffers)
                        vkc_fanout_store16<T>(fan, row * norm + e, out);
                    }
                }
            }
            if (PREFETCH) {
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) cur[c] = nxt[c];
            } else {
                load_row(row + nwarps, cur);
            }
        }
        }
        if (fan.n_dest > 0) vkc_fanout_signal(fan, gridDim.x); // every thread of the block, warps without a row included
    }

    // Any norm / alignment: one warp per row, three passes over global memory (rows stay L1/L2 resident).
    template <typename T>
    __global__ void __launch_bounds__(256) layernorm_generic_kernel(const T *__restrict__ X, const float *__restrict__ gamma,
                                                                    const float *__restrict__ beta, T *__restrict__ Y, int64_t rows, int64_t norm,
                                                                    float eps) {
        const int     lane = threadIdx.x & 31;
        const int64_t row  = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        if (row >= rows) return;
        vkc_grid_dep_wait();
        vkc_grid_dep_launch();
        const T *xr = X + row * norm;
        T       *yr = Y + row * norm;
        float    s  = 0.f;
        for (int64_t j = lane; j < norm; j += 32) s += St<T>::ld(xr + j);
        const float mean = warp_sum(s) / (float) norm;
        float       q    = 0.f;
        for (int64_t j = lane; j < norm; j += 32) {
            const float d = St<T>::ld(xr + j) - mean;
            q += d * d;
        }
        const float inv = 1.0f / sqrtf(warp_sum(q) / (float) norm + eps);
        for (int64_t j = lane; j < norm; j += 32) {
            float o = (St<T>::ld(xr + j) - mean) * inv * gamma[j];
            if (beta) o += beta[j];
            St<T>::st(yr + j, o);
        }
    }

    template <typename T>
    int launch_ln(vkc_ctx *ctx, const void *X, const float *gamma, const float *beta, void *Y, int64_t rows, int64_t norm, float eps, cudaStream_t st,
                  const VkcFanDev &fan) {
        constexpr int VN      = Vec16<T>::N;
        const int     wpb     = 8; // warps (= rows) per block
        const int64_t blocks  = (rows + wpb - 1) / wpb;
        const int64_t pblocks = std::min<int64_t>(blocks, (int64_t) ctx->sm_count * 2); // persistent warps: two 256-thread blocks per SM
        if (fan.n_dest > 0) Y = fan.dest[0];
        const bool    aligned = (norm % VN == 0) && (((uintptr_t) X & 15) == 0) && (((uintptr_t) Y & 15) == 0) && (((uintptr_t) gamma & 15) == 0) &&
                                (!beta || ((uintptr_t) beta & 15) == 0);
        const int64_t chunks  = (norm + 32 * VN - 1) / (32 * VN);
        if (blocks > INT32_MAX) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "layernorm: too many rows");
#define VKC_LN(C) vkc_launch(ctx, layernorm_kernel<T, C>, dim3((unsigned) pblocks), dim3(wpb * 32), 0, st, (const T *) X, gamma, beta, (T *) Y, rows, (int) norm, eps, fan)
        if (aligned && chunks <= 8) {
            switch (chunks) {
                case 1: VKC_LN(1); break;
                case 2: VKC_LN(2); break;
                case 3: VKC_LN(3); break;
                case 4: VKC_LN(4); break;
                case 5: VKC_LN(5); break;
                case 6: VKC_LN(6); break;
                case 7: VKC_LN(7); break;
                default: VKC_LN(8); break;
            }
        } else if (fan.n_dest > 0) {
            return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "layernorm_fanout: needs 16-byte aligned rows of at most %d elements", 8 * 32 * VN);
        } else {
            vkc_launch(ctx, layernorm_generic_kernel<T>, dim3((unsigned) blocks), dim3(wpb * 32), 0, st, (const T *) X, gamma, beta, (T *) Y, rows, norm, eps);
        }
#undef VKC_LN
        return vkc_post_launch(ctx, "layernorm");
    }

} // namespace

extern "C" int vkc_layernorm(vkc_ctx *ctx, const void *X, const float *gamma, const float *beta, void *Y, int64_t rows, int64_t norm, float eps,
                             int dtype, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, rows >= 0 && norm >= 1, "layernorm: bad extents rows=%lld norm=%lld", (long long) rows, (long long) norm);
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "layernorm: bad dtype %d", dtype);
    if (rows == 0) return VKC_OK;
    VKC_REQUIRE(ctx, X && Y && gamma, "layernorm: null operand");
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    VkcFanDev    fd;
    memset(&fd, 0, sizeof fd);
    switch (dtype) {
        case VKC_F32: return launch_ln<float>(ctx, X, gamma, beta, Y, rows, norm, eps, st, fd);
        case VKC_F16: return launch_ln<__half>(ctx, X, gamma, beta, Y, rows, norm, eps, st, fd);
        default: return launch_ln<__nv_bfloat16>(ctx, X, gamma, beta, Y, rows, norm, eps, st, fd);
    }
}

extern "C" int vkc_layernorm_fanout(vkc_ctx *ctx, const void *X, const float *gamma, const float *beta, int64_t rows, int64_t norm, float eps,
                                    int dtype, const vkc_fanout *fan, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, rows >= 1 && norm >= 1, "layernorm_fanout: bad extents rows=%lld norm=%lld", (long long) rows, (long long) norm);
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "layernorm_fanout: bad dtype %d", dtype);
    VKC_REQUIRE(ctx, X && gamma && fan, "layernorm_fanout: null operand");
    VkcFanDev fd;
    if (int rc = vkc_fan_to_dev(ctx, fan, &fd, "layernorm_fanout")) return rc;
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    switch (dtype) {
        case VKC_F32: return launch_ln<float>(ctx, X, gamma, beta, nullptr, rows, norm, eps, st, fd);
        case VKC_F16: return launch_ln<__half>(ctx, X, gamma, beta, nullptr, rows, norm, eps, st, fd);
        default: return launch_ln<__nv_bfloat16>(ctx, X, gamma, beta, nullptr, rows, norm, eps, st, fd);
    }
}
