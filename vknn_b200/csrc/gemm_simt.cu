// K1 (SIMT form) — batched GEMM on the fp32 FMA pipes. This is the Precision::High (fp32 storage) kernel,
// where tensor-core formats would break the rel <= 1e-4 bound against the scalar CPU reference, and the kernel
// for operands that do not meet the TMA alignment rules (odd leading dimensions such as P[.,197]).
// Accumulation runs over k ascending in fp32, like the reference's inner loop.
#include "common.cuh"

int vkc_gemm_tcgen05(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                     int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                     int b_layout, int epilogue, int dtype, int config, const vkc_gate *gate, cudaStream_t st);

namespace {

    constexpr int TM = 64, TN = 64, TK = 16;

    template <typename T, bool B_KN>
    __global__ void __launch_bounds__(256) gemm_simt_kernel(const T *__restrict__ A, const T *__restrict__ B, const float *__restrict__ bias,
                                                            const T *__restrict__ residual, T *__restrict__ D, int64_t M, int64_t N, int64_t K,
                                                            int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb,
                                                            int64_t ldd, int epilogue) {
        __shared__ float As[TK][TM + 1];
        __shared__ float Bs[TK][TN + 1];
        const int     tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
        const int64_t m0 = (int64_t) blockIdx.y * TM, n0 = (int64_t) blockIdx.x * TN;
        const T      *Ab = A + (int64_t) blockIdx.z * stride_a;
        const T      *Bb = B + (int64_t) blockIdx.z * stride_b;
        float         acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

        for (int64_t k0 = 0; k0 < K; k0 += TK) {
            // A tile: 64 x 16, k fastest across threads
            for (int i = threadIdx.x; i < TM * TK; i += 256) {
                const int     mm = i / TK, kk = i % TK;
                const int64_t m = m0 + mm, k = k0 + kk;
                As[kk][mm] = (m < M && k < K) ? St<T>::ld(Ab + m * lda + k) : 0.f;
            }
            for (int i = threadIdx.x; i < TN * TK; i += 256) {
                int nn, kk;
                if (B_KN) {
                    kk = i / TN;
                    nn = i % TN;
                } else {
                    nn = i / TK;
                    kk = i % TK;
                }
                const int64_t n = n0 + nn, k = k0 + kk;
                float         v = 0.f;
                if (n < N && k < K) v = B_KN ? St<T>::ld(Bb + k * ldb + n) : St<T>::ld(Bb + n * ldb + k);
                Bs[kk][nn] = v;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < TK; ++kk) {
                float a[4], b[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            __syncthreads();
        }
        T       *Db = D + (int64_t) blockIdx.z * stride_d;
        const T *Rb = residual ? residual + (int64_t) blockIdx.z * stride_d : nullptr;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t m = m0 + ty * 4 + i;
            if (m >= M) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t n = n0 + tx * 4 + j;
                if (n >= N) continue;
                float v = acc[i][j];
                if (epilogue & VKC_EPI_BIAS) v += bias[n];
                if (epilogue & VKC_EPI_GELU_ERF) v = vkc_gelu_erf(v);
                if (epilogue & VKC_EPI_RESIDUAL) v += St<T>::ld(Rb + m * ldd + n);
                St<T>::st(Db + m * ldd + n, v);
            }
        }
    }

    template <typename T>
    int launch_simt(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N, int64_t K,
                    int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd, int b_layout,
                    int epilogue, cudaStream_t st) {
        dim3 grid((unsigned) ((N + TN - 1) / TN), (unsigned) ((M + TM - 1) / TM), (unsigned) batch);
        if (b_layout == VKC_B_KN)
            gemm_simt_kernel<T, true><<<grid, 256, 0, st>>>((const T *) A, (const T *) B, bias, (const T *) residual, (T *) D, M, N, K, stride_a,
                                                           stride_b, stride_d, lda, ldb, ldd, epilogue);
        else
            gemm_simt_kernel<T, false><<<grid, 256, 0, st>>>((const T *) A, (const T *) B, bias, (const T *) residual, (T *) D, M, N, K, stride_a,
                                                            stride_b, stride_d, lda, ldb, ldd, epilogue);
        return vkc_post_launch(ctx, "gemm_simt");
    }

} // namespace

extern "C" int vkc_gemm(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                        int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                        int b_layout, int epilogue, int dtype, vkc_stream stream) {
    return vkc_gemm_ex(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout, epilogue, dtype, -1, stream);
}

static int gemm_dispatch(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                           int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                           int b_layout, int epilogue, int dtype, int config, const vkc_gate *gate, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, config >= -1 && config < vkc_gemm_config_count(), "gemm: bad configuration index %d", config);
    VKC_REQUIRE(ctx, M >= 0 && N >= 0 && K >= 0 && batch >= 0, "gemm: negative extent");
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "gemm: bad dtype %d", dtype);
    VKC_REQUIRE(ctx, b_layout == VKC_B_KN || b_layout == VKC_B_NK, "gemm: bad b_layout %d", b_layout);
    VKC_REQUIRE(ctx, (epilogue & ~7) == 0, "gemm: bad epilogue mask %d", epilogue);
    if (M == 0 || N == 0 || batch == 0) return VKC_OK;
    VKC_REQUIRE(ctx, A && B && D, "gemm: null operand");
    VKC_REQUIRE(ctx, !(epilogue & VKC_EPI_BIAS) || bias, "gemm: bias epilogue without a bias pointer");
    VKC_REQUIRE(ctx, !(epilogue & VKC_EPI_RESIDUAL) || residual, "gemm: residual epilogue without a residual pointer");
    VKC_REQUIRE(ctx, lda >= K && ldd >= N && ldb >= (b_layout == VKC_B_KN ? N : K), "gemm: leading dimension smaller than the row");
    VKC_REQUIRE(ctx, batch <= 65535 && (M + TM - 1) / TM <= 65535, "gemm: grid too large");
    cudaStream_t st = vkc_pick_stream(ctx, stream);

    bool want_tc = dtype != VKC_F32 && ctx->impl != VKC_IMPL_SIMT && K > 0;
    if (ctx->impl == VKC_IMPL_AUTO) want_tc = want_tc && M >= 32 && N >= 32 && K >= 32; // the reference's tiled-path rule (ops/matmul.cpp:141)
    if (want_tc) {
        int rc = vkc_gemm_tcgen05(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout, epilogue,
                                  dtype, config, gate, st);
        if (rc != VKC_ERR_UNSUPPORTED || ctx->impl == VKC_IMPL_TCGEN05 || config >= 0) return rc;
    } else if (config >= 0) {
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm: a tensor-core configuration was requested for a problem the tensor-core kernel does not take");
    }
    if (gate) { // the fp32-pipe kernel has no gate of its own: a one-warp wait kernel in front of it
        int rc = vkc_peer_wait(ctx, gate->flags, gate->n, gate->state, stream);
        if (rc) return rc;
    }
    switch (dtype) {
        case VKC_F32:
            return launch_simt<float>(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout, epilogue, st);
        case VKC_F16:
            return launch_simt<__half>(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout, epilogue, st);
        default:
            return launch_simt<__nv_bfloat16>(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout,
                                              epilogue, st);
    }
}

extern "C" int vkc_gemm_ex(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                           int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                           int b_layout, int epilogue, int dtype, int config, vkc_stream stream) {
    return gemm_dispatch(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout, epilogue, dtype, config,
                         nullptr, stream);
}

extern "C" int vkc_gemm_gated(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                              int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                              int b_layout, int epilogue, int dtype, int config, const vkc_gate *gate, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, gate && gate->flags && gate->state && gate->n >= 1 && gate->n <= 32, "gemm_gated: a gate with 1..32 flags and a state buffer is required");
    return gemm_dispatch(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout, epilogue, dtype, config, gate,
                         stream);
}
