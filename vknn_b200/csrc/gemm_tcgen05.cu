// K1 — batched GEMM on the 5th-generation tensor cores with a fused bias / GELU(erf) / residual epilogue.
//
//   D[b,m,n] = epi( sum_k A[b,m,k] * B[b,k,n] ),  A/B/D in f16 or bf16, fp32 accumulation in tensor memory.
//
// One CTA computes one 128 x BN output tile (BN in {64, 128, 192, 256}, chosen per problem to fill the 148 SMs in
// as few waves as possible). Small and medium problems run two CTAs per SM so that one CTA's epilogue overlaps the
// other's main loop. Warp roles:
//   warp 0   : TMA producer  — one elected lane streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle)
//              through a multi-stage shared-memory ring, completion on per-stage "full" mbarriers;
//   warp 1   : MMA issuer    — owns the tensor-memory allocation; one elected lane issues four
//              tcgen05.mma (M=128, N=BN, K=16) per stage and commits the stage's "empty" mbarrier;
//   warps 2-5: epilogue      — each warp owns the 32 TMEM lanes (= output rows) it may address, reads the
//              accumulator with tcgen05.ld in 32-column slabs, applies the epilogue in fp32 and stores.
// B is taken either as [N,K] rows (K contiguous, "K-major") or as [K,N] rows (N contiguous, "MN-major"),
// so weights in the reference's row-major [K,N] initializer layout are consumed without a transpose.
// M/N/K tails rely on TMA zero fill for loads and on predicated stores.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"
#include <cmath>
#include <cstdlib>

int vkc_gemm_tcgen05_pair(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                          int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                          int b_layout, int epilogue, int dtype, int bn, cudaStream_t st);

namespace {

    constexpr int BM       = 128;
    constexpr int BK       = 64;
    constexpr int kThreads = 192;

    struct GemmParams {
        const float *bias;
        const void  *residual;
        void        *D;
        int64_t      M, N, K;
        int64_t      ldd, stride_d;
        int          epilogue;
        int          a_bcast, b_bcast; // batch stride 0: always read batch slice 0
        int         *dev_err;
        long long   *timeline; // optional clock64 stamps of CTA (0,0,0)
        int          tma_out;  // D (and the residual) meet the TMA alignment rules: staged, coalesced epilogue
    };

    // GELU(erf) on two values at once with packed fp32 arithmetic and no special-function unit: erf(x), x = h/sqrt(2)
    // clamped to [-3, 3] (erf(3) = 1 - 2.2e-5), is x * P(x^2) with a degree-8 polynomial fitted to |error| < 2.1e-5,
    // so GELU is within 5e-5 of the erff form everywhere, far below the rounding of the 16-bit output. The operation
    // order of the reference chain (erf, +1, *h, *0.5) is kept.
    __device__ __forceinline__ float2 gelu_erf_pair(float2 h) {
        const float2 k = make_float2(0.70710678118f, 0.70710678118f);
        float2       x = ptx::fmul2(h, k);
        x.x            = fminf(fmaxf(x.x, -3.0f), 3.0f);
        x.y            = fminf(fmaxf(x.y, -3.0f), 3.0f);
        const float2 u = ptx::fmul2(x, x);
        auto         c = [](float v) { return make_float2(v, v); };
        float2       p = c(3.912539981e-08f);
        p              = ptx::ffma2(p, u, c(-1.883036475e-06f));
        p              = ptx::ffma2(p, u, c(4.008835822e-05f));
        p              = ptx::ffma2(p, u, c(-5.029218737e-04f));
        p              = ptx::ffma2(p, u, c(4.196857568e-03f));
        p              = ptx::ffma2(p, u, c(-2.499890141e-02f));
        p              = ptx::ffma2(p, u, c(1.109308004e-01f));
        p              = ptx::ffma2(p, u, c(-3.752196431e-01f));
        p              = ptx::ffma2(p, u, c(1.128250599e+00f));
        float2 t       = ptx::ffma2(p, x, c(1.0f)); // erf + 1
        t              = ptx::fmul2(t, h);
        return ptx::fmul2(t, c(0.5f));
    }

    template <int BN, int kStages> constexpr int smem_bytes() {
        return kStages * (BM * BK * 2 + BN * BK * 2) + 1024 /*align*/ + 256 /*barriers*/ + BN * 4 /*bias*/;
    }
    __host__ __device__ constexpr int tmem_cols(int bn) { return bn <= 32 ? 32 : bn <= 64 ? 64 : bn <= 128 ? 128 : 256; } // power of two >= BN

    template <int BN, int kStages, int kCtasPerSm, typename T, bool B_KN>
    __global__ void __launch_bounds__(kThreads, kCtasPerSm)
        gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmD,
                            const __grid_constant__ CUtensorMap tmR, GemmParams p) {
        static_assert((BN / 64 + (BN % 64 != 0)) * 16384 <= kStages * (BM * BK * 2 + BN * BK * 2), "epilogue staging must fit in the operand ring");
        constexpr uint32_t A_BYTES = BM * BK * 2;
        constexpr uint32_t B_BYTES = BN * BK * 2;
        constexpr bool     kBf16   = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdesc  = ptx::idesc_f16(BM, BN, kBf16, false, B_KN);

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sA    = base;
        const uint32_t sB    = base + kStages * A_BYTES;
        const uint32_t sBar  = sB + kStages * B_BYTES; // full[kStages], empty[kStages], accum : 8 bytes each
        volatile int  *ctl   = (volatile int *) (gbase + kStages * (A_BYTES + B_BYTES) + 8 * (2 * kStages + 1));
        // ctl[0] = tmem base (written by tcgen05.alloc), ctl[1] = abort flag
        const uint32_t sSlot = sBar + 8 * (2 * kStages + 1);
        float         *sbias = (float *) (gbase + kStages * (A_BYTES + B_BYTES) + 256); // BN floats

        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN, bz = blockIdx.z;
        long long *tl = (p.timeline && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) ? p.timeline : nullptr;
        if (tl && threadIdx.x == 0) tl[0] = clock64();
        const int num_kb = (int) ((p.K + BK - 1) / BK);

        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) {
                ptx::mbar_init(sBar + 8 * s, 1);
                ptx::mbar_init(sBar + 8 * (kStages + s), 1);
            }
            ptx::mbar_init(sBar + 8 * 2 * kStages, 1);
            for (int w = 0; w < 4; ++w) ptx::mbar_init(sBar + 8 * (2 * kStages + 2 + w), 1); // residual tile landed, per epilogue warp
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmA);
            ptx::prefetch_tmap(&tmB);
        }
        if (warp == 1) {
            ptx::tmem_alloc(sSlot, tmem_cols(BN));
            ptx::tmem_relinquish();
        }
        if (warp >= 2 && (p.epilogue & VKC_EPI_BIAS)) {
            for (int j = threadIdx.x - 64; j < BN; j += kThreads - 64) sbias[j] = (int64_t) n0 + j < p.N ? __ldg(p.bias + n0 + j) : 0.f;
        }
        ptx::tc_fence_before();
        __syncthreads();
        ptx::tc_fence_after();
        const uint32_t tmem = (uint32_t) ctl[0];
        if (tl && threadIdx.x == 0) tl[1] = clock64();

        if (warp == 0) {
            if (ptx::elect_one()) {
                const int za = p.a_bcast ? 0 : bz, zb = p.b_bcast ? 0 : bz;
                for (int kb = 0; kb < num_kb; ++kb) {
                    const int      s  = kb % kStages;
                    const uint32_t ph = (kb / kStages) & 1;
                    if (!ptx::mbar_wait(sBar + 8 * (kStages + s), ph ^ 1, ctl + 1, p.dev_err)) break;
                    const uint32_t full = sBar + 8 * s;
                    ptx::mbar_expect_tx(full, A_BYTES + B_BYTES);
                    ptx::tma_load_3d(sA + s * A_BYTES, &tmA, kb * BK, m0, za, full);
                    if (!B_KN) {
                        ptx::tma_load_3d(sB + s * B_BYTES, &tmB, kb * BK, n0, zb, full);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c) ptx::tma_load_3d(sB + s * B_BYTES + c * (BK * 128), &tmB, n0 + c * 64, kb * BK, zb, full);
                    }
                }
            }
        } else if (warp == 1) {
            if (ptx::elect_one()) {
                bool ok = true;
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    const int      s  = kb % kStages;
                    const uint32_t ph = (kb / kStages) & 1;
                    ok                = ptx::mbar_wait(sBar + 8 * s, ph, ctl + 1, p.dev_err);
                    if (!ok) break;
                    if (tl && kb == 0) tl[2] = clock64();
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = ptx::smem_desc_sw128(sA + s * A_BYTES + k * 32, 16, 1024);
                        const uint64_t bd = B_KN ? ptx::smem_desc_sw128(sB + s * B_BYTES + k * (16 * 128), BK * 128, 1024)
                                                 : ptx::smem_desc_sw128(sB + s * B_BYTES + k * 32, 16, 1024);
                        ptx::mma_f16_ss(tmem, ad, bd, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(sBar + 8 * (kStages + s)); // frees the stage once these MMAs have read it
                }
                if (ok) ptx::tc_commit(sBar + 8 * 2 * kStages); // accumulator complete
                if (tl) tl[3] = clock64();
            }
        } else {
            const bool ok = ptx::mbar_wait(sBar + 8 * 2 * kStages, 0, ctl + 1, p.dev_err);
            ptx::tc_fence_after();
            if (tl && threadIdx.x == 64) tl[4] = clock64();
            if (ok) {
                const int     q   = warp & 3; // the TMEM lane quarter this warp may address
                const int64_t m   = (int64_t) m0 + q * 32 + lane;
                T            *drow = (T *) p.D + (int64_t) bz * p.stride_d + m * p.ldd;
                const T      *rrow = p.residual ? (const T *) p.residual + (int64_t) bz * p.stride_d + m * p.ldd : nullptr;
                const bool    vec_ok = (p.ldd % 8 == 0) && (p.stride_d % 8 == 0) && (((uintptr_t) p.D & 15) == 0) &&
                                    (!p.residual || ((uintptr_t) p.residual & 15) == 0);
                if (p.tma_out) {
                    // Staged epilogue. The operand ring is idle now; each warp owns 32 output rows and, per 64-column
                    // slab, a 32 x 128 B staging block there (128-byte swizzle so that 8 lanes writing 8 different rows
                    // hit different banks). The residual slab is TMA-loaded into the same block, the result is written
                    // over it and leaves with one TMA store: global traffic is full 128-byte lines both ways.
                    constexpr int kSlabs = (BN + 63) / 64;
                    const uint32_t rbar  = sBar + 8 * (2 * kStages + 2 + q);
                    const int      row0  = m0 + q * 32;
                    const bool     rows_in = row0 < p.M; // warp-uniform
                    int            nslab = 0;
                    for (int sl = 0; sl < kSlabs; ++sl)
                        if ((int64_t) n0 + sl * 64 < p.N) nslab = sl + 1;
                    bool rok = true;
                    if ((p.epilogue & VKC_EPI_RESIDUAL) && rows_in) {
                        if (lane == 0) {
                            ptx::mbar_expect_tx(rbar, (uint32_t) nslab * 4096u);
                            for (int sl = 0; sl < nslab; ++sl) ptx::tma_load_3d(base + sl * 16384 + q * 4096, &tmR, n0 + sl * 64, row0, bz, rbar);
                        }
                        rok = ptx::mbar_wait(rbar, 0, ctl + 1, p.dev_err);
                        rok = __all_sync(0xffffffffu, rok);
                    }
#pragma unroll 1
                    for (int sl = 0; sl < nslab && rok; ++sl) {
                        uint8_t *blk = gbase + sl * 16384 + q * 4096 + lane * 128;
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            uint32_t r[32];
                            ptx::tmem_ld_x32(tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (sl * 64 + hf * 32), r);
                            ptx::tc_wait_ld();
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                            if (p.epilogue & VKC_EPI_BIAS) {
#pragma unroll
                                for (int j = 0; j < 32; j += 4) {
                                    const float4 bv = *reinterpret_cast<const float4 *>(sbias + sl * 64 + hf * 32 + j);
                                    v[j] += bv.x, v[j + 1] += bv.y, v[j + 2] += bv.z, v[j + 3] += bv.w;
                                }
                            }
                            if (p.epilogue & VKC_EPI_GELU_ERF) {
#pragma unroll
                                for (int j = 0; j < 32; j += 2) {
                                    const float2 g2 = gelu_erf_pair(make_float2(v[j], v[j + 1]));
                                    v[j] = g2.x, v[j + 1] = g2.y;
                                }
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                uint4 *slot = reinterpret_cast<uint4 *>(blk + (((hf * 4 + u) ^ (lane & 7)) << 4));
                                if (p.epilogue & VKC_EPI_RESIDUAL) {
                                    const uint4 rv = *slot;
                                    const T    *rt = reinterpret_cast<const T *>(&rv);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) v[u * 8 + j] += St<T>::ld(rt + j);
                                }
                                uint4 ov;
                                T    *ot = reinterpret_cast<T *>(&ov);
#pragma unroll
                                for (int j = 0; j < 8; ++j) St<T>::st(ot + j, v[u * 8 + j]);
                                *slot = ov;
                            }
                        }
                        ptx::fence_proxy_async();
                        __syncwarp();
                        if (lane == 0 && rows_in) {
                            ptx::tma_store_3d(&tmD, base + sl * 16384 + q * 4096, n0 + sl * 64, row0, bz);
                            ptx::bulk_commit_group();
                        }
                    }
                    if (lane == 0) ptx::bulk_wait_group_0();
                    __syncwarp();
                } else
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int64_t nb = (int64_t) n0 + c * 32;
                    if (nb >= p.N) break; // uniform across the CTA
                    uint32_t r[32];
                    ptx::tmem_ld_x32(tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (c * 32), r);
                    ptx::tc_wait_ld();
                    if (m < p.M) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        const bool full = nb + 32 <= p.N;
                        if (p.epilogue & VKC_EPI_BIAS) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 bv = *reinterpret_cast<const float4 *>(sbias + c * 32 + j);
                                v[j] += bv.x, v[j + 1] += bv.y, v[j + 2] += bv.z, v[j + 3] += bv.w;
                            }
                        }
                        if (p.epilogue & VKC_EPI_GELU_ERF) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = vkc_gelu_erf_fast(v[j]);
                        }
                        if (full && vec_ok) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                if (p.epilogue & VKC_EPI_RESIDUAL) {
                                    uint4    rv = *reinterpret_cast<const uint4 *>(rrow + nb + g * 8);
                                    const T *rt = reinterpret_cast<const T *>(&rv);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) v[g * 8 + j] += St<T>::ld(rt + j);
                                }
                                uint4 ov;
                                T    *ot = reinterpret_cast<T *>(&ov);
#pragma unroll
                                for (int j = 0; j < 8; ++j) St<T>::st(ot + j, v[g * 8 + j]);
                                *reinterpret_cast<uint4 *>(drow + nb + g * 8) = ov;
                            }
                        } else {
                            for (int j = 0; j < 32; ++j) {
                                if (nb + j < p.N) {
                                    float o = v[j];
                                    if (p.epilogue & VKC_EPI_RESIDUAL) o += St<T>::ld(rrow + nb + j);
                                    St<T>::st(drow + nb + j, o);
                                }
                            }
                        }
                    }
                }
            }
        }
        if (tl && threadIdx.x == 64) tl[5] = clock64();
        if (ctl[1]) {
            // aborted: give copies still in flight time to land before the CTA releases its shared memory
            for (int i = 0; i < 50; ++i) __nanosleep(20000);
        }
        ptx::tc_fence_before();
        __syncthreads();
        if (warp == 1) ptx::tmem_dealloc(tmem, tmem_cols(BN));
        if (tl && threadIdx.x == 0) tl[6] = clock64();
    }

    template <int BN, int kStages, int kCtasPerSm, typename T, bool B_KN>
    int launch(vkc_ctx *ctx, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmD, const CUtensorMap &tmR, const GemmParams &p,
               int64_t batch, cudaStream_t st) {
        auto          kern = gemm_tcgen05_kernel<BN, kStages, kCtasPerSm, T, B_KN>;
        constexpr int smem = smem_bytes<BN, kStages>();
        static_assert(smem * kCtasPerSm <= 227 * 1024, "shared memory budget");
        if (int rc = vkc_configure_smem(ctx, kern, smem)) return rc;
        dim3 grid((unsigned) ((p.M + BM - 1) / BM), (unsigned) ((p.N + BN - 1) / BN), (unsigned) batch);
        kern<<<grid, kThreads, smem, st>>>(tmA, tmB, tmD, tmR, p);
        return vkc_post_launch(ctx, "gemm_tcgen05");
    }

    // Tile width: fewest waves over the SMs first, then the least padded work. Wide tiles re-read A less often.
    struct TileChoice {
        int bn;
        bool two_ctas;
    };
    TileChoice choose_tile(int64_t M, int64_t N, int64_t batch, int sms) {
        const int64_t mt = (M + BM - 1) / BM;
        TileChoice    best {128, true};
        double        best_cost = 1e300;
        const int     cands[4]  = {256, 192, 128, 64};
        for (int bn : cands) {
            const int64_t tiles = mt * ((N + bn - 1) / bn) * batch;
            // two co-resident CTAs share one tensor pipe: model a slot as half an SM
            const double waves = std::ceil((double) tiles / (2.0 * sms));
            const double cost  = waves * (bn + 48.0); // per-tile time ~ width + fixed prologue/epilogue
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best      = {bn, true};
            }
        }
        // very large problems: the deep 4-stage 256-wide pipeline, one CTA per SM
        if (mt * ((N + 255) / 256) * batch >= 4 * (int64_t) sms) best = {256, false};
        return best;
    }

} // namespace

// Returns VKC_ERR_UNSUPPORTED (without touching ctx->err semantics beyond the message) when the operands do not
// meet the TMA alignment rules; the caller then uses the SIMT kernel.
int vkc_gemm_tcgen05(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                     int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                     int b_layout, int epilogue, int dtype, cudaStream_t st) {
    if (dtype != VKC_F16 && dtype != VKC_BF16) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: 16-bit storage only");
    if ((lda % 8) || (ldb % 8) || (stride_a % 8) || (stride_b % 8) || ((uintptr_t) A & 15) || ((uintptr_t) B & 15))
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: operand strides/bases must be multiples of 16 bytes");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > 65535) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: extent too large");

    {
        // CTA-pair form (256-row tiles over two SMs); selection heuristics live here
        static const char *force = getenv("VKNN_GEMM_PAIR");
        const int          bn    = force ? atoi(force) : 0;
        if ((bn == 128 || bn == 256) && M > 128)
            return vkc_gemm_tcgen05_pair(ctx, A, B, bias, residual, D, M, N, K, batch, stride_a, stride_b, stride_d, lda, ldb, ldd, b_layout, epilogue,
                                         dtype, bn, st);
    }
    const bool a_bcast = stride_a == 0 || batch == 1, b_bcast = stride_b == 0 || batch == 1;
    const TileChoice tc = choose_tile(M, N, batch, ctx->sm_count);
    const int        BN = tc.bn;

    CUtensorMap tmA, tmB;
    {
        uint64_t dims[3] = {(uint64_t) K, (uint64_t) M, (uint64_t) (a_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) lda * 2, (uint64_t) (a_bcast ? (uint64_t) lda * 2 * (uint64_t) M : (uint64_t) stride_a * 2)};
        uint32_t box[3]  = {BK, BM, 1};
        int      rc      = vkc_make_tmap(ctx, &tmA, dtype, A, 3, dims, str, box);
        if (rc) return rc;
    }
    if (b_layout == VKC_B_NK) {
        uint64_t dims[3] = {(uint64_t) K, (uint64_t) N, (uint64_t) (b_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) ldb * 2, (uint64_t) (b_bcast ? (uint64_t) ldb * 2 * (uint64_t) N : (uint64_t) stride_b * 2)};
        uint32_t box[3]  = {BK, (uint32_t) BN, 1};
        int      rc      = vkc_make_tmap(ctx, &tmB, dtype, B, 3, dims, str, box);
        if (rc) return rc;
    } else {
        uint64_t dims[3] = {(uint64_t) N, (uint64_t) K, (uint64_t) (b_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) ldb * 2, (uint64_t) (b_bcast ? (uint64_t) ldb * 2 * (uint64_t) K : (uint64_t) stride_b * 2)};
        uint32_t box[3]  = {64, BK, 1};
        int      rc      = vkc_make_tmap(ctx, &tmB, dtype, B, 3, dims, str, box);
        if (rc) return rc;
    }
    GemmParams p;
    p.bias     = bias;
    p.residual = residual;
    p.D        = D;
    p.M        = M;
    p.N        = N;
    p.K        = K;
    p.ldd      = ldd;
    p.stride_d = stride_d;
    p.epilogue = epilogue;
    p.a_bcast  = a_bcast;
    p.b_bcast  = b_bcast;
    p.dev_err  = ctx->dev_err;
    p.timeline = ctx->timeline;
    // output / residual maps for the staged epilogue (box = 64 columns x 32 rows, one per epilogue warp and slab)
    CUtensorMap tmD = tmA, tmR = tmA;
    p.tma_out       = 0;
    if ((ldd % 8 == 0) && (stride_d % 8 == 0) && (((uintptr_t) D & 15) == 0) && (!(epilogue & VKC_EPI_RESIDUAL) || (((uintptr_t) residual & 15) == 0))) {
        uint64_t dims[3] = {(uint64_t) N, (uint64_t) M, (uint64_t) batch};
        uint64_t str[2]  = {(uint64_t) ldd * 2, (uint64_t) (batch > 1 ? (uint64_t) stride_d * 2 : (uint64_t) ldd * 2 * (uint64_t) M)};
        uint32_t box[3]  = {64, 32, 1};
        int      rc      = vkc_make_tmap(ctx, &tmD, dtype, D, 3, dims, str, box);
        if (rc == VKC_OK && (epilogue & VKC_EPI_RESIDUAL)) rc = vkc_make_tmap(ctx, &tmR, dtype, residual, 3, dims, str, box);
        p.tma_out = rc == VKC_OK ? 1 : 0;
    }

#define VKC_GEMM_LAUNCH(BN_, ST_, C_, T_)                                                                       \
    (b_layout == VKC_B_KN ? launch<BN_, ST_, C_, T_, true>(ctx, tmA, tmB, tmD, tmR, p, batch, st) \
                          : launch<BN_, ST_, C_, T_, false>(ctx, tmA, tmB, tmD, tmR, p, batch, st))
#define VKC_GEMM_BY_TILE(T_)                                                         \
    do {                                                                             \
        if (!tc.two_ctas) return VKC_GEMM_LAUNCH(256, 4, 1, T_);                     \
        switch (BN) {                                                                \
            case 256: return VKC_GEMM_LAUNCH(256, 2, 2, T_);                         \
            case 192: return VKC_GEMM_LAUNCH(192, 2, 2, T_);                         \
            case 128: return VKC_GEMM_LAUNCH(128, 3, 2, T_);                         \
            default: return VKC_GEMM_LAUNCH(64, 4, 2, T_);                           \
        }                                                                            \
    } while (0)
    if (dtype == VKC_F16) VKC_GEMM_BY_TILE(__half);
    VKC_GEMM_BY_TILE(__nv_bfloat16);
#undef VKC_GEMM_BY_TILE
#undef VKC_GEMM_LAUNCH
}
