// K1 (CTA-pair form) — the same GEMM as gemm_tcgen05.cu, computed by pairs of CTAs on two SMs that drive ONE
// tcgen05.mma.cta_group::2 stream: a pair owns a 256 x BN output tile, each CTA holds its own 128 rows of A and
// HALF of the B tile in shared memory, and the tensor cores of both SMs read both halves. Per CTA and 64-deep
// k-block that is 16 KB of A plus BN*64 bytes of B for 128 x BN x 64 MACs, half the operand traffic per flop of the
// single-CTA kernel, which is what the medium-size encoder GEMMs are bound by.
//
// Roles per CTA: warp 0 = TMA producer (its A rows, its B half; completion bytes are counted on the LEADER CTA's
// "full" mbarrier), warp 1 = tensor-memory owner and, in the leader CTA only, MMA issuer (commits each stage's
// "empty" mbarrier in both CTAs), warps 2-5 = epilogue over the CTA's own 128 accumulator rows.
// The two CTAs synchronise with a cluster barrier after mbarrier initialisation and before exit; every mbarrier
// wait in between is bounded like everywhere else in this library.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace {

    constexpr int BM       = 128; // rows per CTA (256 per pair)
    constexpr int BK       = 64;
    constexpr int kThreads = 192;

    struct PairParams {
        const float *bias;
        const void  *residual;
        void        *D;
        int64_t      M, N, K;
        int64_t      ldd, stride_d;
        int          epilogue;
        int          a_bcast, b_bcast;
        int         *dev_err;
    };

    template <int BN, int kStages> constexpr int pair_smem_bytes() { return kStages * (BM * BK * 2 + (BN / 2) * BK * 2) + 1024 + 256 + BN * 4; }

    template <int BN, int kStages, typename T, bool B_KN>
    __global__ void __launch_bounds__(kThreads, 1)
        gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, PairParams p) {
        constexpr uint32_t A_BYTES = BM * BK * 2;
        constexpr uint32_t B_BYTES = (BN / 2) * BK * 2; // this CTA's half of the B tile
        constexpr bool     kBf16   = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdesc  = ptx::idesc_f16(2 * BM, BN, kBf16, false, B_KN);
        constexpr int      kCols   = BN <= 128 ? 128 : 256;

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sA    = base;
        const uint32_t sB    = base + kStages * A_BYTES;
        const uint32_t sBar  = sB + kStages * B_BYTES; // full[kStages], empty[kStages], accum
        volatile int  *ctl   = (volatile int *) (gbase + kStages * (A_BYTES + B_BYTES) + 8 * (2 * kStages + 1));
        const uint32_t sSlot = sBar + 8 * (2 * kStages + 1);
        float         *sbias = (float *) (gbase + kStages * (A_BYTES + B_BYTES) + 256);

        const int      warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const uint32_t rank = ptx::cluster_ctarank(); // 0 = leader
        const int      pair = blockIdx.x >> 1;
        const int      m0 = pair * (2 * BM) + (int) rank * BM, n0 = blockIdx.y * BN, bz = blockIdx.z;
        const int      num_kb = (int) ((p.K + BK - 1) / BK);

        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) {
                ptx::mbar_init(sBar + 8 * s, 1);
                ptx::mbar_init(sBar + 8 * (kStages + s), 1);
            }
            ptx::mbar_init(sBar + 8 * 2 * kStages, 1);
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmA);
            ptx::prefetch_tmap(&tmB);
        }
        if (warp == 1) {
            ptx::tmem_alloc_pair(sSlot, kCols);
            ptx::tmem_relinquish_pair();
        }
        if (warp >= 2 && (p.epilogue & VKC_EPI_BIAS)) {
            for (int j = threadIdx.x - 64; j < BN; j += kThreads - 64) sbias[j] = (int64_t) n0 + j < p.N ? __ldg(p.bias + n0 + j) : 0.f;
        }
        ptx::tc_fence_before();
        __syncthreads();
        ptx::cluster_sync(); // both CTAs' mbarriers exist before either side signals them
        ptx::tc_fence_after();
        const uint32_t tmem = (uint32_t) ctl[0];

        if (warp == 0) {
            if (ptx::elect_one()) {
                const int za = p.a_bcast ? 0 : bz, zb = p.b_bcast ? 0 : bz;
                for (int kb = 0; kb < num_kb; ++kb) {
                    const int      s  = kb % kStages;
                    const uint32_t ph = (kb / kStages) & 1;
                    if (!ptx::mbar_wait(sBar + 8 * (kStages + s), ph ^ 1, ctl + 1, p.dev_err)) break;
                    const uint32_t full_leader = ptx::mapa(sBar + 8 * s, 0);
                    if (rank == 0) ptx::mbar_expect_tx(sBar + 8 * s, 2 * (A_BYTES + B_BYTES)); // bytes of both CTAs
                    ptx::tma_load_3d_pair(sA + s * A_BYTES, &tmA, kb * BK, m0, za, full_leader);
                    if (!B_KN) {
                        ptx::tma_load_3d_pair(sB + s * B_BYTES, &tmB, kb * BK, n0 + (int) rank * (BN / 2), zb, full_leader);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 128; ++c)
                            ptx::tma_load_3d_pair(sB + s * B_BYTES + c * (BK * 128), &tmB, n0 + (int) rank * (BN / 2) + c * 64, kb * BK, zb, full_leader);
                    }
                }
            }
        } else if (warp == 1) {
            if (rank == 0 && ptx::elect_one()) {
                bool ok = true;
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    const int      s  = kb % kStages;
                    const uint32_t ph = (kb / kStages) & 1;
                    ok                = ptx::mbar_wait(sBar + 8 * s, ph, ctl + 1, p.dev_err);
                    if (!ok) break;
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = ptx::smem_desc_sw128(sA + s * A_BYTES + k * 32, 16, 1024);
                        const uint64_t bd = B_KN ? ptx::smem_desc_sw128(sB + s * B_BYTES + k * (16 * 128), BK * 128, 1024)
                                                 : ptx::smem_desc_sw128(sB + s * B_BYTES + k * 32, 16, 1024);
                        ptx::mma_f16_ss_pair(tmem, ad, bd, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    // the stage is free in BOTH CTAs once these MMAs have read it
                    ptx::tc_commit_pair(sBar + 8 * (kStages + s));
                    ptx::tc_commit_pair(ptx::mapa(sBar + 8 * (kStages + s), 1));
                }
                if (ok) {
                    ptx::tc_commit_pair(sBar + 8 * 2 * kStages);
                    ptx::tc_commit_pair(ptx::mapa(sBar + 8 * 2 * kStages, 1));
                }
            }
        } else {
            const bool ok = ptx::mbar_wait(sBar + 8 * 2 * kStages, 0, ctl + 1, p.dev_err);
            ptx::tc_fence_after();
            if (ok) {
                const int     q   = warp & 3;
                const int64_t m   = (int64_t) m0 + q * 32 + lane;
                T            *drow = (T *) p.D + (int64_t) bz * p.stride_d + m * p.ldd;
                const T      *rrow = p.residual ? (const T *) p.residual + (int64_t) bz * p.stride_d + m * p.ldd : nullptr;
                const bool    vec_ok = (p.ldd % 8 == 0) && (p.stride_d % 8 == 0) && (((uintptr_t) p.D & 15) == 0) &&
                                    (!p.residual || ((uintptr_t) p.residual & 15) == 0);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int64_t nb = (int64_t) n0 + c * 32;
                    if (nb >= p.N) break;
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
        if (ctl[1]) {
            for (int i = 0; i < 50; ++i) __nanosleep(20000); // aborted: let copies in flight land
        }
        ptx::tc_fence_before();
        __syncthreads();
        ptx::cluster_sync(); // neither CTA leaves while the other may still touch its shared memory or barriers
        if (warp == 1) ptx::tmem_dealloc_pair(tmem, kCols);
    }

    template <int BN, int kStages, typename T, bool B_KN>
    int launch_pair(vkc_ctx *ctx, const CUtensorMap &tmA, const CUtensorMap &tmB, const PairParams &p, int64_t batch, cudaStream_t st) {
        auto          kern = gemm_pair_kernel<BN, kStages, T, B_KN>;
        constexpr int smem = pair_smem_bytes<BN, kStages>();
        static_assert(smem <= 227 * 1024, "shared memory budget");
        if (int rc = vkc_configure_smem(ctx, kern, smem)) return rc;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim          = dim3((unsigned) (2 * ((p.M + 2 * BM - 1) / (2 * BM))), (unsigned) ((p.N + BN - 1) / BN), (unsigned) batch);
        cfg.blockDim         = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream           = st;
        cudaLaunchAttribute attr[1];
        attr[0].id               = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs                = attr;
        cfg.numAttrs             = 1;
        VKC_CUDA(ctx, cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p));
        return vkc_post_launch(ctx, "gemm_pair");
    }

} // namespace

// BN = 256 or 128 (bn argument). Returns VKC_ERR_UNSUPPORTED when the operands do not meet the TMA alignment rules.
int vkc_gemm_tcgen05_pair(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                          int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                          int b_layout, int epilogue, int dtype, int bn, cudaStream_t st) {
    if (dtype != VKC_F16 && dtype != VKC_BF16) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_pair: 16-bit storage only");
    if ((lda % 8) || (ldb % 8) || (stride_a % 8) || (stride_b % 8) || ((uintptr_t) A & 15) || ((uintptr_t) B & 15))
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_pair: operand strides/bases must be multiples of 16 bytes");
    if (M > INT32_MAX - 512 || N > INT32_MAX - 512 || K > INT32_MAX || batch > 65535) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_pair: extent too large");
    const bool a_bcast = stride_a == 0 || batch == 1, b_bcast = stride_b == 0 || batch == 1;
    CUtensorMap tmA, tmB;
    {
        uint64_t dims[3] = {(uint64_t) K, (uint64_t) M, (uint64_t) (a_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) lda * 2, (uint64_t) (a_bcast ? (uint64_t) lda * 2 * (uint64_t) M : (uint64_t) stride_a * 2)};
        uint32_t box[3]  = {BK, BM, 1};
        if (int rc = vkc_make_tmap(ctx, &tmA, dtype, A, 3, dims, str, box)) return rc;
    }
    if (b_layout == VKC_B_NK) {
        uint64_t dims[3] = {(uint64_t) K, (uint64_t) N, (uint64_t) (b_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) ldb * 2, (uint64_t) (b_bcast ? (uint64_t) ldb * 2 * (uint64_t) N : (uint64_t) stride_b * 2)};
        uint32_t box[3]  = {BK, (uint32_t) (bn / 2), 1};
        if (int rc = vkc_make_tmap(ctx, &tmB, dtype, B, 3, dims, str, box)) return rc;
    } else {
        uint64_t dims[3] = {(uint64_t) N, (uint64_t) K, (uint64_t) (b_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) ldb * 2, (uint64_t) (b_bcast ? (uint64_t) ldb * 2 * (uint64_t) K : (uint64_t) stride_b * 2)};
        uint32_t box[3]  = {64, BK, 1};
        if (int rc = vkc_make_tmap(ctx, &tmB, dtype, B, 3, dims, str, box)) return rc;
    }
    PairParams p;
    p.bias = bias, p.residual = residual, p.D = D;
    p.M = M, p.N = N, p.K = K, p.ldd = ldd, p.stride_d = stride_d;
    p.epilogue = epilogue, p.a_bcast = a_bcast, p.b_bcast = b_bcast, p.dev_err = ctx->dev_err;
#define VKC_PAIR(BN_, ST_, T_) \
    (b_layout == VKC_B_KN ? launch_pair<BN_, ST_, T_, true>(ctx, tmA, tmB, p, batch, st) : launch_pair<BN_, ST_, T_, false>(ctx, tmA, tmB, p, batch, st))
    if (dtype == VKC_F16) return bn == 256 ? VKC_PAIR(256, 6, __half) : VKC_PAIR(128, 8, __half);
    return bn == 256 ? VKC_PAIR(256, 6, __nv_bfloat16) : VKC_PAIR(128, 8, __nv_bfloat16);
#undef VKC_PAIR
}
