// K2 — fused prefill attention on the 5th-generation tensor cores (flash style: the score matrix never leaves
// the SM). One CTA owns one 128-row query tile of one (batch, head) and walks the key/value sequence in tiles
// of 128 keys.
//
//   warp 0    TMA producer: Q once, then K and V tiles through two independent 2-stage shared-memory rings
//             (128-byte swizzle, plain per-CTA tiled loads; out-of-range rows arrive as zeros).
//   warp 1    MMA issuer (one elected lane) and owner of the tensor-memory allocation (512 columns):
//               S[j%2]  (128 fp32 cols each)  = Q . K_j^T      tcgen05.mma, both operands from shared memory
//               O       (D fp32 cols)        += P_j . V_j      P from tensor memory (or shared memory), V MN-major
//             S is double buffered so Q.K_{j+1}^T runs while the softmax warps work on S_j.
//   warps 2-5 softmax: thread r owns row r. Pass 1 reads S_j from TMEM for the row maximum, pass 2 re-reads it,
//             computes P = exp2(S*scale*log2e - m) in fp32, packs to the storage type and writes P to TMEM
//             (tcgen05.st) for the P.V MMA. The running maximum is only raised when it grows by more than 8
//             (a factor 256), so the O accumulator in TMEM is rescaled rarely; sums stay in fp32.
//             After the last tile the same warps read O, divide by the row sum and store the tile.
// Masking: keys >= kv_len[b] (or >= Skv) and, for causal, keys > row + (Skv - Sq) get probability 0; key tiles
// entirely above the diagonal are skipped.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace {

    constexpr int BM = 128, BN = 128;
    constexpr int kThreads   = 192;
    constexpr int kTmemCols  = 512;
    constexpr int kColS      = 0;   // S0 at 0, S1 at 128
    constexpr int kColO      = 256; // D columns
    constexpr int kColP      = 384; // P0 at 384, P1 at 448 (64 columns each: 128 packed 16-bit values per row)
    constexpr float kRescaleThreshold = 8.0f;

    struct AttnParams {
        void          *O;
        int64_t        os[3];
        int64_t        Sq, Skv, Hq, Hkv;
        float          scale_log2;
        int            causal;
        const int32_t *kv_len;
        int           *dev_err;
    };

    template <int D, int KS, int VS, bool P_TMEM> struct Smem {
        static constexpr uint32_t Q_BYTES  = BM * D * 2;
        static constexpr uint32_t KV_BYTES = BN * D * 2;
        static constexpr uint32_t P_BYTES  = P_TMEM ? 0 : BM * BN * 2;
        static constexpr uint32_t oQ   = 0;
        static constexpr uint32_t oK   = oQ + Q_BYTES;
        static constexpr uint32_t oV   = oK + KS * KV_BYTES;
        static constexpr uint32_t oP   = oV + VS * KV_BYTES;
        static constexpr uint32_t oBar = oP + P_BYTES;
        // barriers: q_full, k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[2], s_empty[2], p_full[2], pv_done[2]
        static constexpr int nBar = 1 + 2 * KS + 2 * VS + 8;
        static constexpr uint32_t oCtl  = oBar + 8 * nBar;
        static constexpr uint32_t total = oCtl + 16 + 1024;
    };

    __device__ __forceinline__ float fast_exp2(float x) {
        float y;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
        return y;
    }
    template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
    template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }

    template <typename T, int D, bool P_TMEM>
    __global__ void __launch_bounds__(kThreads, 1)
        attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            AttnParams p) {
        constexpr int KS = 2, VS = 2;
        using L               = Smem<D, KS, VS, P_TMEM>;
        constexpr bool kBf16  = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdescQK = ptx::idesc_f16(BM, BN, kBf16, false, false);
        constexpr uint32_t kIdescPV = ptx::idesc_f16(BM, D, kBf16, false, true);
        constexpr int      DCH      = D / 64; // 64-element (128-byte) spans per row

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sQ = base + L::oQ, sK = base + L::oK, sV = base + L::oV, sP = base + L::oP, sBar = base + L::oBar;
        volatile int  *ctl = (volatile int *) (gbase + L::oCtl); // ctl[0] = tmem base, ctl[1] = abort flag
        auto           bar = [&](int i) { return sBar + 8u * (uint32_t) i; };
        constexpr int  bQ = 0, bKF = 1, bKE = 1 + KS, bVF = 1 + 2 * KS, bVE = 1 + 2 * KS + VS, bSF = 1 + 2 * KS + 2 * VS, bSE = bSF + 2,
                      bPF = bSF + 4, bPV = bSF + 6;

        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int b = blockIdx.z, h = blockIdx.y;
        const int hk = h / (int) (p.Hq / p.Hkv);
        // heavy (late) query tiles first when causal
        const int     mt = p.causal ? (int) gridDim.x - 1 - (int) blockIdx.x : (int) blockIdx.x;
        const int64_t m0 = (int64_t) mt * BM;

        int64_t len = p.kv_len ? (int64_t) p.kv_len[b] : p.Skv;
        if (len > p.Skv) len = p.Skv;
        if (len < 0) len = 0;
        int64_t kend = len;
        if (p.causal) {
            int64_t last = m0 + BM - 1;
            if (last > p.Sq - 1) last = p.Sq - 1;
            const int64_t lim = last + (p.Skv - p.Sq) + 1;
            if (lim < kend) kend = lim;
        }
        const int n_tiles = kend > 0 ? (int) ((kend + BN - 1) / BN) : 0;

        if (threadIdx.x == 0) {
            for (int i = 0; i < L::nBar; ++i) {
                const bool many = (i >= bSE && i < bSE + 2) || (i >= bPF && i < bPF + 2); // arrived on by all 128 softmax threads
                ptx::mbar_init(bar(i), many ? 128 : 1);
            }
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmQ);
            ptx::prefetch_tmap(&tmK);
            ptx::prefetch_tmap(&tmV);
        }
        if (warp == 1) {
            ptx::tmem_alloc(base + L::oCtl, kTmemCols);
            ptx::tmem_relinquish();
        }
        ptx::tc_fence_before();
        __syncthreads();
        ptx::tc_fence_after();
        const uint32_t tmem = (uint32_t) ctl[0];

        if (warp == 0) {
            // ------------------------------------------------------------------ TMA producer
            if (n_tiles > 0 && ptx::elect_one()) {
                ptx::mbar_expect_tx(bar(bQ), L::Q_BYTES);
#pragma unroll
                for (int c = 0; c < DCH; ++c) ptx::tma_load_4d(sQ + c * (BM * 128), &tmQ, c * 64, (int) m0, h, b, bar(bQ));
                for (int j = 0; j < n_tiles; ++j) {
                    const int ks = j % KS, vs = j % VS;
                    if (!ptx::mbar_wait(bar(bKE + ks), ((j / KS) & 1) ^ 1, ctl + 1, p.dev_err)) break;
                    ptx::mbar_expect_tx(bar(bKF + ks), L::KV_BYTES);
#pragma unroll
                    for (int c = 0; c < DCH; ++c) ptx::tma_load_4d(sK + ks * L::KV_BYTES + c * (BN * 128), &tmK, c * 64, j * BN, hk, b, bar(bKF + ks));
                    if (!ptx::mbar_wait(bar(bVE + vs), ((j / VS) & 1) ^ 1, ctl + 1, p.dev_err)) break;
                    ptx::mbar_expect_tx(bar(bVF + vs), L::KV_BYTES);
#pragma unroll
                    for (int c = 0; c < DCH; ++c) ptx::tma_load_4d(sV + vs * L::KV_BYTES + c * (BN * 128), &tmV, c * 64, j * BN, hk, b, bar(bVF + vs));
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------------ MMA issuer
            if (n_tiles > 0 && ptx::elect_one()) {
                auto issue_qk = [&](int j) -> bool {
                    const int ks = j % KS, sb = j & 1;
                    if (!ptx::mbar_wait(bar(bKF + ks), (j / KS) & 1, ctl + 1, p.dev_err)) return false;
                    if (!ptx::mbar_wait(bar(bSE + sb), ((j / 2) & 1) ^ 1, ctl + 1, p.dev_err)) return false;
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const uint32_t off = (uint32_t) (k / 4) * (BM * 128) + (uint32_t) (k % 4) * 32;
                        const uint64_t ad  = ptx::smem_desc_sw128(sQ + off, 16, 1024);
                        const uint64_t bd  = ptx::smem_desc_sw128(sK + ks * L::KV_BYTES + off, 16, 1024);
                        ptx::mma_f16_ss(tmem + kColS + sb * BN, ad, bd, kIdescQK, k != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(bar(bKE + ks));
                    ptx::tc_commit(bar(bSF + sb));
                    return true;
                };
                bool ok = ptx::mbar_wait(bar(bQ), 0, ctl + 1, p.dev_err);
                ok      = ok && issue_qk(0);
                for (int j = 0; j < n_tiles && ok; ++j) {
                    if (j + 1 < n_tiles) ok = issue_qk(j + 1);
                    if (!ok) break;
                    const int vs = j % VS, pb = j & 1;
                    if (!ptx::mbar_wait(bar(bVF + vs), (j / VS) & 1, ctl + 1, p.dev_err)) break;
                    if (!ptx::mbar_wait(bar(bPF + pb), (j / 2) & 1, ctl + 1, p.dev_err)) break;
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k) {
                        // V tile: D/64 spans of [128 keys x 128 B]; 16 keys per MMA step = 2048 B
                        const uint64_t bd = ptx::smem_desc_sw128(sV + vs * L::KV_BYTES + k * 2048, BN * 128, 1024);
                        if (P_TMEM) {
                            ptx::mma_f16_ts(tmem + kColO, tmem + kColP + pb * 64 + k * 8, bd, kIdescPV, (j | k) != 0 ? 1u : 0u);
                        } else {
                            const uint32_t off = (uint32_t) (k / 4) * (BM * 128) + (uint32_t) (k % 4) * 32;
                            const uint64_t ad  = ptx::smem_desc_sw128(sP + off, 16, 1024);
                            ptx::mma_f16_ss(tmem + kColO, ad, bd, kIdescPV, (j | k) != 0 ? 1u : 0u);
                        }
                    }
                    ptx::tc_commit(bar(bVE + vs));
                    ptx::tc_commit(bar(bPV + pb));
                }
            }
        } else {
            // ------------------------------------------------------------------ softmax + epilogue (thread = row)
            const int      q      = warp & 3;
            const int      r      = q * 32 + lane;
            const int64_t  row    = m0 + r;
            const uint32_t tlane  = (uint32_t) (q * 32) << 16;
            const int64_t  my_lim = p.causal ? row + (p.Skv - p.Sq) : p.Skv; // keys <= my_lim visible
            float          m_used = -INFINITY, l = 0.f;
            bool           ok     = true;
            for (int j = 0; j < n_tiles; ++j) {
                const int     sb = j & 1;
                const int64_t kv0 = (int64_t) j * BN;
                ok = ptx::mbar_wait(bar(bSF + sb), (j / 2) & 1, ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tc_fence_after();
                const bool need_mask = (kv0 + BN > len) || (p.causal && kv0 + BN - 1 > m0 + (p.Skv - p.Sq));
                // pass 1: row maximum (raw scores)
                float mx = -INFINITY;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    ptx::tmem_ld_x32(tmem + tlane + kColS + sb * BN + c * 32, v);
                    ptx::tc_wait_ld();
                    if (need_mask) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int64_t key = kv0 + c * 32 + i;
                            if (key < len && key <= my_lim) mx = fmaxf(mx, __uint_as_float(v[i]));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
                    }
                }
                const float mx2 = mx * p.scale_log2; // scale > 0
                float       alpha = 1.f;
                bool        rescale = false;
                if (mx2 > m_used + kRescaleThreshold || m_used == -INFINITY) {
                    if (mx2 > m_used) {
                        alpha   = m_used == -INFINITY ? 0.f : fast_exp2(m_used - mx2);
                        rescale = j > 0 && m_used != -INFINITY;
                        m_used  = mx2;
                    }
                }
                const float m_safe = m_used == -INFINITY ? 0.f : m_used;
                l *= alpha;
                // O rescale first (it needs P.V of the previous tile finished), then P
                if (__any_sync(0xffffffffu, rescale)) {
                    ok = ptx::mbar_wait(bar(bPV + ((j - 1) & 1)), ((j - 1) / 2) & 1, ctl + 1, p.dev_err);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    ptx::tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_x32(tmem + tlane + kColO + c * 32, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        ptx::tmem_st_x32(tmem + tlane + kColO + c * 32, v);
                    }
                }
                // pass 2: probabilities
                if (!P_TMEM && j > 0) {
                    // the single shared-memory P buffer is free once P.V of the previous tile has read it
                    ok = ptx::mbar_wait(bar(bPV + ((j - 1) & 1)), ((j - 1) / 2) & 1, ctl + 1, p.dev_err);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    ptx::tmem_ld_x32(tmem + tlane + kColS + sb * BN + c * 32, v);
                    ptx::tc_wait_ld();
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        float p0 = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, -m_safe));
                        float p1 = fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, -m_safe));
                        if (need_mask) {
                            const int64_t key = kv0 + c * 32 + i;
                            if (!(key < len && key <= my_lim)) p0 = 0.f;
                            if (!(key + 1 < len && key + 1 <= my_lim)) p1 = 0.f;
                        }
                        l += p0 + p1;
                        pk[i / 2] = pack2<T>(p0, p1);
                    }
                    if (P_TMEM) {
                        ptx::tmem_st_x16(tmem + tlane + kColP + sb * 64 + c * 16, pk);
                    } else {
                        // K-major 128-byte-swizzled rows: two spans of 64 keys, 16-byte units XORed with (row % 8)
                        const uint32_t rowoff = (uint32_t) (c / 2) * (BM * 128) + (uint32_t) (r / 8) * 1024 + (uint32_t) (r % 8) * 128;
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const uint32_t unit = (uint32_t) ((c & 1) * 4 + u) ^ (uint32_t) (r & 7);
                            uint4          val  = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
                            *reinterpret_cast<uint4 *>(gbase + L::oP + rowoff + unit * 16) = val;
                        }
                    }
                }
                ptx::tc_wait_st();
                if (!P_TMEM) ptx::fence_proxy_async();
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(bSE + sb));
                ptx::mbar_arrive(bar(bPF + sb));
            }
            // epilogue
            if (n_tiles > 0 && ok) {
                ok = ptx::mbar_wait(bar(bPV + ((n_tiles - 1) & 1)), ((n_tiles - 1) / 2) & 1, ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                ptx::tc_fence_after();
                const float inv = 1.0f / l; // l == 0 (no visible key) stores NaN like the reference's 0/0
                T          *orow = (T *) p.O + (int64_t) b * p.os[0] + (int64_t) h * p.os[1] + row * p.os[2];
                const bool  vec_ok = (p.os[0] % 8 == 0) && (p.os[1] % 8 == 0) && (p.os[2] % 8 == 0) && (((uintptr_t) p.O & 15) == 0);
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t v[32];
                    if (n_tiles > 0) {
                        ptx::tmem_ld_x32(tmem + tlane + kColO + c * 32, v);
                        ptx::tc_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0u;
                    }
                    if (row < p.Sq) {
                        if (vec_ok) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                uint4     ov;
                                uint32_t *o32 = reinterpret_cast<uint32_t *>(&ov);
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    o32[i] = pack2<T>(__uint_as_float(v[g * 8 + 2 * i]) * inv, __uint_as_float(v[g * 8 + 2 * i + 1]) * inv);
                                *reinterpret_cast<uint4 *>(orow + c * 32 + g * 8) = ov;
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) St<T>::st(orow + c * 32 + i, __uint_as_float(v[i]) * inv);
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
        if (warp == 1) ptx::tmem_dealloc(tmem, kTmemCols);
    }

    template <typename T, int D, bool P_TMEM>
    int launch_attn(vkc_ctx *ctx, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const AttnParams &p, int64_t B, cudaStream_t st) {
        auto          kern = attn_prefill_kernel<T, D, P_TMEM>;
        constexpr int smem = (int) Smem<D, 2, 2, P_TMEM>::total;
        static bool   attr_set = false;
        if (!attr_set) {
            VKC_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            attr_set = true;
        }
        dim3 grid((unsigned) ((p.Sq + BM - 1) / BM), (unsigned) p.Hq, (unsigned) B);
        kern<<<grid, kThreads, smem, st>>>(tq, tk, tv, p);
        return vkc_post_launch(ctx, "attn_prefill_tcgen05");
    }

    int make_qkv_map(vkc_ctx *ctx, CUtensorMap *map, int dtype, const void *base, int64_t B, int64_t H, int64_t S, int64_t D, const int64_t *str) {
        // dims innermost first: {D, S, H, B}; element strides {1, str[2], str[1], str[0]}
        uint64_t dims[4] = {(uint64_t) D, (uint64_t) S, (uint64_t) H, (uint64_t) B};
        uint64_t sb[3]   = {(uint64_t) str[2] * 2, (uint64_t) str[1] * 2, (uint64_t) str[0] * 2};
        // a size-1 dimension may carry any stride; give it a valid one
        if (H == 1 && (sb[1] == 0 || sb[1] % 16)) sb[1] = sb[0] * (uint64_t) S;
        if (B == 1 && (sb[2] == 0 || sb[2] % 16)) sb[2] = sb[1] * (uint64_t) H;
        uint32_t box[4] = {64, 128, 1, 1};
        return vkc_make_tmap(ctx, map, dtype, base, 4, dims, sb, box);
    }

} // namespace

// Whether P is handed to the P.V MMA through tensor memory (default) or through shared memory.
static int g_p_in_tmem = 1;
extern "C" VKC_API void vkc_debug_set_attn_p_in_tmem(int on) { g_p_in_tmem = on ? 1 : 0; }

int vkc_attn_prefill_tcgen05(vkc_ctx *ctx, const void *Q, const void *K, const void *V, void *O, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                             int64_t Skv, int64_t D, const int64_t *qs, const int64_t *ks, const int64_t *vs, const int64_t *os, float scale,
                             int causal, const int32_t *kv_len, int dtype, cudaStream_t st) {
    if (dtype != VKC_F16 && dtype != VKC_BF16) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_tcgen05: 16-bit storage only");
    if (D != 64 && D != 128) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_tcgen05: head dim must be 64 or 128");
    if (!(scale > 0.f)) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_tcgen05: scale must be positive");
    for (int i = 0; i < 3; ++i) {
        if ((qs[i] % 8) || (ks[i] % 8) || (vs[i] % 8))
            return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_tcgen05: Q/K/V strides must be multiples of 16 bytes");
    }
    if (((uintptr_t) Q | (uintptr_t) K | (uintptr_t) V) & 15) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_tcgen05: Q/K/V must be 16-byte aligned");
    if (Sq > INT32_MAX - BM || Skv > INT32_MAX - BN) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_tcgen05: sequence too long");

    CUtensorMap tq, tk, tv;
    int         rc;
    if ((rc = make_qkv_map(ctx, &tq, dtype, Q, B, Hq, Sq, D, qs))) return rc;
    if ((rc = make_qkv_map(ctx, &tk, dtype, K, B, Hkv, Skv, D, ks))) return rc;
    if ((rc = make_qkv_map(ctx, &tv, dtype, V, B, Hkv, Skv, D, vs))) return rc;
    AttnParams p;
    p.O = O;
    for (int i = 0; i < 3; ++i) p.os[i] = os[i];
    p.Sq = Sq, p.Skv = Skv, p.Hq = Hq, p.Hkv = Hkv;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal     = causal;
    p.kv_len     = kv_len;
    p.dev_err    = ctx->dev_err;
#define VKC_ATTN(T_, D_) (g_p_in_tmem ? launch_attn<T_, D_, true>(ctx, tq, tk, tv, p, B, st) : launch_attn<T_, D_, false>(ctx, tq, tk, tv, p, B, st))
    if (dtype == VKC_F16) return D == 64 ? VKC_ATTN(__half, 64) : VKC_ATTN(__half, 128);
    return D == 64 ? VKC_ATTN(__nv_bfloat16, 64) : VKC_ATTN(__nv_bfloat16, 128);
#undef VKC_ATTN
}
