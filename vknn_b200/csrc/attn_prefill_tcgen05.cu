// K2 — fused prefill attention on the 5th-generation tensor cores (flash style: the score matrix never leaves
// the SM). One CTA owns TWO 128-row query tiles (A and B) of one (batch, head) and walks the key/value
// sequence in tiles of 128 keys; while the softmax warps of one query tile work, the tensor core runs the
// MMAs of the other.
//
//   warp 0     TMA producer: both Q tiles once, then K and V tiles through two independent 2-stage
//              shared-memory rings (128-byte swizzle, plain per-CTA tiled loads; rows past the end read as zeros).
//   warp 1     MMA issuer (one elected lane) and owner of the tensor-memory allocation (512 columns):
//                S_t (128 fp32 columns)  = Q_t . K_j^T     both operands from shared memory (K-major)
//                O_t (D fp32 columns)   += P_t . V_j       P_t from tensor memory, V_j MN-major from its row-major tile
//              issue order per key tile j:  P.V_A(j), Q.K_A(j+1), P.V_B(j), Q.K_B(j+1).
//   warps 2-5  softmax of tile A, warps 6-9 softmax of tile B; thread r owns row r of its tile. The row of S is
//              read from TMEM once into registers; P = exp2(S*scale*log2e - m) in fp32 is packed to the storage
//              type and written over the first 64 columns of S_t (tcgen05.st), which the P.V MMA reads as its A
//              operand. The running maximum is raised only when it grows by more than 8 (factor 256), so O_t in
//              TMEM is rescaled rarely; row sums stay in fp32. After the last key tile the same warps read O_t,
//              divide by the row sum and store.
// Ordering notes: tcgen05.commit covers every MMA issued before it, so "S_t(j) ready" also means P.V_t(j-1) has
// finished and O_t may be rescaled; Q.K_t(j+1) overwrites the columns P_t(j) lives in and is issued after
// P.V_t(j) by the same thread, which the tensor pipe executes in order.
// Masking: keys >= kv_len[b] (or >= Skv) and, for causal, keys > row + (Skv - Sq) get probability 0; key tiles
// entirely above a query tile's diagonal are skipped for that tile.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace {

    constexpr int BM = 128, BN = 128; // rows per query tile, keys per key tile
    constexpr int kQTiles    = 2;
    constexpr int kThreads   = 64 + kQTiles * 128;
    constexpr int kTmemCols  = 512;
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

    template <int D, int KS, int VS> struct Smem {
        static constexpr uint32_t Q_BYTES  = BM * D * 2; // per query tile
        static constexpr uint32_t KV_BYTES = BN * D * 2;
        static constexpr uint32_t oQ   = 0;
        static constexpr uint32_t oK   = oQ + kQTiles * Q_BYTES;
        static constexpr uint32_t oV   = oK + KS * KV_BYTES;
        static constexpr uint32_t oBar = oV + VS * KV_BYTES;
        // barriers: q_full, k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[2], p_full[2], o_final[2]
        static constexpr int nBar = 1 + 2 * KS + 2 * VS + 6;
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

    template <typename T, int D>
    __global__ void __launch_bounds__(kThreads, 1)
        attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            AttnParams p) {
        constexpr int KS = 2, VS = 2;
        using L               = Smem<D, KS, VS>;
        constexpr bool kBf16  = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdescQK = ptx::idesc_f16(BM, BN, kBf16, false, false);
        constexpr uint32_t kIdescPV = ptx::idesc_f16(BM, D, kBf16, false, true);
        constexpr int      DCH      = D / 64; // 64-element (128-byte) spans per row
        constexpr int      kColS    = 0;      // S_A at 0, S_B at 128; P_t aliases the first 64 columns of S_t
        constexpr int      kColO    = 256;    // O_A at 256, O_B at 256 + D

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sQ = base + L::oQ, sK = base + L::oK, sV = base + L::oV, sBar = base + L::oBar;
        volatile int  *ctl = (volatile int *) (gbase + L::oCtl); // ctl[0] = tmem base, ctl[1] = abort flag
        auto           bar = [&](int i) { return sBar + 8u * (uint32_t) i; };
        constexpr int  bQ = 0, bKF = 1, bKE = 1 + KS, bVF = 1 + 2 * KS, bVE = 1 + 2 * KS + VS, bSF = 1 + 2 * KS + 2 * VS, bPF = bSF + 2,
                      bOF = bSF + 4;

        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int b = blockIdx.z, h = blockIdx.y;
        const int hk = h / (int) (p.Hq / p.Hkv);
        // heavy (late) query tiles first when causal
        const int     mt = p.causal ? (int) gridDim.x - 1 - (int) blockIdx.x : (int) blockIdx.x;
        const int64_t m0 = (int64_t) mt * (kQTiles * BM);

        int64_t len = p.kv_len ? (int64_t) p.kv_len[b] : p.Skv;
        if (len > p.Skv) len = p.Skv;
        if (len < 0) len = 0;
        // key tiles each query tile needs
        int n_t[kQTiles];
#pragma unroll
        for (int t = 0; t < kQTiles; ++t) {
            int64_t kend = len;
            const int64_t first = m0 + (int64_t) t * BM;
            if (first >= p.Sq) kend = 0; // tile entirely past the end of the query sequence
            if (p.causal && kend > 0) {
                int64_t last = first + BM - 1;
                if (last > p.Sq - 1) last = p.Sq - 1;
                const int64_t lim = last + (p.Skv - p.Sq) + 1;
                if (lim < kend) kend = lim;
                if (kend < 0) kend = 0;
            }
            n_t[t] = (int) ((kend + BN - 1) / BN);
        }
        const int n_max = n_t[0] > n_t[1] ? n_t[0] : n_t[1];

        if (threadIdx.x == 0) {
            for (int i = 0; i < L::nBar; ++i) ptx::mbar_init(bar(i), (i >= bPF && i < bPF + 2) ? 128 : 1);
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
            if (n_max > 0 && ptx::elect_one()) {
                ptx::mbar_expect_tx(bar(bQ), kQTiles * L::Q_BYTES);
#pragma unroll
                for (int t = 0; t < kQTiles; ++t)
#pragma unroll
                    for (int c = 0; c < DCH; ++c)
                        ptx::tma_load_4d(sQ + t * L::Q_BYTES + c * (BM * 128), &tmQ, c * 64, (int) (m0 + t * BM), h, b, bar(bQ));
                for (int j = 0; j < n_max; ++j) {
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
            if (n_max > 0 && ptx::elect_one()) {
                auto issue_qk = [&](int t, int j) {
                    const int ks = j % KS;
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const uint32_t off = (uint32_t) (k / 4) * (BM * 128) + (uint32_t) (k % 4) * 32;
                        const uint64_t ad  = ptx::smem_desc_sw128(sQ + t * L::Q_BYTES + off, 16, 1024);
                        const uint64_t bd  = ptx::smem_desc_sw128(sK + ks * L::KV_BYTES + off, 16, 1024);
                        ptx::mma_f16_ss(tmem + kColS + t * BN, ad, bd, kIdescQK, k != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(bar(bSF + t));
                };
                auto issue_pv = [&](int t, int j) {
                    const int vs = j % VS;
#pragma unroll
                    for (int k = 0; k < BN / 16; ++k) {
                        // V tile: D/64 spans of [128 keys x 128 B]; 16 keys per MMA step = 2048 B
                        const uint64_t bd = ptx::smem_desc_sw128(sV + vs * L::KV_BYTES + k * 2048, BN * 128, 1024);
                        ptx::mma_f16_ts(tmem + kColO + t * D, tmem + kColS + t * BN + k * 8, bd, kIdescPV, (j | k) != 0 ? 1u : 0u);
                    }
                };
                bool ok = ptx::mbar_wait(bar(bQ), 0, ctl + 1, p.dev_err);
                ok      = ok && ptx::mbar_wait(bar(bKF + 0), 0, ctl + 1, p.dev_err);
                if (ok) {
                    ptx::tc_fence_after();
#pragma unroll
                    for (int t = 0; t < kQTiles; ++t)
                        if (n_t[t] > 0) issue_qk(t, 0);
                    ptx::tc_commit(bar(bKE + 0));
                }
                for (int j = 0; j < n_max && ok; ++j) {
                    const int vs = j % VS;
                    ok = ptx::mbar_wait(bar(bVF + vs), (j / VS) & 1, ctl + 1, p.dev_err);
                    const bool more = j + 1 < n_max;
#pragma unroll
                    for (int t = 0; t < kQTiles && ok; ++t) {
                        if (j < n_t[t]) {
                            ok = ptx::mbar_wait(bar(bPF + t), j & 1, ctl + 1, p.dev_err);
                            if (!ok) break;
                            ptx::tc_fence_after();
                            issue_pv(t, j);
                            if (j + 1 < n_t[t]) {
                                ok = ptx::mbar_wait(bar(bKF + (j + 1) % KS), ((j + 1) / KS) & 1, ctl + 1, p.dev_err);
                                if (!ok) break;
                                ptx::tc_fence_after();
                                issue_qk(t, j + 1);
                            } else {
                                ptx::tc_commit(bar(bOF + t)); // O_t complete
                            }
                        }
                    }
                    if (!ok) break;
                    ptx::tc_commit(bar(bVE + vs));
                    if (more) ptx::tc_commit(bar(bKE + (j + 1) % KS));
                }
            }
        } else {
            // ------------------------------------------------------------------ softmax + epilogue (thread = row)
            const int      t      = (warp - 2) >> 2;       // query tile of this warpgroup
            const int      q      = warp & 3;              // TMEM lane quarter this warp may address
            const int      r      = q * 32 + lane;
            const int64_t  row    = m0 + (int64_t) t * BM + r;
            const uint32_t tS     = tmem + ((uint32_t) (q * 32) << 16) + kColS + t * BN;
            const uint32_t tO     = tmem + ((uint32_t) (q * 32) << 16) + kColO + t * D;
            const int64_t  my_lim = p.causal ? row + (p.Skv - p.Sq) : p.Skv; // keys <= my_lim visible
            const int      n      = n_t[t];
            float          m_used = -INFINITY, l = 0.f;
            bool           ok     = true;
            for (int j = 0; j < n; ++j) {
                const int64_t kv0 = (int64_t) j * BN;
                ok = ptx::mbar_wait(bar(bSF + t), j & 1, ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) ptx::tmem_ld_x32(tS + c * 32, s[c]);
                ptx::tc_wait_ld();
                const bool need_mask = (kv0 + BN > len) || (p.causal && kv0 + BN - 1 > m0 + (int64_t) t * BM + (p.Skv - p.Sq));
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int64_t key = kv0 + c * 32 + i;
                            if (!(key < len && key <= my_lim)) s[c][i] = 0xff800000u; // -inf
                        }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    mx0 = fmaxf(mx0, __uint_as_float(s[0][i]));
                    mx1 = fmaxf(mx1, __uint_as_float(s[1][i]));
                    mx2 = fmaxf(mx2, __uint_as_float(s[2][i]));
                    mx3 = fmaxf(mx3, __uint_as_float(s[3][i]));
                }
                const float mxs = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2; // scale > 0
                float       alpha = 1.f;
                bool        rescale = false;
                if (mxs > m_used + kRescaleThreshold || (m_used == -INFINITY && mxs > m_used)) {
                    alpha   = m_used == -INFINITY ? 0.f : fast_exp2(m_used - mxs);
                    rescale = j > 0 && m_used != -INFINITY;
                    m_used  = mxs;
                }
                l *= alpha;
                if (__any_sync(0xffffffffu, rescale)) {
                    // P.V_t(j-1) finished before S_t(j) was signalled, so O_t is quiescent here
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_x32(tO + c * 32, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        ptx::tmem_st_x32(tO + c * 32, v);
                    }
                }
                const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
                float       l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int c = 0; c < 4; c += 2) {
                    uint32_t pk[32];
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc)
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = fast_exp2(fmaf(__uint_as_float(s[c + cc][i]), p.scale_log2, neg_m));
                            const float p1 = fast_exp2(fmaf(__uint_as_float(s[c + cc][i + 1]), p.scale_log2, neg_m));
                            l0 += p0;
                            l1 += p1;
                            pk[cc * 16 + i / 2] = pack2<T>(p0, p1);
                        }
                    ptx::tmem_st_x32(tS + (c / 2) * 32, pk);
                }
                l += l0 + l1;
                ptx::tc_wait_st();
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(bPF + t));
            }
            // epilogue
            if (n > 0 && ok) {
                ok = ptx::mbar_wait(bar(bOF + t), 0, ctl + 1, p.dev_err);
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
                    if (n > 0) {
                        ptx::tmem_ld_x32(tO + c * 32, v);
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

    template <typename T, int D>
    int launch_attn(vkc_ctx *ctx, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const AttnParams &p, int64_t B, cudaStream_t st) {
        auto          kern = attn_prefill_kernel<T, D>;
        constexpr int smem = (int) Smem<D, 2, 2>::total;
        if (int rc = vkc_configure_smem(ctx, kern, smem)) return rc;
        dim3 grid((unsigned) ((p.Sq + kQTiles * BM - 1) / (kQTiles * BM)), (unsigned) p.Hq, (unsigned) B);
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
    if (Sq > INT32_MAX - 2 * BM || Skv > INT32_MAX - BN) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_tcgen05: sequence too long");

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
    if (dtype == VKC_F16) return D == 64 ? launch_attn<__half, 64>(ctx, tq, tk, tv, p, B, st) : launch_attn<__half, 128>(ctx, tq, tk, tv, p, B, st);
    return D == 64 ? launch_attn<__nv_bfloat16, 64>(ctx, tq, tk, tv, p, B, st) : launch_attn<__nv_bfloat16, 128>(ctx, tq, tk, tv, p, B, st);
}
