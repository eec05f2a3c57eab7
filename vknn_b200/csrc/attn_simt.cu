// K2 (SIMT form) — fused attention O = softmax(Q.K^T * scale + mask) . V on the fp32 pipes, one warp per query
// row with an online softmax. This is the Precision::High (fp32 storage) kernel, the kernel for additive-mask
// graphs and for head sizes the tensor-core kernel does not cover; it never materialises the score matrix.
// Per element the arithmetic follows the reference's node order: (q.k) * scale, + mask, max-subtract, expf,
// sum, divide — with the sum carried in fp32 and rescaled online instead of the reference's double.
#include "common.cuh"

int vkc_attn_prefill_tcgen05(vkc_ctx *ctx, const void *Q, const void *K, const void *V, void *O, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                             int64_t Skv, int64_t D, const int64_t *qs, const int64_t *ks, const int64_t *vs, const int64_t *os, float scale,
                             int causal, const int32_t *kv_len, int dtype, const vkc_fanout *fan, cudaStream_t st);

namespace {

    constexpr int kRows = 8;  // query rows (= warps) per CTA
    constexpr int kKeys = 32; // keys per shared-memory block
    constexpr int kMaxD = 256;

    struct AttnSimtParams {
        int64_t        B, Hq, Hkv, Sq, Skv, D;
        int64_t        qs[3], ks[3], vs[3], os[3];
        float          scale;
        int            causal;
        const float   *mask;
        const int32_t *kv_len;
    };

    template <typename T>
    __global__ void __launch_bounds__(kRows * 32) attn_simt_kernel(const T *__restrict__ Q, const T *__restrict__ K, const T *__restrict__ V,
                                                                   T *__restrict__ O, AttnSimtParams p) {
        extern __shared__ float sm[];
        const int     D    = (int) p.D;
        float        *Ks   = sm;                          // [kKeys][D + 1]
        float        *Vs   = Ks + kKeys * (D + 1);        // [kKeys][D]
        float        *Qs   = Vs + kKeys * D;              // [kRows][D]
        const int     warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int64_t b = blockIdx.z, h = blockIdx.y, hk = h / (p.Hq / p.Hkv);
        const int64_t i0 = (int64_t) blockIdx.x * kRows, i = i0 + warp;
        const bool    row_ok = i < p.Sq;
        const T      *qb = Q + b * p.qs[0] + h * p.qs[1];
        const T      *kb = K + b * p.ks[0] + hk * p.ks[1];
        const T      *vb = V + b * p.vs[0] + hk * p.vs[1];

        for (int d = lane; d < D; d += 32) Qs[warp * D + d] = row_ok ? St<T>::ld(qb + i * p.qs[2] + d) : 0.f;

        int64_t len = p.kv_len ? (int64_t) p.kv_len[b] : p.Skv;
        if (len > p.Skv) len = p.Skv;
        int64_t kend = len; // keys any row of this CTA can see
        if (p.causal) {
            int64_t last = i0 + kRows - 1;
            if (last > p.Sq - 1) last = p.Sq - 1;
            int64_t lim = last + (p.Skv - p.Sq) + 1;
            if (lim < kend) kend = lim;
        }
        const int64_t my_lim = p.causal ? i + (p.Skv - p.Sq) : p.Skv; // keys j <= my_lim are visible

        float     m = -INFINITY, l = 0.f;
        float     o[kMaxD / 32];
        const int nd = (D + 31) / 32;
#pragma unroll
        for (int dd = 0; dd < kMaxD / 32; ++dd) o[dd] = 0.f;

        for (int64_t j0 = 0; j0 < kend; j0 += kKeys) {
            __syncthreads();
            for (int e = threadIdx.x; e < kKeys * D; e += kRows * 32) {
                const int     jj = e / D, d = e % D;
                const int64_t j  = j0 + jj;
                const bool    ok = j < len;
                Ks[jj * (D + 1) + d] = ok ? St<T>::ld(kb + j * p.ks[2] + d) : 0.f;
                Vs[jj * D + d]       = ok ? St<T>::ld(vb + j * p.vs[2] + d) : 0.f;
            }
            __syncthreads();
            const int64_t j = j0 + lane;
            float         s = 0.f;
            for (int d = 0; d < D; ++d) s = fmaf(Qs[warp * D + d], Ks[lane * (D + 1) + d], s);
            s = s * p.scale;
            if (p.mask && row_ok && j < p.Skv) s = s + p.mask[i * p.Skv + j];
            if (!row_ok || j >= len || j > my_lim) s = -INFINITY;
            float bm = s;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, off));
            const float m_new = fmaxf(m, bm);
            if (m_new == -INFINITY) continue; // nothing visible yet (warp-uniform)
            const float alpha = expf(m - m_new);
            const float pj    = expf(s - m_new);
            float       ps    = pj;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            l = l * alpha + ps;
            m = m_new;
#pragma unroll
            for (int dd = 0; dd < kMaxD / 32; ++dd) o[dd] *= alpha;
            for (int jj = 0; jj < kKeys; ++jj) {
                const float pv = __shfl_sync(0xffffffffu, pj, jj);
#pragma unroll
                for (int dd = 0; dd < kMaxD / 32; ++dd) {
                    if (dd < nd) {
                        const int d = lane + 32 * dd;
                        if (d < D) o[dd] = fmaf(pv, Vs[jj * D + d], o[dd]);
                    }
                }
            }
        }
        if (row_ok) {
            T          *ob  = O + b * p.os[0] + h * p.os[1] + i * p.os[2];
            const float inv = 1.0f / l; // l == 0 (every key masked) yields NaN, as the reference's 0/0 does
#pragma unroll
            for (int dd = 0; dd < kMaxD / 32; ++dd) {
                const int d = lane + 32 * dd;
                if (dd < nd && d < D) St<T>::st(ob + d, o[dd] * inv);
            }
        }
    }

    template <typename T>
    int launch_attn_simt(vkc_ctx *ctx, const void *Q, const void *K, const void *V, void *O, const AttnSimtParams &p, cudaStream_t st) {
        const size_t smem = sizeof(float) * (size_t) (kKeys * (p.D + 1) + kKeys * p.D + kRows * p.D);
        auto         kern = attn_simt_kernel<T>;
        if (smem > 48 * 1024) {
            if (int rc = vkc_configure_smem(ctx, kern, 100 * 1024)) return rc;
        }
        dim3 grid((unsigned) ((p.Sq + kRows - 1) / kRows), (unsigned) p.Hq, (unsigned) p.B);
        kern<<<grid, kRows * 32, smem, st>>>((const T *) Q, (const T *) K, (const T *) V, (T *) O, p);
        return vkc_post_launch(ctx, "attn_simt");
    }

} // namespace

extern "C" int vkc_attn_prefill(vkc_ctx *ctx, const void *Q, const void *K, const void *V, void *O, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                                int64_t Skv, int64_t D, const int64_t *q_strides, const int64_t *k_strides, const int64_t *v_strides,
                                const int64_t *o_strides, float scale, int causal, const float *mask, const int32_t *kv_len, int dtype,
                                vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, B >= 0 && Hq >= 1 && Hkv >= 1 && Sq >= 0 && Skv >= 0 && D >= 1, "attn_prefill: bad extents");
    VKC_REQUIRE(ctx, Hq % Hkv == 0, "attn_prefill: Hq=%lld is not a multiple of Hkv=%lld", (long long) Hq, (long long) Hkv);
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "attn_prefill: bad dtype %d", dtype);
    VKC_REQUIRE(ctx, D <= kMaxD, "attn_prefill: head dim %lld exceeds %d", (long long) D, kMaxD);
    if (B == 0 || Sq == 0) return VKC_OK;
    VKC_REQUIRE(ctx, Skv >= 1, "attn_prefill: empty key sequence");
    VKC_REQUIRE(ctx, Q && K && V && O, "attn_prefill: null tensor");
    VKC_REQUIRE(ctx, Hq <= 65535 && B <= 65535, "attn_prefill: grid too large");
    cudaStream_t st = vkc_pick_stream(ctx, stream);

    AttnSimtParams p;
    p.B = B, p.Hq = Hq, p.Hkv = Hkv, p.Sq = Sq, p.Skv = Skv, p.D = D;
    const int64_t dq[3] = {Hq * Sq * D, Sq * D, D}, dk[3] = {Hkv * Skv * D, Skv * D, D};
    for (int i = 0; i < 3; ++i) {
        p.qs[i] = q_strides ? q_strides[i] : dq[i];
        p.ks[i] = k_strides ? k_strides[i] : dk[i];
        p.vs[i] = v_strides ? v_strides[i] : dk[i];
        p.os[i] = o_strides ? o_strides[i] : dq[i];
    }
    p.scale = scale, p.causal = causal ? 1 : 0, p.mask = mask, p.kv_len = kv_len;

    const bool tc_shape = dtype != VKC_F32 && !mask && (D == 64 || D == 128);
    if (tc_shape && ctx->impl != VKC_IMPL_SIMT) {
        int rc = vkc_attn_prefill_tcgen05(ctx, Q, K, V, O, B, Hq, Hkv, Sq, Skv, D, p.qs, p.ks, p.vs, p.os, scale, p.causal, kv_len, dtype, nullptr, st);
        if (rc != VKC_ERR_UNSUPPORTED || ctx->impl == VKC_IMPL_TCGEN05) return rc;
    } else if (ctx->impl == VKC_IMPL_TCGEN05) {
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill: the tensor-core kernel needs 16-bit storage, no additive mask and D in {64,128}");
    }
    switch (dtype) {
        case VKC_F32: return launch_attn_simt<float>(ctx, Q, K, V, O, p, st);
        case VKC_F16: return launch_attn_simt<__half>(ctx, Q, K, V, O, p, st);
        default: return launch_attn_simt<__nv_bfloat16>(ctx, Q, K, V, O, p, st);
    }
}

extern "C" int vkc_attn_prefill_fanout(vkc_ctx *ctx, const void *Q, const void *K, const void *V, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                                       int64_t Skv, int64_t D, const int64_t *q_strides, const int64_t *k_strides, const int64_t *v_strides,
                                       const int64_t *o_strides, float scale, int causal, const int32_t *kv_len, int dtype, const vkc_fanout *fan,
                                       vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, fan, "attn_prefill_fanout: null fan-out description");
    VKC_REQUIRE(ctx, B >= 1 && Hq >= 1 && Hkv >= 1 && Sq >= 1 && Skv >= 1 && D >= 1, "attn_prefill_fanout: bad extents");
    VKC_REQUIRE(ctx, Hq % Hkv == 0, "attn_prefill_fanout: Hq=%lld is not a multiple of Hkv=%lld", (long long) Hq, (long long) Hkv);
    VKC_REQUIRE(ctx, Q && K && V, "attn_prefill_fanout: null tensor");
    VKC_REQUIRE(ctx, Hq <= 65535 && B <= 65535, "attn_prefill_fanout: grid too large");
    if ((dtype != VKC_F16 && dtype != VKC_BF16) || (D != 64 && D != 128))
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_fanout: needs the tensor-core kernel (16-bit storage, D in {64,128})");
    int64_t       qs[3], ks[3], vs[3], os[3];
    const int64_t dq[3] = {Hq * Sq * D, Sq * D, D}, dk[3] = {Hkv * Skv * D, Skv * D, D};
    for (int i = 0; i < 3; ++i) {
        qs[i] = q_strides ? q_strides[i] : dq[i];
        ks[i] = k_strides ? k_strides[i] : dk[i];
        vs[i] = v_strides ? v_strides[i] : dk[i];
        os[i] = o_strides ? o_strides[i] : dq[i];
    }
    return vkc_attn_prefill_tcgen05(ctx, Q, K, V, nullptr, B, Hq, Hkv, Sq, Skv, D, qs, ks, vs, os, scale, causal ? 1 : 0, kv_len, dtype, fan,
                                    vkc_pick_stream(ctx, stream));
}
