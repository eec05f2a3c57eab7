// K3 — single-query (decode) attention over a KV cache with grouped query heads, HBM-bound.
//
// The cache is split along its length into fixed chunks; one CTA owns one (sequence, kv head, chunk) and
// serves all G = Hq/Hkv query heads of the group from registers, so every K and V row is read from HBM
// exactly once, with 128-bit loads that are contiguous across the 8 lanes sharing a row (4 rows per warp
// instruction). Dot products are reduced with warp shuffles, the softmax is online in fp32 (exp2 with the
// scale folded in), and each CTA writes one partial (max, sum, o) per query head to a scratch buffer that
// a small second kernel merges. Sequences shorter than Lmax simply launch fewer working CTAs: per-sequence
// kv_len bounds both the chunk count and the last chunk.
//
// Algorithmic bytes per call: sum_b 2 * Hkv * kv_len[b] * D * sizeof(T)  (+ Q and O).
#include "common.cuh"
#include <mutex>
#include <cstdlib>

int vkc_attn_decode_tcgen05(vkc_ctx *ctx, const void *Q, const void *Kc, const void *Vc, int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D,
                            const int32_t *kv_len, float scale, float *part_ml, float *part_o, int *nslots, int min_tiles, int parts_stride, int dtype,
                            cudaStream_t st);

namespace {

    constexpr int kWarps = 4;

    __host__ __device__ inline int decode_chunk(int64_t B, int64_t Hkv, int64_t Lmax) {
        int chunk = 512;
        while (chunk > 128 && B * Hkv * ((Lmax + chunk - 1) / chunk) < 2 * 148) chunk >>= 1;
        return chunk;
    }

    // Partial slots per (sequence, query head) the scratch must hold: enough for either kernel form. The tensor-core
    // form gives every CTA an equal run of at least 2 * chunk keys, wherever the run starts, so a (sequence, kv head)
    // unit is cut into at most ceil(Lmax / (2 * chunk)) + 1 pieces, with two slots each.
    __host__ __device__ inline int decode_slots(int64_t Lmax, int chunk) { return 2 * ((int) ((Lmax + 2 * chunk - 1) / (2 * chunk)) + 1); }

    template <typename T> __device__ __forceinline__ void unpack8(const uint4 &raw, float (&f)[8]);
    template <> __device__ __forceinline__ void unpack8<__half>(const uint4 &raw, float (&f)[8]) {
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 t = __half22float2(h[i]);
            f[2 * i]       = t.x;
            f[2 * i + 1]   = t.y;
        }
    }
    template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4 &raw, float (&f)[8]) {
        const uint32_t *u = reinterpret_cast<const uint32_t *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i]     = __uint_as_float(u[i] << 16);
            f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }

    // CH = 16-byte chunks of a row held per lane: D = CH * 64 elements of a 16-bit type. G = query heads per kv head.
    template <typename T, int CH, int G>
    __global__ void __launch_bounds__(kWarps * 32) attn_decode_kernel(const T *__restrict__ Q, const T *__restrict__ Kc, const T *__restrict__ Vc,
                                                                      float *__restrict__ part_ml, float *__restrict__ part_o,
                                                                      const int32_t *__restrict__ kv_len, int64_t Hkv, int64_t Lmax, float scale_log2,
                                                                      int chunk, int max_splits) {
        constexpr int D  = CH * 64;
        constexpr int DL = CH * 8; // dims per lane
        const int     b = blockIdx.z, hk = blockIdx.y, split = blockIdx.x;
        int64_t       len = kv_len ? (int64_t) kv_len[b] : Lmax;
        if (len > Lmax) len = Lmax;
        const int64_t start = (int64_t) split * chunk;
        if (start >= len) return;
        const int64_t end = start + chunk < len ? start + chunk : len;

        const int     warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int     sub = lane & 7, slot = lane >> 3;
        const int64_t Hq = Hkv * G;

        // this lane's slice of the G query rows: dims [c*64 + sub*8, +8) for c < CH, pre-scaled by scale*log2(e)
        float q[G][DL];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const T *qr = Q + ((int64_t) b * Hq + (int64_t) hk * G + g) * D;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(qr + c * 64 + sub * 8);
                float       f[8];
                unpack8<T>(raw, f);
#pragma unroll
                for (int e = 0; e < 8; ++e) q[g][c * 8 + e] = f[e] * scale_log2;
            }
        }
        float m[G], l[G], o[G][DL];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.f;
#pragma unroll
            for (int e = 0; e < DL; ++e) o[g][e] = 0.f;
        }

        const T *kbase = Kc + ((int64_t) b * Hkv + hk) * Lmax * D;
        const T *vbase = Vc + ((int64_t) b * Hkv + hk) * Lmax * D;

        // keys are dealt to (warp, slot) pairs round-robin in steps of 4 * kWarps
        uint4   kr[CH], vr[CH], kn[CH], vn[CH];
        int64_t j = start + warp * 4 + slot;
        auto    load_row = [&](int64_t jj, uint4(&kk)[CH], uint4(&vv)[CH]) {
            if (jj < end) {
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    kk[c] = __ldg(reinterpret_cast<const uint4 *>(kbase + jj * D + c * 64 + sub * 8));
                    vv[c] = __ldg(reinterpret_cast<const uint4 *>(vbase + jj * D + c * 64 + sub * 8));
                }
            } else {
#pragma unroll
                for (int c = 0; c < CH; ++c) {
                    kk[c] = make_uint4(0, 0, 0, 0);
                    vv[c] = make_uint4(0, 0, 0, 0);
                }
            }
        };
        load_row(j, kr, vr);
        const int64_t jstep = 4 * kWarps;
        // every lane of the warp runs the same number of iterations (shuffles below are warp-wide)
        const int64_t jwarp_first = start + warp * 4;
        for (int64_t jw = jwarp_first; jw < end; jw += jstep, j += jstep) {
            load_row(j + jstep, kn, vn); // software prefetch of the next row
            float s[G];
#pragma unroll
            for (int g = 0; g < G; ++g) s[g] = 0.f;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                float f[8];
                unpack8<T>(kr[c], f);
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int e = 0; e < 8; ++e) s[g] = fmaf(q[g][c * 8 + e], f[e], s[g]);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                s[g] += __shfl_xor_sync(0xffffffffu, s[g], 1);
                s[g] += __shfl_xor_sync(0xffffffffu, s[g], 2);
                s[g] += __shfl_xor_sync(0xffffffffu, s[g], 4);
            }
            const bool valid = j < end;
            float      pr[G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float sg = valid ? s[g] : -INFINITY;
                if (sg > m[g]) {
                    const float alpha = exp2f(m[g] - sg);
                    l[g] *= alpha;
#pragma unroll
                    for (int e = 0; e < DL; ++e) o[g][e] *= alpha;
                    m[g] = sg;
                }
                pr[g] = valid ? exp2f(sg - m[g]) : 0.f;
                l[g] += pr[g];
            }
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                float f[8];
                unpack8<T>(vr[c], f);
#pragma unroll
                for (int g = 0; g < G; ++g)
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[g][c * 8 + e] = fmaf(pr[g], f[e], o[g][c * 8 + e]);
            }
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                kr[c] = kn[c];
                vr[c] = vn[c];
            }
        }

        // merge the 4 key slots of the warp (lanes with equal `sub`), then the warps through shared memory
#pragma unroll
        for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
                const float lo = __shfl_xor_sync(0xffffffffu, l[g], off);
                const float mn = fmaxf(m[g], mo);
                const float a  = mn == -INFINITY ? 0.f : exp2f(m[g] - mn);
                const float bo = mn == -INFINITY ? 0.f : exp2f(mo - mn);
                l[g]           = l[g] * a + lo * bo;
#pragma unroll
                for (int e = 0; e < DL; ++e) {
                    const float oo = __shfl_xor_sync(0xffffffffu, o[g][e], off);
                    o[g][e]        = o[g][e] * a + oo * bo;
                }
                m[g] = mn;
            }
        }
        __shared__ float sm_m[kWarps][G], sm_l[kWarps][G];
        __shared__ float sm_o[kWarps][G][D];
        if (slot == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                if (sub == 0) {
                    sm_m[warp][g] = m[g];
                    sm_l[warp][g] = l[g];
                }
#pragma unroll
                for (int c = 0; c < CH; ++c)
#pragma unroll
                    for (int e = 0; e < 8; ++e) sm_o[warp][g][c * 64 + sub * 8 + e] = o[g][c * 8 + e];
            }
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < G * D; idx += kWarps * 32) {
            const int g = idx / D, d = idx % D;
            float     mt = -INFINITY;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) mt = fmaxf(mt, sm_m[w][g]);
            float lt = 0.f, ot = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float a = sm_m[w][g] == -INFINITY ? 0.f : exp2f(sm_m[w][g] - mt);
                lt += sm_l[w][g] * a;
                ot += sm_o[w][g][d] * a;
            }
            const int64_t hq  = (int64_t) hk * G + g;
            const int64_t row = ((int64_t) b * Hq + hq) * max_splits + split;
            part_o[row * D + d] = ot;
            if (d == 0) {
                part_ml[row * 2 + 0] = mt;
                part_ml[row * 2 + 1] = lt;
            }
        }
    }

    // One CTA per (sequence, query head): merges the per-chunk partials and writes the output row.
    template <typename T>
    __global__ void attn_decode_combine_kernel(const float *__restrict__ part_ml, const float *__restrict__ part_o, T *__restrict__ O,
                                               const int32_t *__restrict__ kv_len, int64_t Hq, int64_t Lmax, int D, int chunk,
                                               const int *__restrict__ nslots, int G, int max_splits) {
        const int b = blockIdx.y, hq = blockIdx.x;
        int64_t   len = kv_len ? (int64_t) kv_len[b] : Lmax;
        if (len > Lmax) len = Lmax;
        // partial slots this (sequence, head) filled: one per chunk, or what the tensor-core form recorded for the kv head
        const int     ns  = len <= 0 ? 0 : (nslots ? nslots[(int64_t) b * (Hq / G) + hq / G] : (int) ((len + chunk - 1) / chunk));
        const int64_t row = ((int64_t) b * Hq + hq) * max_splits;
        float         mt  = -INFINITY;
        for (int s = 0; s < ns; ++s) mt = fmaxf(mt, part_ml[(row + s) * 2]);
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float lt = 0.f, ot = 0.f;
            for (int s = 0; s < ns; ++s) {
                const float ms = part_ml[(row + s) * 2];
                const float a  = ms == -INFINITY ? 0.f : exp2f(ms - mt);
                lt += part_ml[(row + s) * 2 + 1] * a;
                ot += part_o[(row + s) * D + d] * a;
            }
            St<T>::st(O + ((int64_t) b * Hq + hq) * D + d, ot / lt); // len == 0 gives 0/0 = NaN like the reference
        }
    }

    template <typename T, int CH>
    int launch_decode(vkc_ctx *ctx, const void *Q, const void *Kc, const void *Vc, void *O, int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax,
                      const int32_t *kv_len, float scale, float *ws, cudaStream_t st) {
        const int     G          = (int) (Hq / Hkv);
        const int     chunk      = decode_chunk(B, Hkv, Lmax);
        const int     max_splits = decode_slots(Lmax, chunk); // slot stride; the SIMT form fills ceil(Lmax/chunk) of them
        constexpr int D          = CH * 64;
        float        *part_ml    = ws;
        float        *part_o     = ws + (size_t) B * Hq * max_splits * 2;
        int          *nslots     = reinterpret_cast<int *>(part_o + (size_t) B * Hq * max_splits * D); // [B][Hkv], tensor-core form only
        const float   sl2        = scale * 1.4426950408889634f;
        dim3          grid((unsigned) max_splits, (unsigned) Hkv, (unsigned) B);
        bool          split_done = false;
        if (ctx->impl != VKC_IMPL_SIMT) {
            const int dtype = std::is_same<T, __half>::value ? VKC_F16 : VKC_BF16;
            int       rc    = vkc_attn_decode_tcgen05(ctx, Q, Kc, Vc, B, Hq, Hkv, Lmax, D, kv_len, scale, part_ml, part_o, nslots, 2 * chunk / 128, max_splits, dtype, st);
            if (rc == VKC_OK) split_done = true;
            else if (rc != VKC_ERR_UNSUPPORTED || ctx->impl == VKC_IMPL_TCGEN05) return rc;
        }
#define VKC_DEC(G_)                                                                                                                    \
    attn_decode_kernel<T, CH, G_><<<grid, kWarps * 32, 0, st>>>((const T *) Q, (const T *) Kc, (const T *) Vc, part_ml, part_o, kv_len, Hkv, \
                                                                Lmax, sl2, chunk, max_splits)
        if (!split_done) switch (G) {
            case 1: VKC_DEC(1); break;
            case 2: VKC_DEC(2); break;
            case 4: VKC_DEC(4); break;
            case 8: VKC_DEC(8); break;
            default: return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_decode: group size %d (Hq/Hkv) must be 1, 2, 4 or 8", G);
        }
#undef VKC_DEC
        if (!split_done) {
            int rc = vkc_post_launch(ctx, "attn_decode");
            if (rc) return rc;
        }
        dim3 cgrid((unsigned) Hq, (unsigned) B);
        attn_decode_combine_kernel<T><<<cgrid, D < 128 ? D : 128, 0, st>>>(part_ml, part_o, (T *) O, kv_len, Hq, Lmax, D, chunk, split_done ? nslots : nullptr, G,
                                                                           max_splits);
        return vkc_post_launch(ctx, "attn_decode_combine");
    }

} // namespace

// ---- fixed scratch for vkc_attn_decode_noalloc ------------------------------------------------------------------
// The array lives in every GPU's memory from the moment the library is loaded there until the process exits.
// On the host its name is only a handle: the device address has to be asked for, once per device, with that
// device current.
constexpr size_t kStaticScratchBytes = (size_t) 16 << 20;
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
static void      *g_decode_static_ptr[kMaxDevices] = {nullptr};
static std::mutex g_decode_static_mu; // guards the one-time address lookup (host threads may make their first calls together)

extern "C" size_t vkc_attn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Lmax <= 0 || D <= 0) return 0;
    const int    chunk      = decode_chunk(B, Hkv, Lmax);
    const size_t max_splits = (size_t) decode_slots(Lmax, chunk);
    return (size_t) B * (size_t) Hq * max_splits * (size_t) (D + 2) * sizeof(float) + (size_t) B * (size_t) Hkv * sizeof(int);
}

int vkc_attn_decode_tc_items(int sm_count, int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D, const int32_t *kv_len, int min_tiles,
                             int parts_stride, int cta, int32_t *items, int max_items, int *grid_out);

extern "C" int vkc_attn_decode_items(int sm_count, int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D, const int32_t *kv_len_host, int cta,
                                     int32_t *items, int max_items, int32_t *plan) {
    if (sm_count < 1 || B < 1 || Hq < 1 || Hkv < 1 || Lmax < 1 || Hq % Hkv || (!items && max_items > 0)) return VKC_ERR_INVALID;
    const int chunk = decode_chunk(B, Hkv, Lmax), slots = decode_slots(Lmax, chunk);
    int       grid  = 0;
    const int n     = vkc_attn_decode_tc_items(sm_count, B, Hq, Hkv, Lmax, D, kv_len_host, 2 * chunk / 128, slots, cta, items, max_items, &grid);
    if (plan) plan[0] = grid, plan[1] = slots, plan[2] = 2 * chunk / 128;
    return n < 0 ? (grid > 0 ? VKC_ERR_INVALID : VKC_ERR_UNSUPPORTED) : n;
}

extern "C" int vkc_attn_decode(vkc_ctx *ctx, const void *Q, const void *Kc, const void *Vc, void *O, int64_t B, int64_t Hq, int64_t Hkv,
                               int64_t Lmax, int64_t D, const int32_t *kv_len, float scale, void *workspace, size_t workspace_bytes, int dtype,
                               vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, B >= 0 && Hq >= 1 && Hkv >= 1 && Lmax >= 1 && D >= 1, "attn_decode: bad extents");
    VKC_REQUIRE(ctx, Hq % Hkv == 0, "attn_decode: Hq=%lld is not a multiple of Hkv=%lld", (long long) Hq, (long long) Hkv);
    if (dtype != VKC_F16 && dtype != VKC_BF16) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_decode: the KV cache must be f16 or bf16");
    if (D != 64 && D != 128 && D != 256) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_decode: head dim %lld not in {64,128,256}", (long long) D);
    if (B == 0) return VKC_OK;
    VKC_REQUIRE(ctx, Q && Kc && Vc && O, "attn_decode: null tensor");
    VKC_REQUIRE(ctx, B <= 65535 && Hkv <= 65535, "attn_decode: grid too large");
    VKC_REQUIRE(ctx, !(((uintptr_t) Q | (uintptr_t) Kc | (uintptr_t) Vc) & 15), "attn_decode: Q/K/V must be 16-byte aligned");
    const size_t need = vkc_attn_decode_workspace_bytes(B, Hq, Hkv, Lmax, D);
    float       *ws   = (float *) workspace;
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    if (!ws) {
        int rc = vkc_ensure_scratch(ctx, need, st);
        if (rc) return rc;
        ws = (float *) ctx->scratch;
    } else {
        VKC_REQUIRE(ctx, workspace_bytes >= need, "attn_decode: workspace of %zu bytes is smaller than the %zu required", workspace_bytes, need);
    }
#define VKC_DEC_T(T)                                                                                         \
    (D == 64 ? launch_decode<T, 1>(ctx, Q, Kc, Vc, O, B, Hq, Hkv, Lmax, kv_len, scale, ws, st)                \
             : D == 128 ? launch_decode<T, 2>(ctx, Q, Kc, Vc, O, B, Hq, Hkv, Lmax, kv_len, scale, ws, st)     \
                        : launch_decode<T, 4>(ctx, Q, Kc, Vc, O, B, Hq, Hkv, Lmax, kv_len, scale, ws, st))
    if (dtype == VKC_F16) return VKC_DEC_T(__half);
    return VKC_DEC_T(__nv_bfloat16);
#undef VKC_DEC_T
}

extern "C" size_t vkc_attn_decode_noalloc_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int vkc_attn_decode_noalloc(vkc_ctx *ctx, const void *Q, const void *Kc, const void *Vc, void *O, int64_t B, int64_t Hq, int64_t Hkv,
                                       int64_t Lmax, int64_t D, const int32_t *kv_len, float scale, int dtype, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, ctx->device >= 0 && ctx->device < kMaxDevices, "attn_decode_noalloc: device ordinal %d out of range", ctx->device);
    const size_t need = vkc_attn_decode_workspace_bytes(B, Hq, Hkv, Lmax, D);
    if (need > kStaticScratchBytes)
        return vkc_fail(ctx, VKC_ERR_INVALID,
                        "attn_decode_noalloc: this shape needs %zu bytes of partial-result scratch, more than the fixed %zu-byte area; "
                        "use vkc_attn_decode with a caller workspace instead",
                        need, kStaticScratchBytes);
    void *area = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_decode_static_mu);
        area = g_decode_static_ptr[ctx->device];
    }
    if (!area) {
        // one-time set-up for this device: resolve the device address of the file-scope array. With lazy module loading this
        // is also the moment the driver places the library's code and the array itself on the device.
        std::lock_guard<std::mutex> lk(g_decode_static_mu);
        int cur = -1;
        VKC_CUDA(ctx, cudaGetDevice(&cur));
        if (cur != ctx->device) VKC_CUDA(ctx, cudaSetDevice(ctx->device));
        void       *ptr = nullptr;
        cudaError_t e   = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
        if (cur != ctx->device) cudaSetDevice(cur);
        if (e != cudaSuccess || !ptr) return vkc_fail(ctx, VKC_ERR_CUDA, "cudaGetSymbolAddress(decode scratch): %s", cudaGetErrorString(e));
        g_decode_static_ptr[ctx->device] = ptr;
        area                             = ptr;
    }
    // Nothing in the area has to start at zero: the split kernel writes every (row, split) partial that the merge
    // kernel reads for this call, and stale contents beyond them are never read.
    return vkc_attn_decode(ctx, Q, Kc, Vc, O, B, Hq, Hkv, Lmax, D, kv_len, scale, area, kStaticScratchBytes, dtype,
                           stream);
}
