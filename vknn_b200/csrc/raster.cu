// K6 — 3D Gaussian-splatting rasterizer (the step after the encoder): project, depth-sort, composite.
//
// Follows the reference's CPU specification of the renderer, scripts/yonosplat/ref_rasterizer.py:22-75 (its compute
// shaders shaders/raster_{preprocess,duplicate,bitonic,ranges,composite,fill}.comp implement the same pipeline with a
// per-tile key sort): every pixel composites, front to back in camera depth, exactly the gaussians whose pixel box
// covers it.
//
//   raster_preprocess_kernel  one thread per gaussian: camera-space mean, 2D covariance J (R S R^T) J^T + 0.3 I, conic,
//                             3-sigma radius, pixel box clipped to the image, validity (z > near, det > 1e-12); emits a
//                             record and a sort key (depth bits, invalid gaussians last).
//   raster_sort_*             bitonic sort of (key, index) pairs: blocks of 2048 pairs in shared memory for the short
//                             strides, one global pass per longer stride. Ties are broken by index, so the order is a
//                             pure function of the inputs.
//   raster_composite_kernel   one CTA per 16x16 pixel tile, one thread per pixel. The CTA walks the sorted records in
//                             chunks of 256; each thread tests one record's pixel box against the tile and the hits are
//                             compacted in order into shared memory (ballot prefix), then every pixel thread composites
//                             the compacted records: alpha = min(0.99, opacity * exp(min(power, 0))), gated at 1/255,
//                             C += alpha * T * colour, T *= 1 - alpha. No binning pass and no duplicated keys: the
//                             records (a few MB) stay in L2 and each tile streams them once. When the image has few tiles
//                             the depth order is cut into segments, one CTA per (tile, segment), and a combine kernel
//                             joins the segments' (C, T) pairs in order, so that the whole GPU is busy.
// Arithmetic is templated: double (default: decisions such as the radius ceiling and the 1/255 gate fall exactly as in
// the float64 specification) or float.
#include "common.cuh"

namespace {

    constexpr int kTile = 16;

    template <typename F> struct Rec {
        F   u, v, a, b, c, opac, r, g, bl;
        int x0, x1, y0, y1; // pixel box [x0, x1) x [y0, y1); x0 >= x1 marks an invalid record
    };

    struct Cam {
        double r[9], t[3], fx, fy, cx, cy, znear;
        int    H, W;
    };

    template <typename F>
    __global__ void __launch_bounds__(256) raster_preprocess_kernel(const float *__restrict__ means, const float *__restrict__ covs,
                                                                    const float *__restrict__ colors, const float *__restrict__ opac, int64_t n,
                                                                    int64_t npad, Cam cam, Rec<F> *__restrict__ rec,
                                                                    unsigned long long *__restrict__ keys, unsigned *__restrict__ idx) {
        const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= npad) return;
        unsigned long long key = ~0ull; // padding and invalid gaussians sort last
        idx[i]                 = (unsigned) i;
        if (i < n) {
            Rec<F> o;
            o.x0 = o.y0 = 0, o.x1 = o.y1 = 0;
            const F R[9] = {(F) cam.r[0], (F) cam.r[1], (F) cam.r[2], (F) cam.r[3], (F) cam.r[4], (F) cam.r[5], (F) cam.r[6], (F) cam.r[7], (F) cam.r[8]};
            const F m[3] = {(F) means[3 * i], (F) means[3 * i + 1], (F) means[3 * i + 2]};
            F       p[3];
#pragma unroll
            for (int a = 0; a < 3; ++a) p[a] = m[0] * R[a * 3] + m[1] * R[a * 3 + 1] + m[2] * R[a * 3 + 2] + (F) cam.t[a];
            const F z = p[2], fx = (F) cam.fx, fy = (F) cam.fy;
            F       S[9], T[9], Sc[9];
#pragma unroll
            for (int k = 0; k < 9; ++k) S[k] = (F) covs[9 * i + k];
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int b = 0; b < 3; ++b) T[a * 3 + b] = R[a * 3] * S[b] + R[a * 3 + 1] * S[3 + b] + R[a * 3 + 2] * S[6 + b];
#pragma unroll
            for (int a = 0; a < 3; ++a)
#pragma unroll
                for (int b = 0; b < 3; ++b) Sc[a * 3 + b] = T[a * 3] * R[b * 3] + T[a * 3 + 1] * R[b * 3 + 1] + T[a * 3 + 2] * R[b * 3 + 2];
            const F J00 = fx / z, J02 = -fx * p[0] / (z * z), J11 = fy / z, J12 = -fy * p[1] / (z * z);
            F       JS0[3], JS1[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                JS0[k] = J00 * Sc[k] + J02 * Sc[6 + k];
                JS1[k] = J11 * Sc[3 + k] + J12 * Sc[6 + k];
            }
            const F c00 = JS0[0] * J00 + JS0[2] * J02 + (F) 0.3;
            const F c01 = JS0[1] * J11 + JS0[2] * J12;
            const F c11 = JS1[1] * J11 + JS1[2] * J12 + (F) 0.3;
            const F det = c00 * c11 - c01 * c01;
            if (z > (F) cam.znear && det > (F) 1e-12) {
                const F   mid = (F) 0.5 * (c00 + c11);
                const F   lam = mid + sqrt(fmax((F) 0.1, mid * mid - det));
                const F   rad = ceil((F) 3.0 * sqrt(lam));
                const F   u = fx * p[0] / z + (F) cam.cx, v = fy * p[1] / z + (F) cam.cy;
                // pixel box of the specification: [max(0, floor(u - r)), min(W, ceil(u + r) + 1)); saturate before the
                // conversion so that far-away means cannot overflow the integer
                const F   lim = (F) 1e9;
                const int x0  = (int) fmax((F) 0, fmin(lim, floor(u - rad)));
                const int x1  = (int) fmin((F) cam.W, fmax(-lim, ceil(u + rad) + (F) 1));
                const int y0  = (int) fmax((F) 0, fmin(lim, floor(v - rad)));
                const int y1  = (int) fmin((F) cam.H, fmax(-lim, ceil(v + rad) + (F) 1));
                if (x0 < x1 && y0 < y1) {
                    o.u = u, o.v = v;
                    o.a = c11 / det, o.b = -c01 / det, o.c = c00 / det;
                    o.opac = (F) opac[i];
                    o.r = (F) colors[3 * i], o.g = (F) colors[3 * i + 1], o.bl = (F) colors[3 * i + 2];
                    o.x0 = x0, o.x1 = x1, o.y0 = y0, o.y1 = y1;
                    // z > near > 0: the IEEE bit pattern of a positive double orders like the value
                    key = (unsigned long long) __double_as_longlong((double) z);
                }
            }
            rec[i] = o;
        }
        keys[i] = key;
    }

    __device__ __forceinline__ bool pair_less(unsigned long long ka, unsigned ia, unsigned long long kb, unsigned ib) {
        return ka < kb || (ka == kb && ia < ib);
    }
    __device__ __forceinline__ void cmp_swap(unsigned long long &ka, unsigned &ia, unsigned long long &kb, unsigned &ib, bool up) {
        if (pair_less(kb, ib, ka, ia) == up) {
            unsigned long long tk = ka;
            ka = kb, kb = tk;
            unsigned ti = ia;
            ia = ib, ib = ti;
        }
    }
    constexpr int kSortBlock = 2048; // pairs per CTA in the shared-memory passes (1024 threads, 2 pairs each)

    // Runs every compare-exchange step (k, j) of the bitonic network with k in [k_lo, k_hi] and j < kSortBlock for this
    // CTA's 2048-element block; with k_lo == 2 that is a full sort of each block, later calls finish the short strides of
    // one merge level after the long strides were done in global memory.
    __global__ void __launch_bounds__(1024) raster_sort_local_kernel(unsigned long long *__restrict__ keys, unsigned *__restrict__ idx, int64_t k_lo,
                                                                     int64_t k_hi) {
        __shared__ unsigned long long sk[kSortBlock];
        __shared__ unsigned           si[kSortBlock];
        const int64_t base = (int64_t) blockIdx.x * kSortBlock;
        for (int e = threadIdx.x; e < kSortBlock; e += 1024) sk[e] = keys[base + e], si[e] = idx[base + e];
        __syncthreads();
        for (int64_t k = k_lo; k <= k_hi; k <<= 1) {
            for (int64_t j = (k >> 1) < kSortBlock ? (k >> 1) : (kSortBlock >> 1); j > 0; j >>= 1) {
                const int  t  = threadIdx.x;
                const int  lo = (int) (((t / j) * 2 * j) + (t % j));
                const int  hi = lo + (int) j;
                const bool    up = ((base + lo) & k) == 0;
                cmp_swap(sk[lo], si[lo], sk[hi], si[hi], up);
                __syncthreads();
            }
        }
        for (int e = threadIdx.x; e < kSortBlock; e += 1024) keys[base + e] = sk[e], idx[base + e] = si[e];
    }
    // One compare-exchange step (k, j) with j >= kSortBlock over the whole array.
    __global__ void __launch_bounds__(256) raster_sort_global_kernel(unsigned long long *__restrict__ keys, unsigned *__restrict__ idx, int64_t npad,
                                                                     int64_t k, int64_t j) {
        const int64_t t = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        if (t >= npad / 2) return;
        const int64_t lo = (t / j) * 2 * j + (t % j), hi = lo + j;
        const bool    up = (lo & k) == 0;
        unsigned long long ka = keys[lo], kb = keys[hi];
        unsigned           ia = idx[lo], ib = idx[hi];
        if (pair_less(kb, ib, ka, ia) == up) keys[lo] = kb, keys[hi] = ka, idx[lo] = ib, idx[hi] = ia;
    }

    template <typename F>
    __global__ void __launch_bounds__(256) raster_gather_kernel(const Rec<F> *__restrict__ rec, const unsigned long long *__restrict__ keys,
                                                                const unsigned *__restrict__ idx, int64_t npad, Rec<F> *__restrict__ sorted,
                                                                int *__restrict__ nvalid) {
        const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= npad) return;
        if (keys[i] != ~0ull) {
            sorted[i] = rec[idx[i]];
            if (i + 1 == npad || keys[i + 1] == ~0ull) *nvalid = (int) (i + 1); // valid records form a prefix of the sorted order
        } else if (i == 0) {
            *nvalid = 0;
        }
    }

    template <typename F>
    __global__ void __launch_bounds__(kTile *kTile) raster_composite_kernel(const Rec<F> *__restrict__ sorted, const int *__restrict__ nvalid, int H, int W,
                                                                            float *__restrict__ rgb, float *__restrict__ alpha, F *__restrict__ partial) {
        // hits of the current chunk, split so that the compositing loop reads them with 16-byte shared-memory loads (the
        // loop is bound by those broadcast loads, not by arithmetic): the pixel box, then the nine values padded to VN
        constexpr int VN = sizeof(F) == 4 ? 12 : 10;
        __shared__ __align__(16) int hbox[kTile * kTile][4];
        __shared__ __align__(16) F   hval[kTile * kTile][VN];
        __shared__ int               warp_count[8];
        const int tid = threadIdx.y * kTile + threadIdx.x, lane = tid & 31, warp = tid >> 5;
        const int tx0 = blockIdx.x * kTile, ty0 = blockIdx.y * kTile;
        const int px = tx0 + threadIdx.x, py = ty0 + threadIdx.y;
        const int n  = *nvalid;
        F         C0 = 0, C1 = 0, C2 = 0, T = 1;
        // gridDim.z > 1: this CTA composites only its depth segment of the sorted records (whole chunks of 256) and leaves
        // (C, T) of the segment for the combine kernel: front-to-back compositing is associative in that pair
        const int chunks = (n + kTile * kTile - 1) / (kTile * kTile), per = (chunks + (int) gridDim.z - 1) / (int) gridDim.z;
        const int first = (int) blockIdx.z * per * kTile * kTile;
        const int last  = min(n, first + per * kTile * kTile);
        for (int base = first; base < last; base += kTile * kTile) {
            // each thread tests one record of the chunk against the tile; hits keep their depth order
            Rec<F>    mine;
            bool      take = false;
            const int k    = base + tid;
            if (k < last) {
                mine = sorted[k];
                take = mine.x0 < tx0 + kTile && mine.x1 > tx0 && mine.y0 < ty0 + kTile && mine.y1 > ty0;
            }
            const unsigned bal = __ballot_sync(0xffffffffu, take);
            if (lane == 0) warp_count[warp] = __popc(bal);
            __syncthreads();
            int before = 0, total = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                if (w < warp) before += warp_count[w];
                total += warp_count[w];
            }
            if (take) {
                const int pos = before + __popc(bal & ((1u << lane) - 1u));
                *reinterpret_cast<int4 *>(hbox[pos]) = make_int4(mine.x0, mine.x1, mine.y0, mine.y1);
                F *hv = hval[pos];
                hv[0] = mine.u, hv[1] = mine.v, hv[2] = mine.a, hv[3] = mine.b, hv[4] = mine.c, hv[5] = mine.opac, hv[6] = mine.r, hv[7] = mine.g,
                hv[8] = mine.bl;
            }
            __syncthreads();
            for (int e = 0; e < total; ++e) {
                const int4 bx = *reinterpret_cast<const int4 *>(hbox[e]);
                if (px >= bx.x && px < bx.y && py >= bx.z && py < bx.w) {
                    F gv[VN];
                    if (sizeof(F) == 4) {
#pragma unroll
                        for (int v4 = 0; v4 < 3; ++v4) *reinterpret_cast<float4 *>(&gv[4 * v4]) = *reinterpret_cast<const float4 *>(&hval[e][4 * v4]);
                    } else {
#pragma unroll
                        for (int v2 = 0; v2 < 5; ++v2) *reinterpret_cast<double2 *>(&gv[2 * v2]) = *reinterpret_cast<const double2 *>(&hval[e][2 * v2]);
                    }
                    const F dx = (F) px - gv[0], dy = (F) py - gv[1];
                    const F power = (F) -0.5 * (gv[2] * dx * dx + gv[4] * dy * dy) - gv[3] * dx * dy;
                    const F al    = fmin((F) 0.99, gv[5] * exp(fmin(power, (F) 0)));
                    if (al > (F) (1.0 / 255.0)) {
                        const F w = al * T;
                        C0 += w * gv[6], C1 += w * gv[7], C2 += w * gv[8];
                        T *= (F) 1 - al;
                    }
                }
            }
            __syncthreads();
        }
        if (gridDim.z > 1) {
            if (px < W && py < H) {
                F *o = partial + (((int64_t) blockIdx.z * H + py) * W + px) * 4;
                o[0] = C0, o[1] = C1, o[2] = C2, o[3] = T;
            }
            return;
        }
        if (px < W && py < H) {
            const int64_t o = ((int64_t) py * W + px) * 3;
            rgb[o]     = (float) fmin((F) 1, fmax((F) 0, C0));
            rgb[o + 1] = (float) fmin((F) 1, fmax((F) 0, C1));
            rgb[o + 2] = (float) fmin((F) 1, fmax((F) 0, C2));
            if (alpha) alpha[(int64_t) py * W + px] = (float) ((F) 1 - T);
        }
    }

    // Joins the depth segments of a pixel in order: C = C_0 + T_0 C_1 + T_0 T_1 C_2 + ..., T = T_0 T_1 ...
    template <typename F>
    __global__ void __launch_bounds__(256) raster_combine_kernel(const F *__restrict__ partial, int segs, int H, int W, float *__restrict__ rgb,
                                                                 float *__restrict__ alpha) {
        const int64_t i = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= (int64_t) H * W) return;
        F C0 = 0, C1 = 0, C2 = 0, T = 1;
        for (int s = 0; s < segs; ++s) {
            const F *p = partial + ((int64_t) s * H * W + i) * 4;
            C0 += T * p[0], C1 += T * p[1], C2 += T * p[2];
            T *= p[3];
        }
        rgb[i * 3]     = (float) fmin((F) 1, fmax((F) 0, C0));
        rgb[i * 3 + 1] = (float) fmin((F) 1, fmax((F) 0, C1));
        rgb[i * 3 + 2] = (float) fmin((F) 1, fmax((F) 0, C2));
        if (alpha) alpha[i] = (float) ((F) 1 - T);
    }

    // Depth segments per tile: enough CTAs to fill the SMs several times over when the image has few tiles.
    int raster_segments(int H, int W, int sms) {
        const int64_t tiles = (int64_t) ((W + kTile - 1) / kTile) * ((H + kTile - 1) / kTile);
        int64_t       s     = (8 * (int64_t) sms + tiles - 1) / tiles;
        return (int) (s < 1 ? 1 : (s > 32 ? 32 : s));
    }

    int64_t pad_pow2(int64_t n) {
        int64_t p = kSortBlock;
        while (p < n) p <<= 1;
        return p;
    }

    template <typename F>
    int run_raster(vkc_ctx *ctx, const float *means, const float *covs, const float *colors, const float *opac, int64_t n, const Cam &cam, float *rgb,
                   float *alpha, void *ws, cudaStream_t st) {
        const int64_t npad = pad_pow2(n);
        char         *w    = (char *) ws;
        auto         *keys = (unsigned long long *) w;
        w += npad * 8;
        auto *idx = (unsigned *) w;
        w += npad * 4;
        auto *nvalid = (int *) w;
        w += 256;
        auto *rec = (Rec<F> *) w;
        w += npad * sizeof(Rec<F>);
        auto *sorted = (Rec<F> *) w;
        w += npad * sizeof(Rec<F>);
        auto     *partial = (F *) w;
        const int segs    = raster_segments(cam.H, cam.W, ctx->sm_count);
        raster_preprocess_kernel<F><<<(unsigned) ((npad + 255) / 256), 256, 0, st>>>(means, covs, colors, opac, n, npad, cam, rec, keys, idx);
        if (int rc = vkc_post_launch(ctx, "raster_preprocess")) return rc;
        const unsigned blocks = (unsigned) (npad / kSortBlock);
        raster_sort_local_kernel<<<blocks, 1024, 0, st>>>(keys, idx, 2, kSortBlock);
        if (int rc = vkc_post_launch(ctx, "raster_sort_local")) return rc;
        for (int64_t k = 2 * kSortBlock; k <= npad; k <<= 1) {
            for (int64_t j = k >> 1; j >= kSortBlock; j >>= 1) {
                raster_sort_global_kernel<<<(unsigned) ((npad / 2 + 255) / 256), 256, 0, st>>>(keys, idx, npad, k, j);
                if (int rc = vkc_post_launch(ctx, "raster_sort_global")) return rc;
            }
            raster_sort_local_kernel<<<blocks, 1024, 0, st>>>(keys, idx, k, k);
            if (int rc = vkc_post_launch(ctx, "raster_sort_local")) return rc;
        }
        raster_gather_kernel<F><<<(unsigned) ((npad + 255) / 256), 256, 0, st>>>(rec, keys, idx, npad, sorted, nvalid);
        if (int rc = vkc_post_launch(ctx, "raster_gather")) return rc;
        dim3 grid((unsigned) ((cam.W + kTile - 1) / kTile), (unsigned) ((cam.H + kTile - 1) / kTile), (unsigned) segs);
        raster_composite_kernel<F><<<grid, dim3(kTile, kTile), 0, st>>>(sorted, nvalid, cam.H, cam.W, rgb, alpha, partial);
        if (int rc = vkc_post_launch(ctx, "raster_composite")) return rc;
        if (segs == 1) return VKC_OK;
        raster_combine_kernel<F><<<(unsigned) (((int64_t) cam.H * cam.W + 255) / 256), 256, 0, st>>>(partial, segs, cam.H, cam.W, rgb, alpha);
        return vkc_post_launch(ctx, "raster_combine");
    }

} // namespace

extern "C" size_t vkc_raster_workspace_bytes(int64_t n, int H, int W, int precise) {
    if (n < 0 || H < 1 || W < 1) return 0;
    const int64_t npad = pad_pow2(n);
    const size_t  rec  = precise ? sizeof(Rec<double>) : sizeof(Rec<float>);
    // keys, indices, counter, records, sorted records, and up to 32 depth segments of (C, T) per pixel
    return (size_t) npad * (8 + 4 + 2 * rec) + 256 + (size_t) 32 * H * W * 4 * (precise ? 8 : 4);
}

extern "C" int vkc_raster_gaussians(vkc_ctx *ctx, const float *means, const float *covs, const float *colors, const float *opacities, int64_t n,
                                    const double *w2c, const double *K, int H, int W, double znear, int precise, float *rgb, float *alpha,
                                    void *workspace, size_t workspace_bytes, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, n >= 0 && n <= (int64_t) 1 << 28, "raster: gaussian count out of range");
    VKC_REQUIRE(ctx, H >= 1 && W >= 1 && H <= 16384 && W <= 16384, "raster: bad image size %d x %d", H, W);
    VKC_REQUIRE(ctx, w2c && K && rgb, "raster: null camera or output");
    VKC_REQUIRE(ctx, n == 0 || (means && covs && colors && opacities), "raster: null gaussian attribute");
    VKC_REQUIRE(ctx, workspace && workspace_bytes >= vkc_raster_workspace_bytes(n, H, W, precise), "raster: workspace smaller than vkc_raster_workspace_bytes");
    VKC_REQUIRE(ctx, ((uintptr_t) workspace & 255) == 0, "raster: workspace must be 256-byte aligned");
    Cam cam;
    for (int a = 0; a < 3; ++a) {
        for (int b = 0; b < 3; ++b) cam.r[a * 3 + b] = w2c[a * 4 + b];
        cam.t[a] = w2c[a * 4 + 3];
    }
    cam.fx = K[0], cam.fy = K[4], cam.cx = K[2], cam.cy = K[5];
    cam.znear = znear, cam.H = H, cam.W = W;
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    return precise ? run_raster<double>(ctx, means, covs, colors, opacities, n, cam, rgb, alpha, workspace, st)
                   : run_raster<float>(ctx, means, covs, colors, opacities, n, cam, rgb, alpha, workspace, st);
}
