// K5 — per-element step programs (the reference's FusedPointwise / Binary / Unary / Add family), standalone row
// Softmax and the strided gather copy used for Transpose/Gather/Slice nodes that cannot be absorbed as strides.
// All arithmetic is fp32, in the reference's step order; only loads and the final store touch the storage type.
#include "common.cuh"

namespace {

    constexpr int kMaxSteps = 8, kMaxOperands = 6, kMaxRank = 8;

    struct PwProgram {
        int         nsteps, rank, noperands;
        int         kind[kMaxSteps], code[kMaxSteps], opidx[kMaxSteps];
        float       p0[kMaxSteps], p1[kMaxSteps];
        int64_t     shape[kMaxRank];
        int64_t     ostride[kMaxOperands][kMaxRank];
        const void *operand[kMaxOperands];
        int         same_shape[kMaxOperands]; // operand is dense with the output's shape: index = linear index
    };

    __device__ __forceinline__ float pw_binary(float a, float b, int op) {
        switch (op) {
            case 0: return a * b;
            case 1: return a - b;
            case 2: return a / b;
            case 3: return fmaxf(a, b);
            case 4: return fminf(a, b);
            case 5: return powf(a, b);
            case 16: return a == b ? 1.f : 0.f; // Equal / Greater / GreaterEqual nodes: 1.0 / 0.0 like the reference
            case 17: return a > b ? 1.f : 0.f;
            case 18: return a >= b ? 1.f : 0.f;
            case 19: return a < b ? 1.f : 0.f; // the two above with the operands swapped
            case 20: return a <= b ? 1.f : 0.f;
            default: return a + b;
        }
    }
    __device__ __forceinline__ float pw_unary(float x, int op, float a, float b) {
        switch (op) {
            case 0: return 1.f / (1.f + expf(-x));
            case 1: return tanhf(x);
            case 2: return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) / 6.f;
            case 3: return fminf(fmaxf(a * x + b, 0.f), 1.f);
            case 4: return x > 0 ? x : a * x;
            case 5: return x > 0 ? x : a * (expf(x) - 1.f);
            case 6: return fabsf(x);
            case 7: return -x;
            case 8: return expf(x);
            case 9: return logf(x);
            case 10: return sqrtf(x);
            case 11: return floorf(x);
            case 12: return ceilf(x);
            case 13: return x > 0 ? x : 0.f;
            case 14: return x / (1.f + expf(-x));
            case 15: return erff(x);
            case 16: return cosf(x);
            case 17: return sinf(x);
            case 18: return 1.f / x;
            case 19: return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
            default: return x;
        }
    }
    __device__ __forceinline__ float pw_act(float x, int act, float lo, float hi) {
        switch (act) {
            case 1: return x > 0 ? x : 0.f;
            case 2: return x < 0 ? 0.f : (x > 6.f ? 6.f : x);
            case 3: return x < lo ? lo : (x > hi ? hi : x);
            case 4: return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) / 6.f;
            case 5: return x / (1.f + expf(-x));
            default: return x;
        }
    }

    template <typename T> __global__ void __launch_bounds__(256) pointwise_kernel(const T *__restrict__ X, T *__restrict__ Y, int64_t n, PwProgram pg) {
        int64_t       i      = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        const int64_t stride = (int64_t) gridDim.x * blockDim.x;
        for (; i < n; i += stride) {
            float acc = St<T>::ld(X + i);
            for (int s = 0; s < pg.nsteps; ++s) {
                if (pg.kind[s] == 0) {
                    const int oi = pg.opidx[s];
                    int64_t   io = 0;
                    if (pg.same_shape[oi]) {
                        io = i;
                    } else {
                        int64_t rem = i;
                        for (int d = pg.rank - 1; d >= 0; --d) {
                            const int64_t c = rem % pg.shape[d];
                            rem /= pg.shape[d];
                            io += c * pg.ostride[oi][d];
                        }
                    }
                    acc = pw_binary(acc, St<T>::ld((const T *) pg.operand[oi] + io), pg.code[s]);
                } else if (pg.kind[s] == 3) {
                    // select (Where): acc is the condition; operands opidx / code are the "true" / "false" values
                    const int oi = acc != 0.f ? pg.opidx[s] : pg.code[s];
                    int64_t   io = 0;
                    if (pg.same_shape[oi]) {
                        io = i;
                    } else {
                        int64_t rem = i;
                        for (int d = pg.rank - 1; d >= 0; --d) {
                            const int64_t c = rem % pg.shape[d];
                            rem /= pg.shape[d];
                            io += c * pg.ostride[oi][d];
                        }
                    }
                    acc = St<T>::ld((const T *) pg.operand[oi] + io);
                } else if (pg.kind[s] == 1) {
                    acc = pw_unary(acc, pg.code[s], pg.p0[s], pg.p1[s]);
                } else {
                    acc = pw_act(acc, pg.code[s], pg.p0[s], pg.p1[s]);
                }
            }
            St<T>::st(Y + i, acc);
        }
    }

    // One warp per row: max, sum of exp (fp32), normalise. Rows are re-read from L1/L2 between passes.
    template <typename T> __global__ void __launch_bounds__(256) softmax_kernel(const T *__restrict__ X, T *__restrict__ Y, int64_t outer, int64_t inner) {
        const int     lane = threadIdx.x & 31;
        const int64_t row  = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        if (row >= outer) return;
        const T *xr = X + row * inner;
        T       *yr = Y + row * inner;
        float    mx = -INFINITY;
        for (int64_t j = lane; j < inner; j += 32) mx = fmaxf(mx, St<T>::ld(xr + j));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float s = 0.f;
        for (int64_t j = lane; j < inner; j += 32) s += expf(St<T>::ld(xr + j) - mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        for (int64_t j = lane; j < inner; j += 32) St<T>::st(yr + j, expf(St<T>::ld(xr + j) - mx) / s);
    }

    // One warp per output element: `n` contiguous values reduced in fp32 (the caller has moved the reduced axes last).
    // op: 0 mean, 1 sum, 2 max, 3 min, 4 product, 5 L2 norm (the reference's ReduceType).
    template <typename T> __global__ void __launch_bounds__(256) reduce_rows_kernel(const T *__restrict__ X, T *__restrict__ Y, int64_t rows, int64_t n, int op) {
        const int     lane = threadIdx.x & 31;
        const int64_t row  = (int64_t) blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        if (row >= rows) return;
        const T *xr  = X + row * n;
        float    acc = op == 2 ? -INFINITY : (op == 3 ? INFINITY : (op == 4 ? 1.f : 0.f));
        for (int64_t j = lane; j < n; j += 32) {
            const float v = St<T>::ld(xr + j);
            acc           = op == 2 ? fmaxf(acc, v) : (op == 3 ? fminf(acc, v) : (op == 4 ? acc * v : (op == 5 ? acc + v * v : acc + v)));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float w = __shfl_xor_sync(0xffffffffu, acc, o);
            acc           = op == 2 ? fmaxf(acc, w) : (op == 3 ? fminf(acc, w) : (op == 4 ? acc * w : acc + w));
        }
        if (lane == 0) St<T>::st(Y + row, op == 0 ? acc / (float) n : (op == 5 ? sqrtf(acc) : acc));
    }

    struct CopyDesc {
        int     rank;
        int64_t shape[kMaxRank], istride[kMaxRank], ostride[kMaxRank], offset;
        int     dense_out; // output strides are the dense ones: Y[i]
    };

    template <typename T> __global__ void __launch_bounds__(256) strided_copy_kernel(const T *__restrict__ X, T *__restrict__ Y, int64_t n, CopyDesc cd) {
        int64_t       i      = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        const int64_t stride = (int64_t) gridDim.x * blockDim.x;
        for (; i < n; i += stride) {
            int64_t rem = i, src = cd.offset, dst = 0;
            for (int d = cd.rank - 1; d >= 0; --d) {
                const int64_t c = rem % cd.shape[d];
                rem /= cd.shape[d];
                src += c * cd.istride[d];
                dst += c * cd.ostride[d];
            }
            Y[cd.dense_out ? i : dst] = X[src];
        }
    }

    inline int grid_for(vkc_ctx *ctx, int64_t n) {
        int64_t blocks = (n + 255) / 256;
        int64_t cap    = (int64_t) ctx->sm_count * 16;
        return (int) (blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
    }

    // Row moves for Gather and ScatterND: row r of `rows` copies row_elems contiguous elements from src_off(r) to
    // dst_off(r). One warp walks a row in 16-byte pieces when both ends allow it, else element by element; rows are
    // spread over warps grid-stride. W is the storage word (2 or 4 bytes).
    template <typename W> __device__ __forceinline__ void move_row(const W *__restrict__ s, W *__restrict__ d, int64_t n, int lane) {
        constexpr int kPer = 16 / (int) sizeof(W);
        if ((((uintptr_t) s | (uintptr_t) d) & 15) == 0 && n % kPer == 0) {
            const uint4 *s4 = reinterpret_cast<const uint4 *>(s);
            uint4       *d4 = reinterpret_cast<uint4 *>(d);
            for (int64_t j = lane; j < n / kPer; j += 32) d4[j] = s4[j];
        } else {
            for (int64_t j = lane; j < n; j += 32) d[j] = s[j];
        }
    }

    template <typename W>
    __global__ void __launch_bounds__(256) copy_rows_kernel(const W *__restrict__ src, W *__restrict__ dst, const int64_t *__restrict__ src_off,
                                                            const int64_t *__restrict__ dst_off, int64_t nrows, int64_t row_elems) {
        const int     lane  = threadIdx.x & 31;
        const int64_t warp0 = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t) gridDim.x * 8;
        for (int64_t r = warp0; r < nrows; r += nwarps) {
            const int64_t so = src_off ? __ldg(src_off + r) : r * row_elems, dofs = dst_off ? __ldg(dst_off + r) : r * row_elems;
            move_row(src + so, dst + dofs, row_elems, lane);
        }
    }

    template <typename I> __device__ __forceinline__ int64_t index_value(const I *p, int64_t k);
    template <> __device__ __forceinline__ int64_t index_value<float>(const float *p, int64_t k) { return (int64_t) p[k]; }
    template <> __device__ __forceinline__ int64_t index_value<__half>(const __half *p, int64_t k) { return (int64_t) __half2float(p[k]); }
    template <> __device__ __forceinline__ int64_t index_value<__nv_bfloat16>(const __nv_bfloat16 *p, int64_t k) { return (int64_t) __bfloat162float(p[k]); }
    template <> __device__ __forceinline__ int64_t index_value<int32_t>(const int32_t *p, int64_t k) { return p[k]; }

    // Gather along an axis with indices that are themselves device data: out[o, k, :] = data[o, idx[k], :].
    template <typename W, typename I>
    __global__ void __launch_bounds__(256) gather_rows_kernel(const W *__restrict__ data, const I *__restrict__ idx, W *__restrict__ out, int64_t outer,
                                                              int64_t axis_size, int64_t nidx, int64_t inner) {
        const int     lane  = threadIdx.x & 31;
        const int64_t warp0 = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5), nwarps = (int64_t) gridDim.x * 8;
        for (int64_t r = warp0; r < outer * nidx; r += nwarps) {
            const int64_t o = r / nidx, k = r - o * nidx;
            int64_t       i = index_value<I>(idx, k);
            if (i < 0) i += axis_size;
            i = i < 0 ? 0 : (i >= axis_size ? axis_size - 1 : i); // an index outside the axis reads the nearest row instead of stray memory
            move_row(data + (o * axis_size + i) * inner, out + r * inner, inner, lane);
        }
    }

} // namespace

extern "C" {

int vkc_pointwise(vkc_ctx *ctx, const void *X, void *Y, const int64_t *shape, int rank, int nsteps, const int32_t *steps, const float *params,
                  int noperands, const void *const *operands, const int64_t *op_strides, int dtype, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, rank >= 1 && rank <= kMaxRank && shape, "pointwise: rank %d out of range", rank);
    VKC_REQUIRE(ctx, nsteps >= 0 && nsteps <= kMaxSteps, "pointwise: %d steps exceed the limit of %d", nsteps, kMaxSteps);
    VKC_REQUIRE(ctx, noperands >= 0 && noperands <= kMaxOperands, "pointwise: %d operands exceed the limit of %d", noperands, kMaxOperands);
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "pointwise: bad dtype %d", dtype);
    PwProgram pg;
    memset(&pg, 0, sizeof pg);
    pg.nsteps    = nsteps;
    pg.rank      = rank;
    pg.noperands = noperands;
    int64_t n    = 1;
    for (int d = 0; d < rank; ++d) {
        VKC_REQUIRE(ctx, shape[d] >= 0, "pointwise: negative dim");
        pg.shape[d] = shape[d];
        n *= shape[d];
    }
    for (int o = 0; o < noperands; ++o) {
        VKC_REQUIRE(ctx, operands && operands[o] && op_strides, "pointwise: null operand %d", o);
        pg.operand[o] = operands[o];
        int64_t dense = 1;
        bool    same  = true;
        for (int d = rank - 1; d >= 0; --d) {
            pg.ostride[o][d] = op_strides[o * rank + d];
            if (shape[d] != 1 && pg.ostride[o][d] != dense) same = false;
            dense *= shape[d];
        }
        pg.same_shape[o] = same;
    }
    for (int s = 0; s < nsteps; ++s) {
        pg.kind[s]  = steps[s * 4 + 0];
        pg.code[s]  = steps[s * 4 + 1];
        pg.opidx[s] = steps[s * 4 + 2] - 1; // the reference numbers operands from 1 (0 is the primary)
        if (pg.kind[s] == 3) pg.code[s] -= 1; // select: the "false" operand, numbered the same way
        pg.p0[s]    = params ? params[s * 2 + 0] : 0.f;
        pg.p1[s]    = params ? params[s * 2 + 1] : 0.f;
        VKC_REQUIRE(ctx, pg.kind[s] >= 0 && pg.kind[s] <= 3, "pointwise: bad step kind %d", pg.kind[s]);
        if (pg.kind[s] == 3) VKC_REQUIRE(ctx, pg.code[s] >= 0 && pg.code[s] < noperands, "pointwise: select step %d names operand %d of %d", s, pg.code[s] + 1, noperands);
        if (pg.kind[s] == 0 || pg.kind[s] == 3) VKC_REQUIRE(ctx, pg.opidx[s] >= 0 && pg.opidx[s] < noperands, "pointwise: step %d names operand %d of %d", s, pg.opidx[s] + 1, noperands);
    }
    if (n == 0) return VKC_OK;
    VKC_REQUIRE(ctx, X && Y, "pointwise: null tensor");
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    const int    g  = grid_for(ctx, n);
    switch (dtype) {
        case VKC_F32: pointwise_kernel<float><<<g, 256, 0, st>>>((const float *) X, (float *) Y, n, pg); break;
        case VKC_F16: pointwise_kernel<__half><<<g, 256, 0, st>>>((const __half *) X, (__half *) Y, n, pg); break;
        default: pointwise_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16 *) X, (__nv_bfloat16 *) Y, n, pg); break;
    }
    return vkc_post_launch(ctx, "pointwise");
}

int vkc_softmax(vkc_ctx *ctx, const void *X, void *Y, int64_t outer, int64_t inner, int dtype, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, outer >= 0 && inner >= 1, "softmax: bad extents");
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "softmax: bad dtype %d", dtype);
    if (outer == 0) return VKC_OK;
    VKC_REQUIRE(ctx, X && Y, "softmax: null tensor");
    cudaStream_t  st     = vkc_pick_stream(ctx, stream);
    const int64_t blocks = (outer + 7) / 8;
    VKC_REQUIRE(ctx, blocks <= INT32_MAX, "softmax: too many rows");
    switch (dtype) {
        case VKC_F32: softmax_kernel<float><<<(unsigned) blocks, 256, 0, st>>>((const float *) X, (float *) Y, outer, inner); break;
        case VKC_F16: softmax_kernel<__half><<<(unsigned) blocks, 256, 0, st>>>((const __half *) X, (__half *) Y, outer, inner); break;
        default: softmax_kernel<__nv_bfloat16><<<(unsigned) blocks, 256, 0, st>>>((const __nv_bfloat16 *) X, (__nv_bfloat16 *) Y, outer, inner); break;
    }
    return vkc_post_launch(ctx, "softmax");
}

int vkc_reduce_rows(vkc_ctx *ctx, const void *X, void *Y, int64_t rows, int64_t n, int op, int dtype, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, rows >= 0 && n >= 1, "reduce: bad extents");
    VKC_REQUIRE(ctx, op >= 0 && op <= 5, "reduce: bad op %d", op);
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "reduce: bad dtype %d", dtype);
    if (rows == 0) return VKC_OK;
    VKC_REQUIRE(ctx, X && Y, "reduce: null tensor");
    cudaStream_t  st     = vkc_pick_stream(ctx, stream);
    const int64_t blocks = (rows + 7) / 8;
    VKC_REQUIRE(ctx, blocks <= INT32_MAX, "reduce: too many rows");
    switch (dtype) {
        case VKC_F32: reduce_rows_kernel<float><<<(unsigned) blocks, 256, 0, st>>>((const float *) X, (float *) Y, rows, n, op); break;
        case VKC_F16: reduce_rows_kernel<__half><<<(unsigned) blocks, 256, 0, st>>>((const __half *) X, (__half *) Y, rows, n, op); break;
        default: reduce_rows_kernel<__nv_bfloat16><<<(unsigned) blocks, 256, 0, st>>>((const __nv_bfloat16 *) X, (__nv_bfloat16 *) Y, rows, n, op); break;
    }
    return vkc_post_launch(ctx, "reduce_rows");
}

int vkc_strided_copy2(vkc_ctx *ctx, const void *X, void *Y, const int64_t *shape, const int64_t *in_strides, const int64_t *out_strides, int rank,
                      int64_t in_offset, int dtype, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, rank >= 1 && rank <= kMaxRank && shape && in_strides, "strided_copy: rank %d out of range", rank);
    CopyDesc cd;
    cd.rank      = rank;
    cd.offset    = in_offset;
    cd.dense_out = out_strides ? 0 : 1;
    int64_t n    = 1;
    for (int d = 0; d < rank; ++d) {
        cd.shape[d]   = shape[d];
        cd.istride[d] = in_strides[d];
        cd.ostride[d] = out_strides ? out_strides[d] : 0;
        n *= shape[d];
    }
    if (n == 0) return VKC_OK;
    VKC_REQUIRE(ctx, X && Y, "strided_copy: null tensor");
    cudaStream_t st = vkc_pick_stream(ctx, stream);
    const int    g  = grid_for(ctx, n);
    if (vkc_dtype_size(dtype) == 4)
        strided_copy_kernel<uint32_t><<<g, 256, 0, st>>>((const uint32_t *) X, (uint32_t *) Y, n, cd);
    else
        strided_copy_kernel<uint16_t><<<g, 256, 0, st>>>((const uint16_t *) X, (uint16_t *) Y, n, cd);
    return vkc_post_launch(ctx, "strided_copy");
}

int vkc_strided_copy(vkc_ctx *ctx, const void *X, void *Y, const int64_t *shape, const int64_t *in_strides, int rank, int64_t in_offset, int dtype,
                     vkc_stream stream) {
    return vkc_strided_copy2(ctx, X, Y, shape, in_strides, nullptr, rank, in_offset, dtype, stream);
}

int vkc_copy_rows(vkc_ctx *ctx, const void *src, void *dst, const int64_t *src_off, const int64_t *dst_off, int64_t nrows, int64_t row_elems, int dtype,
                  vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, nrows >= 0 && row_elems >= 0, "copy_rows: bad extents");
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "copy_rows: bad dtype %d", dtype);
    if (nrows == 0 || row_elems == 0) return VKC_OK;
    VKC_REQUIRE(ctx, src && dst, "copy_rows: null tensor");
    cudaStream_t  st     = vkc_pick_stream(ctx, stream);
    const int64_t want   = (nrows + 7) / 8, cap = (int64_t) ctx->sm_count * 16;
    const unsigned blocks = (unsigned) (want < cap ? want : cap);
    if (vkc_dtype_size(dtype) == 4)
        copy_rows_kernel<uint32_t><<<blocks, 256, 0, st>>>((const uint32_t *) src, (uint32_t *) dst, src_off, dst_off, nrows, row_elems);
    else
        copy_rows_kernel<uint16_t><<<blocks, 256, 0, st>>>((const uint16_t *) src, (uint16_t *) dst, src_off, dst_off, nrows, row_elems);
    return vkc_post_launch(ctx, "copy_rows");
}

int vkc_gather_rows(vkc_ctx *ctx, const void *data, const void *index, void *out, int64_t outer, int64_t axis_size, int64_t nidx, int64_t inner,
                    int dtype, int index_dtype, vkc_stream stream) {
    if (!ctx) return VKC_ERR_INVALID;
    VKC_REQUIRE(ctx, outer >= 0 && axis_size >= 1 && nidx >= 0 && inner >= 0, "gather_rows: bad extents");
    VKC_REQUIRE(ctx, dtype == VKC_F32 || dtype == VKC_F16 || dtype == VKC_BF16, "gather_rows: bad dtype %d", dtype);
    VKC_REQUIRE(ctx, index_dtype == VKC_F32 || index_dtype == VKC_F16 || index_dtype == VKC_BF16 || index_dtype == VKC_I32,
                "gather_rows: bad index dtype %d", index_dtype);
    if (outer * nidx == 0 || inner == 0) return VKC_OK;
    VKC_REQUIRE(ctx, data && index && out, "gather_rows: null tensor");
    cudaStream_t  st     = vkc_pick_stream(ctx, stream);
    const int64_t want   = (outer * nidx + 7) / 8, cap = (int64_t) ctx->sm_count * 16;
    const unsigned blocks = (unsigned) (want < cap ? want : cap);
#define VKC_GATHER(W_)                                                                                                                            \
    switch (index_dtype) {                                                                                                                        \
        case VKC_F32: gather_rows_kernel<W_, float><<<blocks, 256, 0, st>>>((const W_ *) data, (const float *) index, (W_ *) out, outer, axis_size, nidx, inner); break; \
        case VKC_F16: gather_rows_kernel<W_, __half><<<blocks, 256, 0, st>>>((const W_ *) data, (const __half *) index, (W_ *) out, outer, axis_size, nidx, inner); break; \
        case VKC_BF16: gather_rows_kernel<W_, __nv_bfloat16><<<blocks, 256, 0, st>>>((const W_ *) data, (const __nv_bfloat16 *) index, (W_ *) out, outer, axis_size, nidx, inner); break; \
        default: gather_rows_kernel<W_, int32_t><<<blocks, 256, 0, st>>>((const W_ *) data, (const int32_t *) index, (W_ *) out, outer, axis_size, nidx, inner); break; \
    }
    if (vkc_dtype_size(dtype) == 4) {
        VKC_GATHER(uint32_t)
    } else {
        VKC_GATHER(uint16_t)
    }
#undef VKC_GATHER
    return vkc_post_launch(ctx, "gather_rows");
}

} // extern "C"
