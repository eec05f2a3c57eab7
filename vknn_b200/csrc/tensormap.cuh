// Host-side construction of TMA tensor maps (tiled mode, 128-byte swizzle) through the driver entry point
// resolved at context creation. Every map built here serves plain per-CTA loads or stores of this GPU's
// own memory.
#pragma once
#include "common.cuh"

typedef CUresult (*vkc_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                        const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// dims[0] is the contiguous dimension. strides_bytes[i] is the byte stride of dims[i+1] (rank-1 entries).
// box[0] * elem_size must be <= 128 bytes for the 128-byte swizzle. Out-of-range elements read as zero.
inline int vkc_make_tmap(vkc_ctx *ctx, CUtensorMap *map, int dtype, const void *base, int rank, const uint64_t *dims,
                         const uint64_t *strides_bytes, const uint32_t *box, bool swizzle128 = true) {
    if (!ctx->encode_tiled) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    if (((uintptr_t) base & 15) != 0) return vkc_fail(ctx, VKC_ERR_INVALID, "tensor base %p is not 16-byte aligned", base);
    CUtensorMapDataType dt;
    size_t              es;
    switch (dtype) {
        case VKC_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; es = 2; break;
        case VKC_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; es = 2; break;
        case VKC_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; es = 4; break;
        default: return vkc_fail(ctx, VKC_ERR_INVALID, "tensor map: bad dtype %d", dtype);
    }
    cuuint64_t gdims[5], gstr[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i]  = box[i];
        estr[i]  = 1;
        if (i > 0) {
            gstr[i - 1] = strides_bytes[i - 1];
            if (gstr[i - 1] % 16 != 0) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "tensor stride %llu bytes is not a multiple of 16", (unsigned long long) gstr[i - 1]);
        }
    }
    if (swizzle128 && gbox[0] * es > 128) return vkc_fail(ctx, VKC_ERR_INVALID, "tensor map inner box exceeds the 128-byte swizzle span");
    CUresult r = ((vkc_encode_tiled_fn) ctx->encode_tiled)(map, dt, (cuuint32_t) rank, const_cast<void *>(base), gdims, gstr, gbox, estr,
                                                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return vkc_fail(ctx, VKC_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int) r);
    return VKC_OK;
}
