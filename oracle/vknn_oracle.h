/* TEST INFRASTRUCTURE — a CPU restatement of the reference's scalar CPU backend for the attention /
 * encoder path. It exists only to CHECK the CUDA kernels (tests/, the smoke check and the bench's
 * cpu_baseline leg). Nothing in the shipped library calls it, links it or falls back to it.
 *
 * Parity status: PINNED. Every function below is compared bit for bit against the reference's own CPU
 * backend executed in this build environment (oracle/_ref/vknn_ref_driver, see tests/golden/make_golden.py),
 * and against the known-answer vectors of the reference's unit tests (tests/test_ops.cpp:290-313,502-608).
 *
 * All tensors are row-major fp32 on the host, exactly like the reference's RtTensor::host buffers.
 * Shapes are passed as int64 arrays with rank <= VKO_MAX_RANK.
 */
#ifndef VKNN_ORACLE_H
#define VKNN_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define VKO_MAX_RANK 8

/* BinaryType / UnaryType / ActType codes, numerically identical to the reference enums
 * (include/vknn/binary_type.h:8, include/vknn/unary_type.h:11-33, include/vknn/act_type.h:7). */
enum { VKO_BIN_MUL = 0, VKO_BIN_SUB = 1, VKO_BIN_DIV = 2, VKO_BIN_MAX = 3, VKO_BIN_MIN = 4, VKO_BIN_POW = 5, VKO_BIN_ADD = 6 };
enum { VKO_UN_SIGMOID = 0, VKO_UN_TANH = 1, VKO_UN_EXP = 8, VKO_UN_SQRT = 10, VKO_UN_RELU = 13, VKO_UN_SILU = 14, VKO_UN_ERF = 15, VKO_UN_RECIP = 18 };
enum { VKO_ACT_NONE = 0, VKO_ACT_RELU = 1, VKO_ACT_RELU6 = 2, VKO_ACT_CLIP = 3, VKO_ACT_HSWISH = 4, VKO_ACT_SILU = 5 };

/* Threads used by vko_matmul's row loop (0 = all cores; the reference itself is single-threaded, and the
 * result does not depend on this). */
void vko_set_threads(int threads);

/* MatMulCpu::run, src/backend/cpu/ops/matmul.cpp:14-116. N-D batched matmul with NumPy broadcast on the
 * batch dims and 1-D promotion; bias (may be NULL) is the rank-1 [N] fusedBias added after the k-sum.
 * Writes the output shape to oshape/orank; returns the number of output elements, or -1 on a bad shape.
 * y == NULL only computes the shape. */
int64_t vko_matmul(const float *a, const int64_t *ashape, int arank, const float *b, const int64_t *bshape, int brank,
                   const float *bias, float *y, int64_t *oshape, int *orank);

/* SoftmaxCpu::run, src/backend/cpu/ops/softmax.cpp:9-47: rows of `inner` contiguous elements;
 * max-subtract, expf in float, sum in double, divide in double then round to float. */
void vko_softmax(const float *x, float *y, int64_t outer, int64_t inner);

/* LayerNormCpu::run, src/backend/cpu/ops/layernorm.cpp:12-75: mean and variance in double (two passes),
 * inv = (float)(1/sqrt(var + eps)); beta may be NULL. */
void vko_layernorm(const float *x, const float *gamma, const float *beta, float *y, int64_t outer, int64_t norm, float eps);

/* BinaryCpu::run (float path), src/backend/cpu/ops/binary.cpp:112-139, and AddCpu::run general path,
 * src/backend/cpu/ops/add.cpp:88-125 (op = VKO_BIN_ADD). Returns output element count; writes shape. */
int64_t vko_binary(const float *a, const int64_t *ashape, int arank, const float *b, const int64_t *bshape, int brank, int op,
                   float *y, int64_t *oshape, int *orank);

/* UnaryCpu::run, src/backend/cpu/ops/unary.cpp:10-69. */
void vko_unary(const float *x, float *y, int64_t n, int op, float p0, float p1);

/* applyPwEpilogue, src/backend/cpu/ops/fused_pointwise.cpp:107-167: runs the step program in place on y
 * (which already holds the primary). steps = 4 ints per step {kind, code, operandIdx, bcast}; params = 2
 * floats per step. operandIdx indexes operands[] with the reference's numbering: 1 is the first extra
 * operand (index 0 is the primary), so operands[0] is unused and may be NULL. */
int vko_pw_epilogue(float *y, const int64_t *oshape, int orank, int nsteps, const int64_t *steps, const float *params,
                    const float *const *operands, const int64_t *const *opshapes, const int *opranks);

/* TransposeCpu::run, src/backend/cpu/ops/transpose.cpp:8-63 (perm NULL => reverse). */
void vko_transpose(const float *x, const int64_t *shape, int rank, const int64_t *perm, float *y);

/* halfToFloat / floatToHalf, include/vknn/dtype.h:60-157 (the reference's own host conversion; note that
 * floatToHalf rounds a tie upward, not to even). */
float    vko_half_to_float(uint16_t h);
uint16_t vko_float_to_half(float v);
void     vko_half_to_float_n(const uint16_t *src, float *dst, int64_t n);
void     vko_float_to_half_n(const float *src, uint16_t *dst, int64_t n);

/* The attention pattern exactly as the reference's passes leave it (probe of the C1 / GQA graphs):
 *   Transpose(K) -> MatMul(Q,K^T) -> Binary Mul(scale)            [no mask]
 *   Transpose(K) -> MatMul(Q,K^T) -> FusedPointwise{Mul scale, Add mask} [additive mask]
 *   -> Softmax(axis=-1) -> MatMul(P,V)
 * composed from the functions above, one (batch, head) unit at a time (units are independent, so the
 * result equals the whole-graph run bit for bit; peak memory is one [Sq,Skv] score tile per thread).
 * q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D], o [B,Hq,Sq,D]; Hq % Hkv == 0, query head h reads kv head h/(Hq/Hkv)
 * (the MatMul batch-broadcast form [B,Hkv,G,..]). Masking, all expressed as the additive -inf tensor
 * the reference graph would carry: causal (key j > query i + (Skv - Sq) masked), kv_len[b] (keys >=
 * kv_len[b] masked; NULL = none), mask (additive fp32 [Sq,Skv] shared by all units; NULL = none).
 * first_unit/num_units select a contiguous range of the B*Hq units (for slices of a large config).
 * threads <= 0 uses all cores. */
int vko_attention(const float *q, const float *k, const float *v, float *o, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                  int64_t Skv, int64_t D, float scale, int causal, const int32_t *kv_len, const float *mask,
                  int64_t first_unit, int64_t num_units, int threads);

/* One pre-LayerNorm encoder block as the reference's passes leave it:
 *   LayerNorm -> MatMul(Wqkv)+fusedBias -> head split -> attention -> head merge -> MatMul(Wo)+fusedBias
 *   -> Add(residual) -> LayerNorm -> MatMul(W1)+fusedBias -> Binary Div(sqrt2) -> Unary Erf -> Add(1)
 *   -> FusedPointwise{Mul h, Mul 0.5} -> MatMul(W2)+fusedBias -> Add(residual)
 * x [B,T,d]; wqkv [d,3d] with columns ordered (q|k|v) x head x head_dim; weights row-major [K,N] fp32. */
int vko_encoder_layer(const float *x, float *y, int64_t B, int64_t T, int64_t d, int64_t H, int64_t dmlp, const float *ln1_g,
                      const float *ln1_b, const float *wqkv, const float *bqkv, const float *wo, const float *bo,
                      const float *ln2_g, const float *ln2_b, const float *w1, const float *b1, const float *w2,
                      const float *b2, float eps, int threads);

#ifdef __cplusplus
}
#endif
#endif
