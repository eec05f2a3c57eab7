/* TEST INFRASTRUCTURE — CPU restatement of the reference's scalar CPU backend for the attention/encoder
 * path; see vknn_oracle.h for scope, the pinning status and the reference file:line each function follows.
 *
 * Bit-exactness notes. The reference accumulates MatMul in fp32 over k ascending, one multiply and one
 * add per step, separately rounded (its x86-64 build has no FMA contraction). The loops below reorder
 * m/n/k for speed and run rows on several threads, but every output element still sees exactly that
 * sequence of operations, so results are bit-identical. This file must be compiled with
 * -ffp-contract=off (the Makefile does).
 */
#include "vknn_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int64_t prod(const int64_t *s, int n) {
    int64_t p = 1;
    for (int i = 0; i < n; ++i) p *= s[i];
    return p;
}

static int resolve_threads(int threads) {
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_num_procs();
    return threads;
#else
    (void) threads;
    return 1;
#endif
}

/* y[M,N] = a[M,K] @ b[K,N] (+ bias[n]); per-element order: acc = 0; acc += a*b for k ascending; + bias. */
static void mm2d(const float *a, const float *b, const float *bias, float *y, int64_t M, int64_t N, int64_t K, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1 && M * N * K > 262144)
    for (int64_t m = 0; m < M; ++m) {
        float *yr = y + m * N;
        for (int64_t n = 0; n < N; ++n) yr[n] = 0.f;
        const float *ar = a + m * K;
        for (int64_t k = 0; k < K; ++k) {
            const float  av = ar[k];
            const float *br = b + k * N;
            for (int64_t n = 0; n < N; ++n) yr[n] = yr[n] + av * br[n];
        }
        if (bias) {
            for (int64_t n = 0; n < N; ++n) yr[n] = yr[n] + bias[n];
        }
    }
}

static int g_threads = 0; /* 0 = all cores */
void vko_set_threads(int t) { g_threads = t; }

int64_t vko_matmul(const float *a, const int64_t *ashape, int arank, const float *b, const int64_t *bshape, int brank,
                   const float *bias, float *y, int64_t *oshape, int *orank) {
    if (arank < 1 || brank < 1 || arank > VKO_MAX_RANK || brank > VKO_MAX_RANK) return -1;
    int64_t sa[VKO_MAX_RANK + 1], sb[VKO_MAX_RANK + 1];
    int     ra = arank, rb = brank;
    int     a1d = arank == 1, b1d = brank == 1;
    if (a1d) {
        sa[0] = 1;
        sa[1] = ashape[0];
        ra    = 2;
    } else {
        memcpy(sa, ashape, sizeof(int64_t) * (size_t) arank);
    }
    if (b1d) {
        sb[0] = bshape[0];
        sb[1] = 1;
        rb    = 2;
    } else {
        memcpy(sb, bshape, sizeof(int64_t) * (size_t) brank);
    }
    int64_t M = sa[ra - 2], K = sa[ra - 1], Kb = sb[rb - 2], N = sb[rb - 1];
    if (K != Kb) return -1;
    int     abr = ra - 2, bbr = rb - 2, br = abr > bbr ? abr : bbr;
    int64_t batch[VKO_MAX_RANK], ast[VKO_MAX_RANK], bst[VKO_MAX_RANK];
    int64_t batchElems = 1, sA = M * K, sB = K * N;
    for (int i = br - 1; i >= 0; --i) {
        int64_t ad = (i < br - abr) ? 1 : sa[i - (br - abr)];
        int64_t bd = (i < br - bbr) ? 1 : sb[i - (br - bbr)];
        if (ad != bd && ad != 1 && bd != 1) return -1;
        batch[i] = ad > bd ? ad : bd;
        ast[i]   = ad == 1 ? 0 : sA;
        bst[i]   = bd == 1 ? 0 : sB;
        sA *= ad;
        sB *= bd;
        batchElems *= batch[i];
    }
    int r = 0;
    for (int i = 0; i < br; ++i) oshape[r++] = batch[i];
    if (!a1d) oshape[r++] = M;
    oshape[r++] = N;
    if (b1d) r--;
    if (r == 0) oshape[r++] = 1;
    *orank = r;
    if (!y) return batchElems * M * N;
    int threads = resolve_threads(g_threads);
    for (int64_t bi = 0; bi < batchElems; ++bi) {
        int64_t ab = 0, bb = 0, rem = bi;
        for (int i = br - 1; i >= 0; --i) {
            int64_t c = rem % batch[i];
            rem /= batch[i];
            ab += c * ast[i];
            bb += c * bst[i];
        }
        mm2d(a + ab, b + bb, bias, y + bi * M * N, M, N, K, threads);
    }
    return batchElems * M * N;
}

void vko_softmax(const float *x, float *y, int64_t outer, int64_t inner) {
    for (int64_t o = 0; o < outer; ++o) {
        const float *xr = x + o * inner;
        float       *yr = y + o * inner;
        float        mx = xr[0];
        for (int64_t i = 1; i < inner; ++i) mx = xr[i] > mx ? xr[i] : mx; /* std::max(mx, xr[i]) */
        double sum = 0;
        for (int64_t i = 0; i < inner; ++i) {
            yr[i] = expf(xr[i] - mx);
            sum += yr[i];
        }
        for (int64_t i = 0; i < inner; ++i) yr[i] = (float) (yr[i] / sum);
    }
}

void vko_layernorm(const float *x, const float *gamma, const float *beta, float *y, int64_t outer, int64_t norm, float eps) {
    for (int64_t r = 0; r < outer; ++r) {
        const float *xr   = x + r * norm;
        float       *yr   = y + r * norm;
        double       mean = 0.0;
        for (int64_t j = 0; j < norm; ++j) mean += xr[j];
        mean /= (double) norm;
        double var = 0.0;
        for (int64_t j = 0; j < norm; ++j) {
            double c = xr[j] - mean;
            var += c * c;
        }
        var /= (double) norm;
        float inv = (float) (1.0 / sqrt(var + eps));
        for (int64_t j = 0; j < norm; ++j) {
            float v = ((float) (xr[j] - mean)) * inv * gamma[j];
            if (beta) v += beta[j];
            yr[j] = v;
        }
    }
}

static float bin_op(float a, float b, int op) {
    switch (op) {
        case VKO_BIN_MUL: return a * b;
        case VKO_BIN_SUB: return a - b;
        case VKO_BIN_DIV: return a / b;
        case VKO_BIN_MAX: return a < b ? b : a; /* std::max(a,b) */
        case VKO_BIN_MIN: return b < a ? b : a; /* std::min(a,b) */
        case VKO_BIN_POW: return powf(a, b);
        default: break;
    }
    return a + b;
}

/* NumPy-style broadcast strides of `s` against an output of rank `rank` (0 on broadcast dims). */
static void bcast_strides(const int64_t *s, int srank, int rank, int64_t *st) {
    int64_t stride = 1;
    int     off    = rank - srank;
    for (int i = rank - 1; i >= 0; --i) {
        int64_t d = i < off ? 1 : s[i - off];
        st[i]     = d == 1 ? 0 : stride;
        stride *= d;
    }
}

int64_t vko_binary(const float *a, const int64_t *ashape, int arank, const float *b, const int64_t *bshape, int brank, int op,
                   float *y, int64_t *oshape, int *orank) {
    int rank = arank > brank ? arank : brank;
    if (rank > VKO_MAX_RANK) return -1;
    for (int i = 0; i < rank; ++i) {
        int64_t ad = i < rank - arank ? 1 : ashape[i - (rank - arank)];
        int64_t bd = i < rank - brank ? 1 : bshape[i - (rank - brank)];
        oshape[i]  = ad > bd ? ad : bd;
    }
    *orank    = rank;
    int64_t n = prod(oshape, rank);
    if (!y) return n;
    int64_t oa[VKO_MAX_RANK], ob[VKO_MAX_RANK], idx[VKO_MAX_RANK];
    bcast_strides(ashape, arank, rank, oa);
    bcast_strides(bshape, brank, rank, ob);
    memset(idx, 0, sizeof idx);
    int64_t ia = 0, ib = 0;
    for (int64_t lin = 0; lin < n; ++lin) {
        y[lin] = bin_op(a[ia], b[ib], op);
        /* odometer increment: same element visit order and offsets as the reference's div/mod walk */
        for (int d = rank - 1; d >= 0; --d) {
            idx[d]++;
            ia += oa[d];
            ib += ob[d];
            if (idx[d] < oshape[d]) break;
            ia -= oa[d] * oshape[d];
            ib -= ob[d] * oshape[d];
            idx[d] = 0;
        }
    }
    return n;
}

static float un_op(float x, int op, float a, float b) {
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
        case 13: return x > 0 ? x : 0;
        case 14: return x / (1.f + expf(-x));
        case 15: return erff(x);
        case 16: return cosf(x);
        case 17: return sinf(x);
        case 18: return 1.f / x;
        case 19: return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x)));
        default: break;
    }
    return x;
}

void vko_unary(const float *x, float *y, int64_t n, int op, float p0, float p1) {
    for (int64_t i = 0; i < n; ++i) y[i] = un_op(x[i], op, p0, p1);
}

static float act_op(float x, int act, float lo, float hi) {
    switch (act) {
        case VKO_ACT_RELU: return x > 0 ? x : 0;
        case VKO_ACT_RELU6: return x < 0 ? 0 : (x > 6 ? 6 : x);
        case VKO_ACT_CLIP: return x < lo ? lo : (x > hi ? hi : x);
        case VKO_ACT_HSWISH: return x * fminf(fmaxf(x + 3.f, 0.f), 6.f) / 6.f;
        case VKO_ACT_SILU: return x / (1.f + expf(-x));
        default: break;
    }
    return x;
}

int vko_pw_epilogue(float *y, const int64_t *oshape, int orank, int nsteps, const int64_t *steps, const float *params,
                    const float *const *operands, const int64_t *const *opshapes, const int *opranks) {
    if (orank > VKO_MAX_RANK || nsteps > 64) return -1;
    int64_t n = prod(oshape, orank);
    int64_t ost[64][VKO_MAX_RANK];
    for (int s = 0; s < nsteps; ++s) {
        if (steps[s * 4] == 0) {
            int oi = (int) steps[s * 4 + 2];
            bcast_strides(opshapes[oi], opranks[oi], orank, ost[s]);
        }
    }
    int64_t ostride[VKO_MAX_RANK];
    int64_t st = 1;
    for (int d = orank - 1; d >= 0; --d) {
        ostride[d] = st;
        st *= oshape[d];
    }
    for (int64_t lin = 0; lin < n; ++lin) {
        float acc = y[lin];
        for (int s = 0; s < nsteps; ++s) {
            int   kind = (int) steps[s * 4], code = (int) steps[s * 4 + 1], oi = (int) steps[s * 4 + 2];
            float p0 = params[s * 2], p1 = params[s * 2 + 1];
            if (kind == 0) {
                int64_t io = 0;
                for (int d = 0; d < orank; ++d) io += ((lin / ostride[d]) % oshape[d]) * ost[s][d];
                acc = bin_op(acc, operands[oi][io], code);
            } else if (kind == 1) {
                acc = un_op(acc, code, p0, p1);
            } else if (kind == 2) {
                acc = act_op(acc, code, p0, p1);
            }
        }
        y[lin] = acc;
    }
    return 0;
}

void vko_transpose(const float *x, const int64_t *shape, int rank, const int64_t *perm, float *y) {
    int64_t p[VKO_MAX_RANK], oshape[VKO_MAX_RANK], ist[VKO_MAX_RANK], idx[VKO_MAX_RANK];
    for (int i = 0; i < rank; ++i) p[i] = perm ? perm[i] : rank - 1 - i;
    int64_t st = 1;
    for (int i = rank - 1; i >= 0; --i) {
        ist[i] = st;
        st *= shape[i];
    }
    for (int i = 0; i < rank; ++i) oshape[i] = shape[p[i]];
    int64_t n = prod(shape, rank);
    memset(idx, 0, sizeof idx);
    for (int64_t lin = 0; lin < n; ++lin) {
        int64_t src = 0;
        for (int d = 0; d < rank; ++d) src += idx[d] * ist[p[d]];
        y[lin] = x[src];
        for (int d = rank - 1; d >= 0; --d) {
            if (++idx[d] < oshape[d]) break;
            idx[d] = 0;
        }
    }
}

float vko_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t) (h & 0x8000) << 16, ex = (h >> 10) & 0x1F, mant = h & 0x3FF, f;
    if (ex == 0) {
        if (mant == 0) {
            f = sign;
        } else {
            ex = 127 - 15 + 1;
            while ((mant & 0x400) == 0) {
                mant <<= 1;
                --ex;
            }
            mant &= 0x3FF;
            f = sign | (ex << 23) | (mant << 13);
        }
    } else if (ex == 0x1F) {
        f = sign | 0x7F800000u | (mant << 13);
    } else {
        f = sign | ((ex - 15 + 127) << 23) | (mant << 13);
    }
    float out;
    memcpy(&out, &f, 4);
    return out;
}

uint16_t vko_float_to_half(float v) {
    uint32_t f;
    memcpy(&f, &v, 4);
    uint32_t sign = (f >> 16) & 0x8000;
    int32_t  ex   = (int32_t) ((f >> 23) & 0xFF) - 127 + 15;
    uint32_t mant = f & 0x7FFFFF;
    if (((f >> 23) & 0xFF) == 0xFF) return (uint16_t) (sign | 0x7C00 | (mant ? 0x200 : 0));
    if (ex >= 0x1F) return (uint16_t) (sign | 0x7C00);
    if (ex <= 0) {
        if (ex < -10) return (uint16_t) sign;
        mant |= 0x800000;
        uint32_t shift = (uint32_t) (14 - ex);
        uint32_t half  = mant >> shift;
        if ((mant >> (shift - 1)) & 1) half += 1;
        return (uint16_t) (sign | half);
    }
    uint16_t out = (uint16_t) (sign | ((uint32_t) ex << 10) | (mant >> 13));
    if (mant & 0x1000) out += 1;
    return out;
}

void vko_half_to_float_n(const uint16_t *src, float *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = vko_half_to_float(src[i]);
}
void vko_float_to_half_n(const float *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = vko_float_to_half(src[i]);
}

/* One (batch, head) unit of the attention pattern, with the reference's op sequence. */
static int attention_unit(const float *q, const float *k, const float *v, float *o, int64_t Sq, int64_t Skv, int64_t D,
                          float scale, const float *mask /* [Sq,Skv] additive or NULL */) {
    float *kt = (float *) malloc(sizeof(float) * (size_t) (D * Skv));
    float *s  = (float *) malloc(sizeof(float) * (size_t) (Sq * Skv));
    if (!kt || !s) {
        free(kt);
        free(s);
        return -1;
    }
    int64_t kshape[2] = {Skv, D}, perm[2] = {1, 0};
    vko_transpose(k, kshape, 2, perm, kt);    /* Transpose(K) */
    mm2d(q, kt, NULL, s, Sq, Skv, D, 1);      /* MatMul(Q, K^T) */
    int64_t n = Sq * Skv;
    if (mask) {
        /* FusedPointwise{Mul scale, Add mask}: acc = s*scale; acc = acc + mask */
        for (int64_t i = 0; i < n; ++i) {
            float acc = s[i] * scale;
            s[i]      = acc + mask[i];
        }
    } else {
        for (int64_t i = 0; i < n; ++i) s[i] = s[i] * scale; /* Binary Mul(scale) */
    }
    vko_softmax(s, s, Sq, Skv);          /* Softmax(axis=-1); in place is safe: row-local, read-before-write */
    mm2d(s, v, NULL, o, Sq, D, Skv, 1);  /* MatMul(P, V) */
    free(kt);
    free(s);
    return 0;
}

int vko_attention(const float *q, const float *k, const float *v, float *o, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                  int64_t Skv, int64_t D, float scale, int causal, const int32_t *kv_len, const float *mask,
                  int64_t first_unit, int64_t num_units, int threads) {
    if (Hkv <= 0 || Hq % Hkv) return -1;
    int64_t G = Hq / Hkv;
    if (num_units < 0) num_units = B * Hq - first_unit;
    threads = resolve_threads(threads);
    int err = 0;
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads) if (threads > 1 && num_units > 1)
    for (int64_t u = first_unit; u < first_unit + num_units; ++u) {
        int64_t      b = u / Hq, h = u % Hq, hk = h / G;
        const float *qu = q + (b * Hq + h) * Sq * D;
        const float *ku = k + (b * Hkv + hk) * Skv * D;
        const float *vu = v + (b * Hkv + hk) * Skv * D;
        float       *ou = o + (b * Hq + h) * Sq * D;
        float       *m  = NULL;
        if (causal || kv_len || mask) {
            m = (float *) malloc(sizeof(float) * (size_t) (Sq * Skv));
            if (!m) {
                err = -1;
                continue;
            }
            int64_t len = kv_len ? kv_len[b] : Skv;
            for (int64_t i = 0; i < Sq; ++i) {
                for (int64_t j = 0; j < Skv; ++j) {
                    float mv = mask ? mask[i * Skv + j] : 0.f;
                    if (j >= len) mv = -INFINITY;
                    if (causal && j > i + (Skv - Sq)) mv = -INFINITY;
                    m[i * Skv + j] = mv;
                }
            }
        }
        if (attention_unit(qu, ku, vu, ou, Sq, Skv, D, scale, m)) err = -1;
        free(m);
    }
    return err;
}

int vko_encoder_layer(const float *x, float *y, int64_t B, int64_t T, int64_t d, int64_t H, int64_t dmlp, const float *ln1_g,
                      const float *ln1_b, const float *wqkv, const float *bqkv, const float *wo, const float *bo,
                      const float *ln2_g, const float *ln2_b, const float *w1, const float *b1, const float *w2,
                      const float *b2, float eps, int threads) {
    int64_t M = B * T, D = d / H;
    threads   = resolve_threads(threads);
    float *h0  = (float *) malloc(sizeof(float) * (size_t) (M * d));
    float *qkv = (float *) malloc(sizeof(float) * (size_t) (M * 3 * d));
    float *qh  = (float *) malloc(sizeof(float) * (size_t) (3 * M * d));
    float *att = (float *) malloc(sizeof(float) * (size_t) (M * d));
    float *x1  = (float *) malloc(sizeof(float) * (size_t) (M * d));
    float *f1  = (float *) malloc(sizeof(float) * (size_t) (M * dmlp));
    float *f2  = (float *) malloc(sizeof(float) * (size_t) (M * dmlp));
    int    rc  = -1;
    if (!h0 || !qkv || !qh || !att || !x1 || !f1 || !f2) goto done;

    vko_layernorm(x, ln1_g, ln1_b, h0, M, d, eps);
    mm2d(h0, wqkv, bqkv, qkv, M, 3 * d, d, threads);
    /* head split: [B,T,3,H,D] -> [3,B,H,T,D] (Reshape + Transpose + Gather; pure data movement) */
    for (int64_t b = 0; b < B; ++b)
        for (int64_t t = 0; t < T; ++t)
            for (int64_t w = 0; w < 3; ++w)
                for (int64_t h = 0; h < H; ++h)
                    memcpy(qh + (((w * B + b) * H + h) * T + t) * D, qkv + ((b * T + t) * 3 + w) * d + h * D, sizeof(float) * (size_t) D);
    if (vko_attention(qh, qh + M * d, qh + 2 * M * d, att, B, H, H, T, T, D, 1.0f / sqrtf((float) D), 0, NULL, NULL, 0, -1, threads))
        goto done;
    /* head merge: [B,H,T,D] -> [B,T,H*D] */
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t t = 0; t < T; ++t)
                memcpy(h0 + (b * T + t) * d + h * D, att + ((b * H + h) * T + t) * D, sizeof(float) * (size_t) D);
    mm2d(h0, wo, bo, att, M, d, d, threads);
    for (int64_t i = 0; i < M * d; ++i) x1[i] = x[i] + att[i]; /* Add(residual) */
    vko_layernorm(x1, ln2_g, ln2_b, h0, M, d, eps);
    mm2d(h0, w1, b1, f1, M, dmlp, d, threads);
    {
        const float sqrt2 = 1.41421356237f; /* rounds to the fp32 constant the exported graph carries */
        for (int64_t i = 0; i < M * dmlp; ++i) {
            float t = f1[i] / sqrt2;   /* Binary Div */
            t       = erff(t);         /* Unary Erf */
            t       = t + 1.0f;        /* Add(1) */
            t       = t * f1[i];       /* FusedPointwise step 1: Mul h */
            f2[i]   = t * 0.5f;        /* FusedPointwise step 2: Mul 0.5 */
        }
    }
    mm2d(f2, w2, b2, att, M, d, dmlp, threads);
    for (int64_t i = 0; i < M * d; ++i) y[i] = x1[i] + att[i]; /* Add(residual) */
    rc = 0;
done:
    free(h0);
    free(qkv);
    free(qh);
    free(att);
    free(x1);
    free(f1);
    free(f2);
    return rc;
}
