// K3 (tensor-core form) — single-query (decode) attention over a KV cache, head_dim 128, f16 / bf16, HBM-bound.
//
// The K and V rows are the only large operands, so the kernel is built around streaming them exactly once
// from HBM into shared memory with TMA and feeding them to the tensor cores WITHOUT passing through registers:
//
//   S^T [128 keys x 16]   = K_tile [128 keys x 128] . Q_g^T [128 x 16]     (tcgen05.mma, M = keys, N = query heads of
//                                                                           the kv group padded to 16)
//   O^T [128 dims x 16]  += V_tile^T [128 dims x 128 keys] . P^T [128 keys x 16]   (A = V tile read MN-major)
//
// so one 128-key tile costs 16 small MMAs and the per-key work left for the CUDA cores is one exp2 per (key,
// head). Persistent CTAs (one per SM) each take an equal share of the key tiles of all (sequence, kv head) units,
// cut into work items at the unit boundaries (sequence, stretch of the
// cache, kv head); the TMA producer runs ahead across item boundaries through a 3-stage ring (192 KB in flight
// per SM).
//
//   warp 0    producer: Q_g tile per item (double buffered), K and V tiles of 128 keys per ring stage.
//   warp 1    MMA issuer + TMEM owner (S^T x4, O^T x4: 128 columns in all); Q.K^T runs two tiles ahead of P.V.
//   warps 2-5 softmax group 0 (even tiles of an item), warps 6-9 softmax group 1 (odd tiles). Each group keeps its
//             own running maximum, row sums and O^T accumulator and emits its own partial, so the two groups never
//             exchange data and their latency chains overlap. Thread r of a group owns key r of its current tile (a
//             TMEM lane of S^T) and, in the item epilogue, output dimension r (a TMEM lane of O^T). Per tile: read 16 columns of S^T, per-head maximum over the
//             tile (warp shuffles + one shared-memory exchange), lazily raised running maximum, p = exp2(s*scale*log2e - m),
//             written as P^T into shared memory in the K-major swizzled layout the MMA expects. Row sums are kept
//             per thread and reduced once per item. Per item: O^T -> per-chunk partial (max, sum, o) in scratch;
//             the merge kernel of the SIMT form combines the chunks.
// Keys past kv_len[b] inside the last tile get p = 0 and their V rows are zeroed in shared memory before the
// P.V MMA, so whatever the cache holds there (even NaN bit patterns) cannot reach the output.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"

namespace {

    constexpr int TK       = 128; // keys per tile
    constexpr int DH       = 128; // head dim
    constexpr int NPAD     = 16;  // query heads per kv head, padded (MMA N)
    constexpr int kStages  = 3;
    constexpr int kThreads = 64 + 2 * 128;
    constexpr int kTmemCols = 128; // S^T[g & 3] at 16 * (g & 3); O^T[group][item & 1] at 64 + 16 * (2 * group + (item & 1))
    constexpr int kMaxPrefix = 1024; // sequences whose item prefix table fits the shared-memory scratch
    constexpr float kRescaleThreshold = 8.0f;

    constexpr uint32_t KV_BYTES = TK * DH * 2;   // 32 KB
    constexpr uint32_t Q_BYTES  = NPAD * DH * 2; // 4 KB
    constexpr uint32_t P_BYTES  = NPAD * TK * 2; // 4 KB
    constexpr uint32_t oK   = 0;
    constexpr uint32_t oV   = oK + kStages * KV_BYTES;
    constexpr uint32_t oQ   = oV + kStages * KV_BYTES;
    constexpr uint32_t oP   = oQ + 2 * Q_BYTES;
    constexpr uint32_t oBar = oP + 4 * P_BYTES;
    // barriers: k_full[ST] k_empty[ST] v_full[ST] v_empty[ST] q_full[2] q_empty[2] s_full[4] s_empty[4] p_full[4]
    //           o_full[2 groups][2] o_empty[2][2] pv_done[2 groups] red_max[2 groups][2] red_sum[2 groups]
    constexpr int bKF = 0, bKE = kStages, bVF = 2 * kStages, bVE = 3 * kStages, bQF = 4 * kStages, bQE = bQF + 2, bSF = bQE + 2, bSE = bSF + 4,
                  bPF = bSE + 4, bOF = bPF + 4, bOE = bOF + 4, bPV = bOE + 4, bRX = bPV + 2, bLS = bRX + 4, nBar = bLS + 2;
    constexpr uint32_t oRed  = oBar + 8 * nBar;             // float red[2 groups][2][4][NPAD] (tile max), float lsum[2 groups][2][4][NPAD]
    constexpr uint32_t oPre  = oRed + 4 * (2 * 2 * 4 * NPAD + 2 * 2 * 4 * NPAD); // int prefix[kMaxPrefix + 1]
    constexpr uint32_t oCtl  = oPre + 4 * (kMaxPrefix + 1);
    constexpr uint32_t kSmemTotal = oCtl + 16 + 1024;

    struct DecParams {
        float         *part_ml, *part_o;
        const int32_t *kv_len;
        int            B, Hkv, G, min_quota, parts_stride; // parts_stride = partial slots per (sequence, query head)
        int           *nslots;                             // [B][Hkv]: partial slots the (sequence, kv head) filled
        int64_t        Lmax;
        float          scale_log2;
        int           *dev_err;
    };

    // Work distribution. The 128-key tiles of all (sequence, kv head) units are numbered in one line, sequence-major
    // (prefix[b] = tiles before sequence b; within a sequence kv head after kv head). CTA c takes the `quota` tiles
    // [c * quota, (c + 1) * quota) of that line, so every CTA streams the same number of bytes whatever the sequence
    // lengths are, and meets at most a handful of unit boundaries. An item is the stretch of a CTA's range that lies
    // in one unit; its partials go to the unit's slot pair number (c - CTA of the unit's first tile).
    struct Item {
        int     b, hk, split, ntiles;
        int64_t start, end;
        bool    valid, last; // last: the item holds the unit's final tile
    };
    // (find_item and its helpers are host/device: the kernel and vkc_attn_decode_tc_items, which walks a host copy of the
    // lengths, run the same arithmetic)
    __host__ __device__ __forceinline__ int64_t seq_len(const DecParams &p, int b) {
        int64_t len = p.kv_len ? (int64_t) p.kv_len[b] : p.Lmax;
        if (len > p.Lmax) len = p.Lmax;
        return len < 0 ? 0 : len;
    }
    __host__ __device__ __forceinline__ int tile_quota(const DecParams &p, const int *prefix, int grid) {
        const int q = (prefix[p.B] + grid - 1) / grid;
        return q > p.min_quota ? q : p.min_quota;
    }
    // The item that starts at tile `pos` of the line; the CTA's range ends at `pos1`.
    __host__ __device__ __forceinline__ Item find_item(const DecParams &p, const int *prefix, int pos, int pos1, int quota) {
        Item it;
        it.valid = false;
        if (pos >= pos1) return it;
        int lo = 0, hi = p.B - 1; // last b with prefix[b] <= pos
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= pos) lo = mid;
            else hi = mid - 1;
        }
        const int64_t len   = seq_len(p, lo);
        const int     tiles = (int) ((len + TK - 1) / TK);
        const int     r     = pos - prefix[lo];
        it.b                = lo;
        it.hk               = r / tiles;
        const int tile      = r - it.hk * tiles;
        const int left      = tiles - tile, room = pos1 - pos;
        it.ntiles           = left < room ? left : room;
        it.last             = left <= room;
        it.split            = pos / quota - (prefix[lo] + it.hk * tiles) / quota;
        it.start            = (int64_t) tile * TK;
        it.end              = it.start + (int64_t) it.ntiles * TK < len ? it.start + (int64_t) it.ntiles * TK : len;
        it.valid            = true;
        return it;
    }

    __device__ __forceinline__ float fast_exp2(float x) {
        float y;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
        return y;
    }

    template <typename T>
    __global__ void __launch_bounds__(kThreads, 1)
        attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                              DecParams p) {
        constexpr bool     kBf16    = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdescQK = ptx::idesc_f16(TK, NPAD, kBf16, false, false); // A = K tile (K-major), B = Q (K-major)
        constexpr uint32_t kIdescPV = ptx::idesc_f16(DH, NPAD, kBf16, true, false);  // A = V tile (MN-major), B = P^T (K-major)

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw    = ptx::smem_u32(smem_raw);
        const uint32_t base   = (raw + 1023u) & ~1023u;
        uint8_t       *gbase  = smem_raw + (base - raw);
        auto           bar    = [&](int i) { return base + oBar + 8u * (uint32_t) i; };
        volatile int  *ctl    = (volatile int *) (gbase + oCtl); // ctl[0] = tmem base, ctl[1] = abort flag
        float         *red    = (float *) (gbase + oRed);        // [2 groups][2][4][NPAD]
        float         *lsum   = red + 2 * 2 * 4 * NPAD;          // [2 groups][2][4][NPAD]
        int           *prefix = (int *) (gbase + oPre);          // [B + 1]

        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int G = p.G;

        if (threadIdx.x == 0) {
            for (int i = 0; i < nBar; ++i) {
                const bool many   = (i >= bSE && i < bSE + 4) || (i >= bPF && i < bPF + 4) || (i >= bOE && i < bOE + 4);
                const bool warps4 = i >= bRX; // one arrival per warp of a softmax group
                ptx::mbar_init(bar(i), many ? 128 : (warps4 ? 4 : 1));
            }
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmQ);
            ptx::prefetch_tmap(&tmK);
            ptx::prefetch_tmap(&tmV);
        }
        for (int b = threadIdx.x; b < p.B; b += kThreads) prefix[b + 1] = (int) (((seq_len(p, b) + TK - 1) / TK) * p.Hkv);
        if (warp == 1) {
            ptx::tmem_alloc(base + oCtl, kTmemCols);
            ptx::tmem_relinquish();
        }
        ptx::tc_fence_before();
        __syncthreads();
        if (threadIdx.x == 0) {
            int acc   = 0;
            prefix[0] = 0;
            for (int b = 0; b < p.B; ++b) {
                acc += prefix[b + 1];
                prefix[b + 1] = acc;
            }
        }
        __syncthreads();
        ptx::tc_fence_after();
        const uint32_t tmem  = (uint32_t) ctl[0];
        const int      quota = tile_quota(p, prefix, (int) gridDim.x);
        const int      pos0  = (int) blockIdx.x * quota;
        const int      pos1  = pos0 + quota < prefix[p.B] ? pos0 + quota : prefix[p.B];

        if (warp == 0) {
            // ------------------------------------------------------------------ producer
            if (ptx::elect_one()) {
                int64_t g  = 0; // tile counter of this CTA, across items
                bool    ok = true;
                int     pos = pos0;
                for (int64_t ii = 0; ok; ++ii) {
                    const Item it = find_item(p, prefix, pos, pos1, quota);
                    if (!it.valid) break;
                    pos += it.ntiles;
                    const int qb = (int) (ii & 1);
                    ok = ptx::mbar_wait(bar(bQE + qb), ((ii >> 1) & 1) ^ 1, ctl + 1, p.dev_err);
                    if (!ok) break;
                    ptx::mbar_expect_tx(bar(bQF + qb), Q_BYTES);
                    const int qrow = it.b * p.Hkv * G + it.hk * G;
                    ptx::tma_load_2d(base + oQ + qb * Q_BYTES, &tmQ, 0, qrow, bar(bQF + qb));
                    ptx::tma_load_2d(base + oQ + qb * Q_BYTES + NPAD * 128, &tmQ, 64, qrow, bar(bQF + qb));
                    for (int t = 0; t < it.ntiles && ok; ++t, ++g) {
                        const int      s  = (int) (g % kStages);
                        const uint32_t ph = (uint32_t) ((g / kStages) & 1);
                        const int      j0 = (int) (it.start + (int64_t) t * TK);
                        ok = ptx::mbar_wait(bar(bKE + s), ph ^ 1, ctl + 1, p.dev_err);
                        if (!ok) break;
                        ptx::mbar_expect_tx(bar(bKF + s), KV_BYTES);
                        ptx::tma_load_4d(base + oK + s * KV_BYTES, &tmK, 0, j0, it.hk, it.b, bar(bKF + s));
                        ptx::tma_load_4d(base + oK + s * KV_BYTES + TK * 128, &tmK, 64, j0, it.hk, it.b, bar(bKF + s));
                        ok = ptx::mbar_wait(bar(bVE + s), ph ^ 1, ctl + 1, p.dev_err);
                        if (!ok) break;
                        ptx::mbar_expect_tx(bar(bVF + s), KV_BYTES);
                        ptx::tma_load_4d(base + oV + s * KV_BYTES, &tmV, 0, j0, it.hk, it.b, bar(bVF + s));
                        ptx::tma_load_4d(base + oV + s * KV_BYTES + TK * 128, &tmV, 64, j0, it.hk, it.b, bar(bVF + s));
                    }
                }
            }
        } else if (warp == 1) {
            // ------------------------------------------------------------------ MMA issuer
            if (ptx::elect_one()) {
                struct Cur {
                    Item    it;
                    int64_t ii, g;
                    int     t, pos; // pos: the item's first tile in the line
                };
                auto advance = [&](const Cur &c) -> Cur {
                    Cur n = c;
                    n.g   = c.g + 1;
                    if (c.t + 1 < c.it.ntiles) {
                        n.t = c.t + 1;
                    } else {
                        n.ii  = c.ii + 1;
                        n.t   = 0;
                        n.pos = c.pos + c.it.ntiles;
                        n.it  = find_item(p, prefix, n.pos, pos1, quota);
                    }
                    return n;
                };
                auto issue_qk = [&](const Cur &c) -> bool {
                    const int s = (int) (c.g % kStages), sb = (int) (c.g & 3), qb = (int) (c.ii & 1);
                    if (c.t == 0 && !ptx::mbar_wait(bar(bQF + qb), (uint32_t) ((c.ii >> 1) & 1), ctl + 1, p.dev_err)) return false;
                    if (!ptx::mbar_wait(bar(bKF + s), (uint32_t) ((c.g / kStages) & 1), ctl + 1, p.dev_err)) return false;
                    if (!ptx::mbar_wait(bar(bSE + sb), (uint32_t) (((c.g >> 2) & 1) ^ 1), ctl + 1, p.dev_err)) return false;
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k = 0; k < DH / 16; ++k) {
                        const uint64_t ad = ptx::smem_desc_sw128(base + oK + s * KV_BYTES + (k / 4) * (TK * 128) + (k % 4) * 32, 16, 1024);
                        const uint64_t bd = ptx::smem_desc_sw128(base + oQ + qb * Q_BYTES + (k / 4) * (NPAD * 128) + (k % 4) * 32, 16, 1024);
                        ptx::mma_f16_ss(tmem + sb * NPAD, ad, bd, kIdescQK, k != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(bar(bKE + s));
                    ptx::tc_commit(bar(bSF + sb));
                    if (c.t == c.it.ntiles - 1) ptx::tc_commit(bar(bQE + qb));
                    return true;
                };
                int  pc[2] = {0, 0}; // items each softmax group has taken part in so far (selects its O^T buffer)
                auto issue_pv = [&](const Cur &c) -> bool {
                    const int s = (int) (c.g % kStages), pb = (int) (c.g & 3), wg = c.t & 1, ob = pc[wg] & 1;
                    if (c.t < 2 && !ptx::mbar_wait(bar(bOE + wg * 2 + ob), (uint32_t) (((pc[wg] >> 1) & 1) ^ 1), ctl + 1, p.dev_err)) return false;
                    if (!ptx::mbar_wait(bar(bVF + s), (uint32_t) ((c.g / kStages) & 1), ctl + 1, p.dev_err)) return false;
                    if (!ptx::mbar_wait(bar(bPF + pb), (uint32_t) ((c.g >> 2) & 1), ctl + 1, p.dev_err)) return false;
                    ptx::tc_fence_after();
                    const uint32_t dcol = tmem + 4 * NPAD + (uint32_t) (wg * 2 + ob) * NPAD;
#pragma unroll
                    for (int k = 0; k < TK / 16; ++k) {
                        // A: V tile, two 64-dim spans of [128 keys x 128 B]; 16 keys per step = 2048 B
                        const uint64_t ad = ptx::smem_desc_sw128(base + oV + s * KV_BYTES + k * 2048, TK * 128, 1024);
                        // B: P^T, two 64-key spans of [16 heads x 128 B]
                        const uint64_t bd = ptx::smem_desc_sw128(base + oP + pb * P_BYTES + (k / 4) * (NPAD * 128) + (k % 4) * 32, 16, 1024);
                        ptx::mma_f16_ss(dcol, ad, bd, kIdescPV, (c.t >= 2 || k != 0) ? 1u : 0u);
                    }
                    ptx::tc_commit(bar(bVE + s));
                    ptx::tc_commit(bar(bPV + wg));
                    if (c.t + 2 >= c.it.ntiles) { // this group's last tile of the item
                        ptx::tc_commit(bar(bOF + wg * 2 + ob));
                        pc[wg]++;
                    }
                    return true;
                };
                // Q.K^T runs two tiles ahead of P.V so that both softmax groups always have a tile to work on
                Cur c0, c1, c2;
                c0.ii = 0, c0.g = 0, c0.t = 0, c0.pos = pos0;
                c0.it = find_item(p, prefix, pos0, pos1, quota);
                bool ok = c0.it.valid && issue_qk(c0);
                if (ok) {
                    c1 = advance(c0);
                    if (c1.it.valid) ok = issue_qk(c1);
                    while (ok) {
                        bool have2 = false;
                        if (c1.it.valid) {
                            c2    = advance(c1);
                            have2 = c2.it.valid;
                            if (have2 && !issue_qk(c2)) break;
                        }
                        if (!issue_pv(c0)) break;
                        if (!c1.it.valid) break;
                        c0 = c1;
                        if (have2) c1 = c2;
                        else c1.it.valid = false;
                    }
                }
            }
        } else {
            // ------------------------------------------------------------------ softmax groups + item epilogue
            const int      wg    = (warp - 2) >> 2;
            const int      q     = warp & 3;
            const int      r     = q * 32 + lane; // key within the tile / output dim in the epilogue
            const uint32_t tlane = (uint32_t) (q * 32) << 16;
            float         *redg  = red + wg * (2 * 4 * NPAD);
            float         *lsg   = lsum + wg * (2 * 4 * NPAD);
            const int64_t  Hq    = (int64_t) p.Hkv * G;
            int64_t        g0    = 0; // tile counter at the start of the current item
            int            pc    = 0; // items this group has taken part in
            int64_t        cnt   = 0; // tiles this group has processed
            bool           ok    = true;
            int            pos   = pos0;
            while (ok) {
                const Item it = find_item(p, prefix, pos, pos1, quota);
                if (!it.valid) break;
                pos += it.ntiles;
                if (it.last && wg == 0 && r == 0) p.nslots[it.b * p.Hkv + it.hk] = 2 * (it.split + 1);
                const int64_t prow = ((int64_t) it.b * Hq + (int64_t) it.hk * G) * p.parts_stride + (int64_t) it.split * 2 + wg;
                if (wg >= it.ntiles) {
                    // this group has no tile in the item: an empty partial (weight 0 in the merge)
                    for (int h = 0; h < G; ++h) {
                        p.part_o[(prow + (int64_t) h * p.parts_stride) * DH + r] = 0.f;
                        if (r == 0) {
                            p.part_ml[(prow + (int64_t) h * p.parts_stride) * 2 + 0] = -INFINITY;
                            p.part_ml[(prow + (int64_t) h * p.parts_stride) * 2 + 1] = 0.f;
                        }
                    }
                    g0 += it.ntiles;
                    continue;
                }
                const int      ob   = pc & 1;
                const uint32_t tO   = tmem + tlane + 4 * NPAD + (uint32_t) (wg * 2 + ob) * NPAD;
                float          m[NPAD], lp[NPAD];
#pragma unroll
                for (int h = 0; h < NPAD; ++h) {
                    m[h]  = -INFINITY;
                    lp[h] = 0.f;
                }
                for (int t = wg; t < it.ntiles; t += 2, ++cnt) {
                    const int64_t g  = g0 + t;
                    const int     sb = (int) (g & 3), rb = (int) (cnt & 1);
                    ok = ptx::mbar_wait(bar(bSF + sb), (uint32_t) ((g >> 2) & 1), ctl + 1, p.dev_err);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    uint32_t sv[16];
                    ptx::tmem_ld_x16(tmem + tlane + sb * NPAD, sv);
                    ptx::tc_wait_ld();
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(bar(bSE + sb));
                    const int64_t key   = it.start + (int64_t) t * TK + r;
                    const bool    valid = key < it.end;
                    float         x[NPAD];
#pragma unroll
                    for (int h = 0; h < NPAD; ++h) x[h] = (valid && h < G) ? __uint_as_float(sv[h]) * p.scale_log2 : -INFINITY;
                    // per-head maximum over the 128 keys of the tile
#pragma unroll
                    for (int h = 0; h < NPAD; ++h) {
                        if (h < G) {
                            float v = x[h];
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
                            if (lane == 0) redg[(rb * 4 + q) * NPAD + h] = v;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar(bRX + wg * 2 + rb));
                    ok = ptx::mbar_wait(bar(bRX + wg * 2 + rb), (uint32_t) ((cnt >> 1) & 1), ctl + 1, p.dev_err);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    bool  need = false;
                    float alpha[NPAD];
#pragma unroll
                    for (int h = 0; h < NPAD; ++h) {
                        alpha[h] = 1.f;
                        if (h < G) {
                            const float tm = fmaxf(fmaxf(redg[(rb * 4 + 0) * NPAD + h], redg[(rb * 4 + 1) * NPAD + h]),
                                                   fmaxf(redg[(rb * 4 + 2) * NPAD + h], redg[(rb * 4 + 3) * NPAD + h]));
                            if (tm > m[h] + kRescaleThreshold || (m[h] == -INFINITY && tm > m[h])) {
                                alpha[h] = m[h] == -INFINITY ? 0.f : fast_exp2(m[h] - tm);
                                need     = need || (t >= 2 && m[h] != -INFINITY);
                                m[h]     = tm;
                            }
                            lp[h] *= alpha[h];
                        }
                    }
                    if (need) { // uniform over the group's 128 threads: every input of the decision is
                        ok = ptx::mbar_wait(bar(bPV + wg), (uint32_t) ((cnt - 1) & 1), ctl + 1, p.dev_err);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                        ptx::tc_fence_after();
                        uint32_t ov[16];
                        ptx::tmem_ld_x16(tO, ov);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int h = 0; h < NPAD; ++h) ov[h] = __float_as_uint(__uint_as_float(ov[h]) * alpha[h]);
                        ptx::tmem_st_x16(tO, ov);
                        ptx::tc_wait_st();
                    }
                    // probabilities -> P^T[sb] (K-major, 128-byte swizzle: row = head, 64 keys per 128-byte span)
                    uint8_t       *pt = gbase + oP + sb * P_BYTES + (r >> 6) * (NPAD * 128);
                    const uint32_t w2 = (uint32_t) (r & 63) * 2;
#pragma unroll
                    for (int h = 0; h < NPAD; ++h) {
                        if (h < G) {
                            const float pv = valid ? fast_exp2(x[h] - m[h]) : 0.f;
                            lp[h] += pv;
                            T pvt;
                            St<T>::st(&pvt, pv);
                            const uint32_t off = (uint32_t) (h >> 3) * 1024 + (uint32_t) (h & 7) * 128 + (((w2 >> 4) ^ (uint32_t) (h & 7)) << 4) + (w2 & 15);
                            *reinterpret_cast<T *>(pt + off) = pvt;
                        }
                    }
                    if (!valid) {
                        // zero this key's V row in the stage: p = 0 must not meet whatever bit pattern lies past kv_len
                        const int s  = (int) (g % kStages);
                        uint8_t  *vr = gbase + oV + s * KV_BYTES + (r >> 3) * 1024 + (r & 7) * 128;
                        // the TMA write of this stage must have landed before it is overwritten
                        ptx::mbar_wait(bar(bVF + s), (uint32_t) ((g / kStages) & 1), ctl + 1, p.dev_err);
#pragma unroll
                        for (int sp = 0; sp < 2; ++sp)
#pragma unroll
                            for (int u = 0; u < 8; ++u) *reinterpret_cast<uint4 *>(vr + sp * (TK * 128) + u * 16) = make_uint4(0, 0, 0, 0);
                    }
                    ptx::fence_proxy_async();
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(bar(bPF + sb));
                }
                if (!ok) break;
                // ---- item epilogue of this group: row sums across its 128 threads, then O^T -> partial
#pragma unroll
                for (int h = 0; h < NPAD; ++h) {
                    if (h < G) {
                        float v = lp[h];
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                        if (lane == 0) lsg[(ob * 4 + q) * NPAD + h] = v;
                    }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar(bLS + wg));
                ok = ptx::mbar_wait(bar(bOF + wg * 2 + ob), (uint32_t) ((pc >> 1) & 1), ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tc_fence_after();
                uint32_t ov[16];
                ptx::tmem_ld_x16(tO, ov);
                ptx::tc_wait_ld();
                ptx::tc_fence_before();
                ptx::mbar_arrive(bar(bOE + wg * 2 + ob));
                ok = ptx::mbar_wait(bar(bLS + wg), (uint32_t) (pc & 1), ctl + 1, p.dev_err); // row sums of all four warps visible
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
#pragma unroll
                for (int h = 0; h < NPAD; ++h) {
                    if (h < G) {
                        const int64_t rowi = prow + (int64_t) h * p.parts_stride;
                        p.part_o[rowi * DH + r] = __uint_as_float(ov[h]);
                        if (r == 0) {
                            const float *ls          = lsg + ob * 4 * NPAD;
                            p.part_ml[rowi * 2 + 0] = m[h];
                            p.part_ml[rowi * 2 + 1] = ls[0 * NPAD + h] + ls[1 * NPAD + h] + ls[2 * NPAD + h] + ls[3 * NPAD + h];
                        }
                    }
                }
                pc++;
                g0 += it.ntiles;
            }
        }
        if (ctl[1]) {
            for (int i = 0; i < 50; ++i) __nanosleep(20000); // aborted: let copies in flight land
        }
        ptx::tc_fence_before();
        __syncthreads();
        if (warp == 1) ptx::tmem_dealloc(tmem, kTmemCols);
    }

    inline int decode_grid(int64_t max_tiles, int min_tiles, int sm_count) {
        const int64_t max_ctas = (max_tiles + min_tiles - 1) / min_tiles;
        return (int) (max_ctas < sm_count ? max_ctas : sm_count);
    }

} // namespace

// Host walk of the split kernel's work distribution (no device): kv_len is a HOST array of B lengths or NULL. Writes the
// items of CTA `cta`, six numbers each — sequence, kv head, first key, end key, slot pair, 1 if the item holds the unit's
// final tile — and returns their number (which may exceed max_items), -1 for a shape the kernel does not take. *grid_out
// receives the grid size.
int vkc_attn_decode_tc_items(int sm_count, int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D, const int32_t *kv_len, int min_tiles,
                             int parts_stride, int cta, int32_t *items, int max_items, int *grid_out) {
    const int64_t G = Hq / Hkv, max_tiles = B * Hkv * ((Lmax + TK - 1) / TK);
    if (D != DH || G > NPAD || min_tiles < 1 || B > kMaxPrefix || B < 1 || Lmax > INT32_MAX - TK || max_tiles > INT32_MAX / 2 ||
        2 * (((Lmax + TK - 1) / TK + min_tiles - 1) / min_tiles + 1) > parts_stride)
        return -1;
    DecParams p = {};
    p.kv_len = kv_len, p.B = (int) B, p.Hkv = (int) Hkv, p.G = (int) G, p.min_quota = min_tiles, p.parts_stride = parts_stride, p.Lmax = Lmax;
    const int grid = decode_grid(max_tiles, min_tiles, sm_count);
    if (grid_out) *grid_out = grid;
    if (cta < 0 || cta >= grid) return -1;
    static thread_local int prefix[kMaxPrefix + 1];
    prefix[0] = 0;
    for (int b = 0; b < p.B; ++b) prefix[b + 1] = prefix[b] + (int) (((seq_len(p, b) + TK - 1) / TK) * p.Hkv);
    const int quota = tile_quota(p, prefix, grid), pos0 = cta * quota;
    const int pos1  = pos0 + quota < prefix[p.B] ? pos0 + quota : prefix[p.B];
    int       n     = 0;
    for (int pos = pos0;;) {
        const Item it = find_item(p, prefix, pos, pos1, quota);
        if (!it.valid) break;
        if (n < max_items) {
            int32_t *row = items + 6 * n;
            row[0] = it.b, row[1] = it.hk, row[2] = (int32_t) it.start, row[3] = (int32_t) it.end, row[4] = it.split, row[5] = it.last;
        }
        ++n;
        pos += it.ntiles;
    }
    return n;
}

// Launches the split kernel only; the caller runs the merge kernel. Every CTA takes at least `min_tiles` 128-key
// tiles; a (sequence, kv head) unit is therefore cut into at most ceil(tiles / min_tiles) + 1 items, each of which fills
// two partial slots (one per softmax group). `parts_stride` slots per (sequence, query head); nslots[b][hk] receives the
// number of slots the unit filled (nothing is written for an empty sequence).
// Returns VKC_ERR_UNSUPPORTED for shapes this form does not cover (the SIMT form then takes over).
int vkc_attn_decode_tcgen05(vkc_ctx *ctx, const void *Q, const void *Kc, const void *Vc, int64_t B, int64_t Hq, int64_t Hkv, int64_t Lmax, int64_t D,
                            const int32_t *kv_len, float scale, float *part_ml, float *part_o, int *nslots, int min_tiles, int parts_stride,
                            int dtype, cudaStream_t st) {
    const int64_t G = Hq / Hkv;
    if (D != DH || G > NPAD || (dtype != VKC_F16 && dtype != VKC_BF16) || !(scale > 0.f) || min_tiles < 1 || B > kMaxPrefix)
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_decode_tcgen05: needs head dim 128, at most 16 query heads per kv head, 16-bit storage");
    const int64_t max_tiles = B * Hkv * ((Lmax + TK - 1) / TK);
    if (Lmax > INT32_MAX - TK || B * Hq > INT32_MAX || max_tiles > INT32_MAX / 2 ||
        2 * (((Lmax + TK - 1) / TK + min_tiles - 1) / min_tiles + 1) > parts_stride)
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_decode_tcgen05: extent too large");
    CUtensorMap tq, tk, tv;
    int         rc;
    {
        uint64_t dims[2] = {(uint64_t) D, (uint64_t) (B * Hq)};
        uint64_t str[1]  = {(uint64_t) D * 2};
        uint32_t box[2]  = {64, NPAD};
        if ((rc = vkc_make_tmap(ctx, &tq, dtype, Q, 2, dims, str, box))) return rc;
    }
    {
        uint64_t dims[4] = {(uint64_t) D, (uint64_t) Lmax, (uint64_t) Hkv, (uint64_t) B};
        uint64_t str[3]  = {(uint64_t) D * 2, (uint64_t) Lmax * D * 2, (uint64_t) Hkv * Lmax * D * 2};
        uint32_t box[4]  = {64, TK, 1, 1};
        if ((rc = vkc_make_tmap(ctx, &tk, dtype, Kc, 4, dims, str, box))) return rc;
        if ((rc = vkc_make_tmap(ctx, &tv, dtype, Vc, 4, dims, str, box))) return rc;
    }
    DecParams p;
    p.part_ml = part_ml, p.part_o = part_o, p.kv_len = kv_len;
    p.B = (int) B, p.Hkv = (int) Hkv, p.G = (int) G, p.min_quota = min_tiles, p.nslots = nslots, p.parts_stride = parts_stride, p.Lmax = Lmax;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.dev_err    = ctx->dev_err;
    const int grid = decode_grid(max_tiles, min_tiles, ctx->sm_count);
#define VKC_DTC(T_)                                                                                                  \
    do {                                                                                                             \
        auto kern_ = attn_decode_tc_kernel<T_>;                                                                      \
        if (int rc_ = vkc_configure_smem(ctx, kern_, (int) kSmemTotal)) return rc_;                                  \
        kern_<<<grid, kThreads, kSmemTotal, st>>>(tq, tk, tv, p); /* plain launch: dependent launch measured 2 % slower here */ \
    } while (0)
    if (dtype == VKC_F16)
        VKC_DTC(__half);
    else
        VKC_DTC(__nv_bfloat16);
#undef VKC_DTC
    return vkc_post_launch(ctx, "attn_decode_tcgen05");
}
