// K1 — batched GEMM on the 5th-generation tensor cores with a fused bias / GELU(erf) / residual epilogue.
//
//   D[b,m,n] = epi( sum_k A[b,m,k] * B[b,k,n] ),  A/B/D in f16 or bf16, fp32 accumulation in tensor memory.
//
// One CTA computes one 128 x BN output tile (BN in {64, 128, 192, 256}). The launcher picks tile width, ring depth,
// CTAs per SM and a split-K factor per problem: short-K problems run two CTAs per SM so that one CTA's epilogue
// overlaps the other's main loop; long-K problems that fit a single wave run one CTA per SM with the deepest operand
// ring that fits; when even the widest tiles leave most SMs idle, K is split over a thread-block cluster of two CTAs.
// Warp roles:
//   warp 0   : TMA producer  — one elected lane streams 128x64 A tiles and BNx64 B tiles (128-byte swizzle)
//              through a multi-stage shared-memory ring, completion on per-stage "full" mbarriers;
//   warp 1   : MMA issuer    — owns the tensor-memory allocation; one elected lane issues four
//              tcgen05.mma (M=128, N=BN, K=16) per stage and commits the stage's "empty" mbarrier;
//   warps 2-5: epilogue      — each warp owns the 32 TMEM lanes (= output rows) it may address, reads the
//              accumulator with tcgen05.ld, applies the epilogue in fp32, packs to the storage type into a
//              128-byte-swizzled staging block in the idle operand ring and stores each 64-column slab with one
//              TMA store (the residual slab is TMA-loaded into the same block first).
// Split-K: the CTAs of a cluster accumulate disjoint K ranges of the same tile; the tile's 64-column slabs are dealt
// out round-robin; every CTA stages its fp32 partial of the slabs it does not own in its ring and bulk-copies it
// (cp.async.bulk shared::cta -> shared::cluster) into the owner's receive area, crediting the owner's mbarrier with
// the bytes; the owner adds the partials in a fixed order and runs the epilogue. No global scratch, no second kernel.
// The kernel sets up barriers and tensor memory before griddepcontrol.wait, so under programmatic dependent launch
// its prologue overlaps the previous kernel's tail.
// B is taken either as [N,K] rows (K contiguous, "K-major") or as [K,N] rows (N contiguous, "MN-major"),
// so weights in the reference's row-major [K,N] initializer layout are consumed without a transpose.
// M/N/K tails rely on TMA zero fill for loads and on predicated stores.
#include "common.cuh"
#include "ptx.cuh"
#include "tensormap.cuh"
#include <cmath>
#include <cstdlib>

namespace {

    constexpr int BM       = 128;
    constexpr int BK       = 64;
    constexpr int kThreads = 192;

    struct GemmParams {
        const float *bias;
        const void  *residual;
        void        *D;
        int64_t      M, N, K;
        int64_t      ldd, stride_d;
        int          epilogue;
        int          a_bcast, b_bcast; // batch stride 0: always read batch slice 0
        int         *dev_err;
        int          tma_out;  // D (and the residual) meet the TMA alignment rules: staged, coalesced epilogue
        // optional gate: A is produced by other GPUs; the TMA producer polls their flags before its first load (vkc_gate_wait)
        const unsigned *gate_flags;
        int             gate_n;
        unsigned       *gate_state;
    };

    // GELU(erf) on two values at once with packed fp32 arithmetic and no special-function unit: erf(x), x = h/sqrt(2)
    // clamped to [-3, 3] (erf(3) = 1 - 2.2e-5), is x * P(x^2) with a degree-8 polynomial fitted to |error| < 2.1e-5,
    // so GELU is within 5e-5 of the erff form everywhere, far below the rounding of the 16-bit output. The operation
    // order of the reference chain (erf, +1, *h, *0.5) is kept.
    __device__ __forceinline__ float2 gelu_erf_pair(float2 h) {
        const float2 k = make_float2(0.70710678118f, 0.70710678118f);
        float2       x = ptx::fmul2(h, k);
        x.x            = fminf(fmaxf(x.x, -3.0f), 3.0f);
        x.y            = fminf(fmaxf(x.y, -3.0f), 3.0f);
        const float2 u = ptx::fmul2(x, x);
        auto         c = [](float v) { return make_float2(v, v); };
        float2       p = c(3.912539981e-08f);
        p              = ptx::ffma2(p, u, c(-1.883036475e-06f));
        p              = ptx::ffma2(p, u, c(4.008835822e-05f));
        p              = ptx::ffma2(p, u, c(-5.029218737e-04f));
        p              = ptx::ffma2(p, u, c(4.196857568e-03f));
        p              = ptx::ffma2(p, u, c(-2.499890141e-02f));
        p              = ptx::ffma2(p, u, c(1.109308004e-01f));
        p              = ptx::ffma2(p, u, c(-3.752196431e-01f));
        p              = ptx::ffma2(p, u, c(1.128250599e+00f));
        float2 t       = ptx::ffma2(p, x, c(1.0f)); // erf + 1
        t              = ptx::fmul2(t, h);
        return ptx::fmul2(t, c(0.5f));
    }

    // Split-K: kSplit CTAs of a cluster each accumulate a K range of the same output tile; the 64-column slabs of the
    // tile are dealt out round-robin to the CTAs, which receive the other CTAs' fp32 partials for their slabs in a
    // dedicated shared-memory area (32 KB per slab and sender) and run the epilogue on the sum.
    constexpr int recv_bytes(int bn, int split) {
        return split > 1 ? (split - 1) * (((bn + 63) / 64 + split - 1) / split) * 32768 : 0;
    }
    template <int BN, int kStages, int kSplit = 1> constexpr int smem_bytes() {
        return kStages * (BM * BK * 2 + BN * BK * 2) + 1024 /*align*/ + 256 /*barriers*/ + 1024 /*bias, BN <= 256 floats*/ + recv_bytes(BN, kSplit);
    }
    __host__ __device__ constexpr int tmem_cols(int bn) { return bn <= 32 ? 32 : bn <= 64 ? 64 : bn <= 128 ? 128 : 256; } // power of two >= BN

    // Epilogue warps of the one-tile form: eight (two per tensor-memory lane quarter, taking the tile's 64-column slabs
    // alternately) where one CTA has the SM to itself and K is not split, else four. The epilogue of this form is not hidden
    // behind anything, and a slab is a chain of latencies: 0.7 us each with one warp per quarter.
    __host__ __device__ constexpr int epi_warps(int ctas_per_sm, int split) { return ctas_per_sm == 1 && split == 1 ? 8 : 4; }
    __host__ __device__ constexpr int threads_of(int ctas_per_sm, int split) { return 64 + 32 * epi_warps(ctas_per_sm, split); }

    template <int BN, int kStages, int kCtasPerSm, typename T, bool B_KN, int kSplit = 1>
    __global__ void __launch_bounds__(threads_of(kCtasPerSm, kSplit), kCtasPerSm)
        gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmD,
                            const __grid_constant__ CUtensorMap tmR, GemmParams p) {
        static_assert((BN / 64 + (BN % 64 != 0)) * 16384 <= kStages * (BM * BK * 2 + BN * BK * 2), "epilogue staging must fit in the operand ring");
        static_assert(kSplit == 1 || 65536 + ((BN + 63) / 64 - ((BN + 63) / 64) / kSplit) * 32768 <= kStages * (BM * BK * 2 + BN * BK * 2),
                      "split-K send staging must fit in the operand ring behind the epilogue staging");
        constexpr int kEpiW = epi_warps(kCtasPerSm, kSplit), kThr = threads_of(kCtasPerSm, kSplit);
        // Residual epilogue without split-K: the residual slabs are fetched by the producer thread while the last K steps still
        // run, into the A stages of the ring that have seen their last use (slab i into the stage that K step num_kb + i would
        // take), instead of by the epilogue warps after the accumulator is complete (1.4 us of exposed latency). The output is
        // staged in the same blocks. Needs more stages than slabs.
        constexpr bool kEarlyRes = kSplit == 1 && kStages > (BN + 63) / 64;
        static_assert(BM * BK * 2 == 16384, "a slab's staging (4 warps x 4 KB) is exactly one A stage");
        static_assert(8 * (2 * kStages + 2 + kEpiW) <= 256, "barrier area");
        constexpr uint32_t A_BYTES = BM * BK * 2;
        constexpr uint32_t B_BYTES = BN * BK * 2;
        constexpr bool     kBf16   = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdesc  = ptx::idesc_f16(BM, BN, kBf16, false, B_KN);

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sA    = base;
        const uint32_t sB    = base + kStages * A_BYTES;
        const uint32_t sBar  = sB + kStages * B_BYTES; // full[kStages], empty[kStages], accum : 8 bytes each
        volatile int  *ctl   = (volatile int *) (gbase + kStages * (A_BYTES + B_BYTES) + 8 * (2 * kStages + 1));
        // ctl[0] = tmem base (written by tcgen05.alloc), ctl[1] = abort flag
        const uint32_t sSlot = sBar + 8 * (2 * kStages + 1);
        float         *sbias = (float *) (gbase + kStages * (A_BYTES + B_BYTES) + 256); // BN floats
        // split-K only: receive area for the other CTAs' partials and the mbarrier their arrivals complete
        constexpr int  kSlabsAll = (BN + 63) / 64, kOwnMax = (kSlabsAll + kSplit - 1) / kSplit;
        const uint32_t sRecv     = base + kStages * (A_BYTES + B_BYTES) + 256 + 1024;
        const uint32_t sRecvBar  = sBar + 8 * (2 * kStages + 6);

        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int krank = kSplit > 1 ? (int) ptx::cluster_ctarank() : 0; // = blockIdx.x % kSplit
        const int m0 = (blockIdx.x / kSplit) * BM, n0 = blockIdx.y * BN, bz = blockIdx.z;
        const int num_kb_all = (int) ((p.K + BK - 1) / BK);
        const int kb_per     = (num_kb_all + kSplit - 1) / kSplit; // the launcher guarantees every rank a non-empty range
        const int kb0        = krank * kb_per;
        const int num_kb     = (kb0 + kb_per < num_kb_all ? kb0 + kb_per : num_kb_all) - kb0;

        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) {
                ptx::mbar_init(sBar + 8 * s, 1);
                ptx::mbar_init(sBar + 8 * (kStages + s), 1);
            }
            ptx::mbar_init(sBar + 8 * 2 * kStages, 1);
            for (int w = 0; w < kEpiW; ++w) ptx::mbar_init(sBar + 8 * (2 * kStages + 2 + w), 1); // residual tile landed, per epilogue warp
            if (kSplit > 1) ptx::mbar_init(sRecvBar, 1); // this CTA's own arrival; the partials arrive as transaction bytes
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmA);
            ptx::prefetch_tmap(&tmB);
        }
        if (warp == 1) {
            ptx::tmem_alloc(sSlot, tmem_cols(BN));
            ptx::tmem_relinquish();
        }
        if (kSplit > 1) {
            if (threadIdx.x == 0) {
                int mine = 0;
                for (int sl = krank; sl < kSlabsAll; sl += kSplit)
                    if ((int64_t) n0 + sl * 64 < p.N) ++mine;
                ptx::mbar_expect_tx(sRecvBar, (uint32_t) ((kSplit - 1) * mine) * 32768u);
            }
            ptx::cluster_arrive(); // barriers exist; the matching wait sits in front of each role's first use of a peer
        }
        ptx::tc_fence_before();
        __syncthreads();
        ptx::tc_fence_after();
        const uint32_t tmem = (uint32_t) ctl[0];
        // Everything above overlapped the previous kernel's tail; global memory from here on. (The set-up barrier comes first so
        // that nothing but the wait itself stands between the previous kernel's end and the producer's first TMA load.)
        vkc_grid_dep_wait();
        vkc_grid_dep_launch();
        if (warp >= 2 && (p.epilogue & VKC_EPI_BIAS)) {
            // The bias goes to shared memory behind the set-up barrier and is published among the epilogue warps only (named
            // barrier 1): in front of that barrier its load latency would sit between the producer thread and its first TMA load.
            for (int j = threadIdx.x - 64; j < BN; j += kThr - 64) sbias[j] = (int64_t) n0 + j < p.N ? __ldg(p.bias + n0 + j) : 0.f;
            asm volatile("bar.sync 1, %0;" ::"n"(kThr - 64) : "memory");
        }

        if (warp == 0) {
            if (ptx::elect_one()) {
                const int za = p.a_bcast ? 0 : bz, zb = p.b_bcast ? 0 : bz;
                bool      gate_ok = true;
                if (p.gate_flags) {
                    gate_ok = vkc_gate_wait(p.gate_flags, p.gate_n, p.gate_state, gridDim.x * gridDim.y * gridDim.z, p.dev_err);
                    if (!gate_ok) ctl[1] = 1; // the other roles leave through their bounded waits
                }
                for (int kb = 0; kb < num_kb && gate_ok; ++kb) {
                    const int      s  = kb % kStages;
                    const uint32_t ph = (kb / kStages) & 1;
                    const int      kx = (kb0 + kb) * BK; // element offset along K
                    if (!ptx::mbar_wait(sBar + 8 * (kStages + s), ph ^ 1, ctl + 1, p.dev_err)) break;
                    const uint32_t full = sBar + 8 * s;
                    ptx::mbar_expect_tx(full, A_BYTES + B_BYTES);
                    ptx::tma_load_3d(sA + s * A_BYTES, &tmA, kx, m0, za, full);
                    if (!B_KN) {
                        ptx::tma_load_3d(sB + s * B_BYTES, &tmB, kx, n0, zb, full);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c) ptx::tma_load_3d(sB + s * B_BYTES + c * (BK * 128), &tmB, n0 + c * 64, kx, zb, full);
                    }
                }
                if (kEarlyRes && gate_ok && !ctl[1] && p.tma_out && (p.epilogue & VKC_EPI_RESIDUAL)) {
                    int nslab = 0;
                    for (int sl = 0; sl < (BN + 63) / 64; ++sl)
                        if ((int64_t) n0 + sl * 64 < p.N) nslab = sl + 1;
                    // one arrival with the byte count per epilogue warp (warp ew handles lane quarter (ew + 2) & 3 and, with eight
                    // warps, the slabs of parity ew / 4)
                    for (int ew = 0; ew < kEpiW; ++ew) {
                        const int q = (ew + 2) & 3, first = kEpiW == 8 ? ew >> 2 : 0, step = kEpiW == 8 ? 2 : 1;
                        int       mine = 0;
                        for (int sl = first; sl < nslab; sl += step) ++mine;
                        if (m0 + q * 32 < p.M && mine > 0) ptx::mbar_expect_tx(sBar + 8 * (2 * kStages + 2 + ew), (uint32_t) mine * 4096u);
                    }
                    for (int sl = 0; sl < nslab; ++sl) {
                        const int kbp = num_kb + sl, s = kbp % kStages;
                        if (!ptx::mbar_wait(sBar + 8 * (kStages + s), (uint32_t) (((kbp / kStages) & 1) ^ 1), ctl + 1, p.dev_err)) break;
                        for (int q = 0; q < 4; ++q) {
                            const int ew = (kEpiW == 8 ? (sl & 1) * 4 : 0) + ((q + 2) & 3);
                            if (m0 + q * 32 < p.M)
                                ptx::tma_load_3d(sA + s * A_BYTES + q * 4096, &tmR, n0 + sl * 64, m0 + q * 32, bz, sBar + 8 * (2 * kStages + 2 + ew));
                        }
                    }
                }
            }
            if (kSplit > 1) ptx::cluster_wait();
        } else if (warp == 1) {
            if (ptx::elect_one()) {
                bool ok = true;
                for (int kb = 0; kb < num_kb && ok; ++kb) {
                    const int      s  = kb % kStages;
                    const uint32_t ph = (kb / kStages) & 1;
                    ok                = ptx::mbar_wait(sBar + 8 * s, ph, ctl + 1, p.dev_err);
                    if (!ok) break;
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t ad = ptx::smem_desc_sw128(sA + s * A_BYTES + k * 32, 16, 1024);
                        const uint64_t bd = B_KN ? ptx::smem_desc_sw128(sB + s * B_BYTES + k * (16 * 128), BK * 128, 1024)
                                                 : ptx::smem_desc_sw128(sB + s * B_BYTES + k * 32, 16, 1024);
                        ptx::mma_f16_ss(tmem, ad, bd, kIdesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    ptx::tc_commit(sBar + 8 * (kStages + s)); // frees the stage once these MMAs have read it
                }
                if (ok) ptx::tc_commit(sBar + 8 * 2 * kStages); // accumulator complete
            }
            if (kSplit > 1) ptx::cluster_wait();
        } else {
            const bool ok = ptx::mbar_wait(sBar + 8 * 2 * kStages, 0, ctl + 1, p.dev_err);
            ptx::tc_fence_after();
            bool recv_ok = true;
            if (kSplit > 1) {
                // Send this CTA's partial of every slab it does not own to the owner: each warp stages its 32 rows of the
                // slab (256 bytes per row, 16-byte chunks XOR-swizzled by row & 7) in the idle operand ring behind the
                // epilogue's own staging blocks, then one bulk copy moves the 8 KB into the owner's receive area and
                // credits the owner's mbarrier.
                const int q = warp & 3;
                ptx::cluster_wait();
                if (ok) {
                    int nth = 0; // ordinal of the slab among the ones this CTA sends
#pragma unroll 1
                    for (int sl = 0; sl < kSlabsAll; ++sl) {
                        const int owner = sl % kSplit;
                        if (owner == krank) continue;
                        if ((int64_t) n0 + sl * 64 >= p.N) break;
                        const int      slot  = (krank - owner - 1 + kSplit) % kSplit;
                        const uint32_t stage = base + 65536u + (uint32_t) (nth * 32768 + q * 8192);
                        const uint32_t dst   = sRecv + (uint32_t) ((slot * kOwnMax + sl / kSplit) * 32768 + q * 8192);
                        ++nth;
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            uint32_t r[32];
                            ptx::tmem_ld_x32(tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (sl * 64 + hf * 32), r);
                            ptx::tc_wait_ld();
#pragma unroll
                            for (int u = 0; u < 8; ++u)
                                ptx::st_shared_v4(stage + (uint32_t) (lane * 256 + (((hf * 8 + u) ^ (lane & 7)) << 4)), r[4 * u], r[4 * u + 1], r[4 * u + 2],
                                                  r[4 * u + 3]);
                        }
                        ptx::fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) ptx::bulk_copy_to_peer(ptx::mapa(dst, (uint32_t) owner), stage, 8192u, ptx::mapa(sRecvBar, (uint32_t) owner));
                    }
                }
                recv_ok = ptx::mbar_wait_cluster(sRecvBar, 0, ctl + 1, p.dev_err);
                recv_ok = __all_sync(0xffffffffu, recv_ok);
            }
            if (ok && recv_ok) {
                const int     q   = warp & 3; // the TMEM lane quarter this warp may address
                const int64_t m   = (int64_t) m0 + q * 32 + lane;
                T            *drow = (T *) p.D + (int64_t) bz * p.stride_d + m * p.ldd;
                const T      *rrow = p.residual ? (const T *) p.residual + (int64_t) bz * p.stride_d + m * p.ldd : nullptr;
                const bool    vec_ok = (p.ldd % 8 == 0) && (p.stride_d % 8 == 0) && (((uintptr_t) p.D & 15) == 0) &&
                                    (!p.residual || ((uintptr_t) p.residual & 15) == 0);
                if (p.tma_out) {
                    // Staged epilogue. The operand ring is idle now; each warp owns 32 output rows and, per 64-column
                    // slab, a 32 x 128 B staging block there (128-byte swizzle so that 8 lanes writing 8 different rows
                    // hit different banks). The residual slab is TMA-loaded into the same block, the result is written
                    // over it and leaves with one TMA store: global traffic is full 128-byte lines both ways.
                    constexpr int kSlabs = (BN + 63) / 64;
                    const int      row0  = m0 + q * 32;
                    const bool     rows_in = row0 < p.M; // warp-uniform
                    // this warp's slabs: first, first + step, ... (split-K: the slabs this CTA owns; eight warps: alternate slabs)
                    const int      first = kEpiW == 8 ? (warp - 2) >> 2 : krank, step = kEpiW == 8 ? 2 : kSplit;
                    const uint32_t rbar  = sBar + 8 * (2 * kStages + 2 + (warp - 2));
                    int            nslab = 0, nmine = 0; // slabs inside N; of those, the ones this warp finishes
                    for (int sl = 0; sl < kSlabs; ++sl)
                        if ((int64_t) n0 + sl * 64 < p.N) {
                            nslab = sl + 1;
                            if (sl % step == first) ++nmine;
                        }
                    // staging block of slab sl: A stage sl, or (residual fetched early) the A stage that K step num_kb + sl would take
                    const bool early = kEarlyRes && (p.epilogue & VKC_EPI_RESIDUAL);
                    auto       blk_of = [&](int sl) { return (uint32_t) ((early ? (num_kb + sl) % kStages : sl) * 16384 + q * 4096); };
                    bool rok = true;
                    if ((p.epilogue & VKC_EPI_RESIDUAL) && rows_in && nmine > 0) {
                        if (lane == 0 && !early) {
                            ptx::mbar_expect_tx(rbar, (uint32_t) nmine * 4096u);
                            for (int sl = first; sl < nslab; sl += step) ptx::tma_load_3d(base + blk_of(sl), &tmR, n0 + sl * 64, row0, bz, rbar);
                        }
                        rok = ptx::mbar_wait(rbar, 0, ctl + 1, p.dev_err);
                        rok = __all_sync(0xffffffffu, rok);
                    }
#pragma unroll 1
                    for (int sl = first; sl < nslab && rok; sl += step) {
                        uint8_t *blk = gbase + blk_of(sl) + lane * 128;
                        // both 32-column halves are fetched before the single wait, so that their arithmetic interleaves
                        uint32_t r2[2][32];
                        ptx::tmem_ld_x32(tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (sl * 64), r2[0]);
                        ptx::tmem_ld_x32(tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (sl * 64 + 32), r2[1]);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
                            float v[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r2[hf][j]);
                            if (kSplit > 1) {
                                // add the other CTAs' partials of this row (fixed order: slot 0, 1, ...)
#pragma unroll
                                for (int slot = 0; slot < kSplit - 1; ++slot) {
                                    const uint8_t *rrow_ = gbase + kStages * (A_BYTES + B_BYTES) + 256 + 1024 +
                                                           (slot * kOwnMax + sl / kSplit) * 32768 + (q * 32 + lane) * 256;
#pragma unroll
                                    for (int u = 0; u < 8; ++u) {
                                        const float4 pv = *reinterpret_cast<const float4 *>(rrow_ + (((hf * 8 + u) ^ (lane & 7)) << 4));
                                        v[4 * u] += pv.x, v[4 * u + 1] += pv.y, v[4 * u + 2] += pv.z, v[4 * u + 3] += pv.w;
                                    }
                                }
                            }
                            if (p.epilogue & VKC_EPI_BIAS) {
#pragma unroll
                                for (int j = 0; j < 32; j += 4) {
                                    const float4 bv = *reinterpret_cast<const float4 *>(sbias + sl * 64 + hf * 32 + j);
                                    v[j] += bv.x, v[j + 1] += bv.y, v[j + 2] += bv.z, v[j + 3] += bv.w;
                                }
                            }
                            if (p.epilogue & VKC_EPI_GELU_ERF) {
#pragma unroll
                                for (int j = 0; j < 32; j += 2) {
                                    const float2 g2 = gelu_erf_pair(make_float2(v[j], v[j + 1]));
                                    v[j] = g2.x, v[j + 1] = g2.y;
                                }
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                uint4 *slot = reinterpret_cast<uint4 *>(blk + (((hf * 4 + u) ^ (lane & 7)) << 4));
                                if (p.epilogue & VKC_EPI_RESIDUAL) {
                                    const uint4 rv = *slot;
                                    const T    *rt = reinterpret_cast<const T *>(&rv);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) v[u * 8 + j] += St<T>::ld(rt + j);
                                }
                                uint4 ov;
                                T    *ot = reinterpret_cast<T *>(&ov);
#pragma unroll
                                for (int j = 0; j < 8; ++j) St<T>::st(ot + j, v[u * 8 + j]);
                                *slot = ov;
                            }
                        }
                        ptx::fence_proxy_async();
                        __syncwarp();
                        if (lane == 0 && rows_in) {
                            ptx::tma_store_3d(&tmD, base + blk_of(sl), n0 + sl * 64, row0, bz);
                            ptx::bulk_commit_group();
                        }
                    }
                    if (lane == 0) ptx::bulk_wait_group_read_0();
                    __syncwarp();
                } else if (warp < 6) // (plain stores, unaligned outputs: one warp per lane quarter does all columns)
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    const int64_t nb = (int64_t) n0 + c * 32;
                    if (nb >= p.N) break; // uniform across the CTA
                    uint32_t r[32];
                    ptx::tmem_ld_x32(tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (c * 32), r);
                    ptx::tc_wait_ld();
                    if (m < p.M) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        const bool full = nb + 32 <= p.N;
                        if (p.epilogue & VKC_EPI_BIAS) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 bv = *reinterpret_cast<const float4 *>(sbias + c * 32 + j);
                                v[j] += bv.x, v[j + 1] += bv.y, v[j + 2] += bv.z, v[j + 3] += bv.w;
                            }
                        }
                        if (p.epilogue & VKC_EPI_GELU_ERF) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = vkc_gelu_erf_fast(v[j]);
                        }
                        if (full && vec_ok) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                if (p.epilogue & VKC_EPI_RESIDUAL) {
                                    uint4    rv = *reinterpret_cast<const uint4 *>(rrow + nb + g * 8);
                                    const T *rt = reinterpret_cast<const T *>(&rv);
#pragma unroll
                                    for (int j = 0; j < 8; ++j) v[g * 8 + j] += St<T>::ld(rt + j);
                                }
                                uint4 ov;
                                T    *ot = reinterpret_cast<T *>(&ov);
#pragma unroll
                                for (int j = 0; j < 8; ++j) St<T>::st(ot + j, v[g * 8 + j]);
                                *reinterpret_cast<uint4 *>(drow + nb + g * 8) = ov;
                            }
                        } else {
                            for (int j = 0; j < 32; ++j) {
                                if (nb + j < p.N) {
                                    float o = v[j];
                                    if (p.epilogue & VKC_EPI_RESIDUAL) o += St<T>::ld(rrow + nb + j);
                                    St<T>::st(drow + nb + j, o);
                                }
                            }
                        }
                    }
                }
            }
        }
        if (ctl[1]) {
            // aborted: give copies still in flight time to land before the CTA releases its shared memory
            for (int i = 0; i < 50; ++i) __nanosleep(20000);
        }
        ptx::tc_fence_before();
        __syncthreads();
        if (warp == 1) ptx::tmem_dealloc(tmem, tmem_cols(BN));
        if (kSplit > 1) ptx::cluster_sync(); // no CTA releases its shared memory while another may still write into it
    }

    template <int BN, int kStages, int kCtasPerSm, typename T, bool B_KN, int kSplit = 1>
    int launch(vkc_ctx *ctx, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmD, const CUtensorMap &tmR, const GemmParams &p,
               int64_t batch, cudaStream_t st) {
        auto          kern = gemm_tcgen05_kernel<BN, kStages, kCtasPerSm, T, B_KN, kSplit>;
        constexpr int smem = smem_bytes<BN, kStages, kSplit>();
        static_assert(smem * kCtasPerSm <= 227 * 1024, "shared memory budget");
        static_assert(8 * (2 * kStages + 7) <= 256, "barrier area");
        if (int rc = vkc_configure_smem(ctx, kern, smem)) return rc;
        dim3 grid((unsigned) ((p.M + BM - 1) / BM) * kSplit, (unsigned) ((p.N + BN - 1) / BN), (unsigned) batch);
        vkc_launch_cluster(ctx, kern, grid, dim3(threads_of(kCtasPerSm, kSplit)), smem, st, (unsigned) kSplit, tmA, tmB, tmD, tmR, p);
        return vkc_post_launch(ctx, "gemm_tcgen05");
    }

    // ---------------------------------------------------------------------------------------------------------------
    // Persistent form: one CTA per SM walks over output tiles (tile t, t + gridDim.x, ...). The accumulator is double
    // buffered in tensor memory, so the epilogue of tile i runs while the tensor pipe already works on tile i + 1, and
    // the operand ring keeps streaming across tile boundaries. The epilogue therefore cannot borrow the operand ring:
    // every epilogue warp owns three 32 x 128 B staging blocks that rotate over its 64-column slabs (residual slab
    // TMA-loaded into the block one slab ahead, result written over it, one TMA store per slab).
    constexpr int kPBlocks = 3; // staging blocks per epilogue warp
    // The persistent form runs EIGHT epilogue warps, two per tensor-memory lane quarter, which take the 64-column slabs of a tile
    // alternately: a slab is a chain of latencies (tensor-memory load, arithmetic, shared-memory store, proxy fence, bulk store)
    // that one warp per quarter cannot hide, and with short K the four-warp epilogue, not the K loop, set the pace of a tile
    // (1.4 us per 128 x 128 tile without and 2.9 us with GELU against 2.3 us of MMAs at K = 768).
    constexpr int kEpiWarpsP = 8, kThreadsP = 64 + kEpiWarpsP * 32;
    template <int BN, int kStages> constexpr int smem_bytes_persistent() {
        return kStages * (BM * BK * 2 + BN * BK * 2) + kEpiWarpsP * 4096 + 1024 /*align*/ + 512 /*barriers*/ + kEpiWarpsP * BN * 4 /*bias, per warp*/;
    }
    __host__ __device__ constexpr int acc_stride(int bn) { return bn <= 128 ? 128 : 256; } // TMEM columns between the two accumulators

    template <int BN, int kStages, typename T, bool B_KN>
    __global__ void __launch_bounds__(kThreadsP, 1)
        gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                       const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmR, GemmParams p, int m_tiles,
                                       int n_tiles, int total_tiles) {
        constexpr uint32_t A_BYTES = BM * BK * 2;
        constexpr uint32_t B_BYTES = BN * BK * 2;
        constexpr bool     kBf16   = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdesc  = ptx::idesc_f16(BM, BN, kBf16, false, B_KN);
        constexpr int      kSlabs  = (BN + 63) / 64;
        constexpr uint32_t kRing   = kStages * (A_BYTES + B_BYTES);
        constexpr uint32_t kStage  = kEpiWarpsP * 4096;

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sA    = base;
        const uint32_t sB    = base + kStages * A_BYTES;
        const uint32_t sOut  = base + kRing;          // one 4 KB staging block per epilogue warp
        const uint32_t sBar  = base + kRing + kStage; // full[kStages], empty[kStages], accFull[2], accEmpty[2], resid[epilogue warps]
        const uint32_t bAccF = sBar + 8 * (2 * kStages), bAccE = bAccF + 16, bRes = bAccE + 16;
        volatile int  *ctl   = (volatile int *) (gbase + kRing + kStage + 8 * (2 * kStages + 4 + kEpiWarpsP)); // [0] tmem base, [1] abort
        const uint32_t sSlot = sBar + 8 * (2 * kStages + 4 + kEpiWarpsP);
        float         *sbias = (float *) (gbase + kRing + kStage + 512); // [epilogue warps][BN]
        static_assert(8 * (2 * kStages + 4 + kEpiWarpsP) + 16 <= 512, "barrier area");

        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int num_kb = (int) ((p.K + BK - 1) / BK);

        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) {
                ptx::mbar_init(sBar + 8 * s, 1);
                ptx::mbar_init(sBar + 8 * (kStages + s), 1);
            }
            for (int b = 0; b < 2; ++b) {
                ptx::mbar_init(bAccF + 8 * b, 1);
                ptx::mbar_init(bAccE + 8 * b, kEpiWarpsP); // one arrival per epilogue warp
            }
            for (int w = 0; w < kEpiWarpsP; ++w) ptx::mbar_init(bRes + 8 * w, 1);
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmA);
            ptx::prefetch_tmap(&tmB);
            ptx::prefetch_tmap(&tmD);
        }
        if (warp == 1) {
            ptx::tmem_alloc(sSlot, 2 * acc_stride(BN));
            ptx::tmem_relinquish();
        }
        ptx::tc_fence_before();
        __syncthreads();
        ptx::tc_fence_after();
        const uint32_t tmem = (uint32_t) ctl[0];
        vkc_grid_dep_wait(); // behind the set-up barrier: only the wait stands between the previous kernel's end and the first TMA load
        vkc_grid_dep_launch();

        // tile t -> (row tile fastest, then column tile, then batch): concurrently running CTAs share few B tiles
        auto tile_of = [&](int t, int &m0, int &n0, int &bz) {
            m0 = (t % m_tiles) * BM;
            n0 = ((t / m_tiles) % n_tiles) * BN;
            bz = t / (m_tiles * n_tiles);
        };

        if (warp == 0) {
            if (ptx::elect_one()) {
                int  it = 0;
                bool ok = true;
                if (p.gate_flags) {
                    ok = vkc_gate_wait(p.gate_flags, p.gate_n, p.gate_state, gridDim.x, p.dev_err);
                    if (!ok) ctl[1] = 1;
                }
                for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                    int m0, n0, bz;
                    tile_of(t, m0, n0, bz);
                    const int za = p.a_bcast ? 0 : bz, zb = p.b_bcast ? 0 : bz;
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int      s  = it % kStages;
                        const uint32_t ph = (it / kStages) & 1;
                        const int      kx = kb * BK;
                        if (!ptx::mbar_wait(sBar + 8 * (kStages + s), ph ^ 1, ctl + 1, p.dev_err)) {
                            ok = false;
                            break;
                        }
                        const uint32_t full = sBar + 8 * s;
                        ptx::mbar_expect_tx(full, A_BYTES + B_BYTES);
                        ptx::tma_load_3d(sA + s * A_BYTES, &tmA, kx, m0, za, full);
                        if (!B_KN) {
                            ptx::tma_load_3d(sB + s * B_BYTES, &tmB, kx, n0, zb, full);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN / 64; ++c) ptx::tma_load_3d(sB + s * B_BYTES + c * (BK * 128), &tmB, n0 + c * 64, kx, zb, full);
                        }
                    }
                }
            }
        } else if (warp == 1) {
            if (ptx::elect_one()) {
                int  it = 0, i = 0;
                bool ok = true;
                for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++i) {
                    const int      buf = i & 1;
                    const uint32_t acc = tmem + (uint32_t) (buf * acc_stride(BN));
                    // the epilogue warps have drained this accumulator (two tiles ago)
                    ok = ptx::mbar_wait(bAccE + 8 * buf, ((i >> 1) & 1) ^ 1, ctl + 1, p.dev_err);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int      s  = it % kStages;
                        const uint32_t ph = (it / kStages) & 1;
                        ok                = ptx::mbar_wait(sBar + 8 * s, ph, ctl + 1, p.dev_err);
                        if (!ok) break;
                        ptx::tc_fence_after();
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) {
                            const uint64_t ad = ptx::smem_desc_sw128(sA + s * A_BYTES + k * 32, 16, 1024);
                            const uint64_t bd = B_KN ? ptx::smem_desc_sw128(sB + s * B_BYTES + k * (16 * 128), BK * 128, 1024)
                                                     : ptx::smem_desc_sw128(sB + s * B_BYTES + k * 32, 16, 1024);
                            ptx::mma_f16_ss(acc, ad, bd, kIdesc, (kb | k) != 0 ? 1u : 0u);
                        }
                        ptx::tc_commit(sBar + 8 * (kStages + s));
                    }
                    if (ok) ptx::tc_commit(bAccF + 8 * buf);
                }
            }
        } else {
            const int      q      = warp & 3;        // the TMEM lane quarter this warp may address
            const int      ew     = warp - 2;        // epilogue warp number
            const int      half   = ew >> 2;         // takes the slabs of this parity
            float         *wbias  = sbias + ew * BN;
            const uint32_t wOut   = sOut + (uint32_t) ew * 4096u;
            uint8_t       *gOut   = gbase + kRing + ew * 4096;
            const uint32_t wRes   = bRes + 8 * ew;
            const bool     resid  = (p.epilogue & VKC_EPI_RESIDUAL) != 0;
            auto           nslabs = [&](int n0) {
                int n = 0;
                for (int sl = 0; sl < kSlabs; ++sl)
                    if ((int64_t) n0 + sl * 64 < p.N) n = sl + 1;
                return n;
            };
            int  g  = 0; // slabs this warp has been through (phase of its residual barrier)
            bool ok = true;
            int  i  = 0;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++i) {
                int m0, n0, bz;
                tile_of(t, m0, n0, bz);
                const int  buf = i & 1, nslab = nslabs(n0), row0 = m0 + q * 32;
                const bool rows_in = row0 < p.M; // warp-uniform
                __syncwarp();
                if (p.epilogue & VKC_EPI_BIAS)
                    for (int j = lane; j < BN; j += 32) wbias[j] = (int64_t) n0 + j < p.N ? __ldg(p.bias + n0 + j) : 0.f;
                __syncwarp();
                ok = ptx::mbar_wait(bAccF + 8 * buf, (i >> 1) & 1, ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t acc = tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (buf * acc_stride(BN));
                if (half >= nslab) { // no slab of this tile is this warp's: it has nothing to drain
                    if (lane == 0) ptx::mbar_arrive(bAccE + 8 * buf);
                    continue;
                }
#pragma unroll 1
                for (int sl = half; sl < nslab; sl += 2, ++g) {
                    if (resid) {
                        // the residual slab goes into the staging block, which is free once the previous store has read it
                        if (lane == 0) {
                            ptx::bulk_wait_group_read_0();
                            ptx::mbar_expect_tx(wRes, 4096u);
                            ptx::tma_load_3d(wOut, &tmR, n0 + sl * 64, row0, bz, wRes);
                        }
                        __syncwarp();
                    }
                    uint32_t r2[2][32];
                    ptx::tmem_ld_x32(acc + (uint32_t) (sl * 64), r2[0]);
                    ptx::tmem_ld_x32(acc + (uint32_t) (sl * 64 + 32), r2[1]);
                    ptx::tc_wait_ld();
                    if (sl + 2 >= nslab) { // this warp's part of the accumulator is drained: the tensor pipe may overwrite it
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(bAccE + 8 * buf);
                    }
                    // bias and GELU in registers first; the staging block is only needed after that
                    float v[2][32];
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[hf][j] = __uint_as_float(r2[hf][j]);
                        if (p.epilogue & VKC_EPI_BIAS) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 bv = *reinterpret_cast<const float4 *>(wbias + sl * 64 + hf * 32 + j);
                                v[hf][j] += bv.x, v[hf][j + 1] += bv.y, v[hf][j + 2] += bv.z, v[hf][j + 3] += bv.w;
                            }
                        }
                        if (p.epilogue & VKC_EPI_GELU_ERF) {
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                const float2 g2 = gelu_erf_pair(make_float2(v[hf][j], v[hf][j + 1]));
                                v[hf][j] = g2.x, v[hf][j + 1] = g2.y;
                            }
                        }
                    }
                    if (resid) {
                        ok = ptx::mbar_wait(wRes, (uint32_t) (g & 1), ctl + 1, p.dev_err);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                    } else {
                        if (lane == 0) ptx::bulk_wait_group_read_0(); // the previous store of this warp has read the block
                        __syncwarp();
                    }
                    uint8_t *blkp = gOut + lane * 128;
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            uint4 *slot = reinterpret_cast<uint4 *>(blkp + (((hf * 4 + u) ^ (lane & 7)) << 4));
                            if (resid) {
                                const uint4 rv = *slot;
                                const T    *rt = reinterpret_cast<const T *>(&rv);
#pragma unroll
                                for (int j = 0; j < 8; ++j) v[hf][u * 8 + j] += St<T>::ld(rt + j);
                            }
                            uint4 ov;
                            T    *ot = reinterpret_cast<T *>(&ov);
#pragma unroll
                            for (int j = 0; j < 8; ++j) St<T>::st(ot + j, v[hf][u * 8 + j]);
                            *slot = ov;
                        }
                    }
                    ptx::fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (rows_in) ptx::tma_store_3d(&tmD, wOut, n0 + sl * 64, row0, bz);
                        ptx::bulk_commit_group();
                    }
                }
            }
            if (lane == 0) ptx::bulk_wait_group_read_0();
            __syncwarp();
        }
        if (ctl[1]) {
            // aborted: give copies still in flight time to land before the CTA releases its shared memory
            for (int i = 0; i < 50; ++i) __nanosleep(20000);
        }
        ptx::tc_fence_before();
        __syncthreads();
        if (warp == 1) ptx::tmem_dealloc(tmem, 2 * acc_stride(BN));
    }

    template <int BN, int kStages, typename T, bool B_KN>
    int launch_persistent(vkc_ctx *ctx, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmD, const CUtensorMap &tmR,
                          const GemmParams &p, int64_t batch, cudaStream_t st) {
        auto          kern = gemm_tcgen05_persistent_kernel<BN, kStages, T, B_KN>;
        constexpr int smem = smem_bytes_persistent<BN, kStages>();
        static_assert(smem <= 227 * 1024, "shared memory budget");
        if (int rc = vkc_configure_smem(ctx, kern, smem)) return rc;
        const int64_t mt = (p.M + BM - 1) / BM, nt = (p.N + BN - 1) / BN, total = mt * nt * batch;
        if (total > INT32_MAX) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: too many tiles");
        const int64_t ctas = total < ctx->sm_count ? total : ctx->sm_count;
        vkc_launch(ctx, kern, dim3((unsigned) ctas), dim3(kThreadsP), smem, st, tmA, tmB, tmD, tmR, p, (int) mt, (int) nt, (int) total);
        return vkc_post_launch(ctx, "gemm_tcgen05_persistent");
    }

    // ---------------------------------------------------------------------------------------------------------------
    // CTA-pair form: two CTAs on two SMs (a cluster of two) drive ONE tcgen05.mma.cta_group::2 stream over a 256 x BN output
    // tile. Each CTA loads its own 128 rows of A and HALF of the B tile; the tensor cores of both SMs read both halves, so
    // per k-step a CTA pulls 16 KB + BN x 64 bytes from L2 for 128 x BN x 64 multiply-adds — half the B traffic of the
    // one-CTA forms, which at 128 x 256 tiles need about 96 bytes per clock and SM and are fed at 55-85. Everything else is the
    // persistent form above: pairs walk over output tiles, the accumulator is double buffered in tensor memory (each CTA holds
    // its 128 rows), the operand ring streams across tile boundaries, every epilogue warp owns rotating staging blocks.
    //   warp 0 (both CTAs): TMA producer; the completion bytes of BOTH CTAs' loads are counted on the LEADER's "full" barrier
    //   warp 1 (leader):    MMA issuer; commits each stage's "empty" barrier and each tile's "accumulator full" barrier in
    //                       both CTAs; waits for "accumulator empty" arrivals from the epilogue warps of both CTAs
    //   warps 2-5:          epilogue over the CTA's own 128 accumulator rows
    // Every CTA fetches what it keeps; no load is shared between the CTAs of a pair.
    template <int BN, int kStages> constexpr int smem_bytes_pair() {
        return kStages * (BM * BK * 2 + (BN / 2) * BK * 2) + 4 * kPBlocks * 4096 + 1024 /*align*/ + 512 /*barriers*/ + 4 * BN * 4 /*bias, per warp*/;
    }

    template <int BN, int kStages, typename T, bool B_KN>
    __global__ void __launch_bounds__(kThreads, 1)
        gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                 const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmR, GemmParams p, int m_tiles,
                                 int n_tiles, int total_tiles) {
        constexpr uint32_t A_BYTES = BM * BK * 2;
        constexpr uint32_t B_BYTES = (BN / 2) * BK * 2; // this CTA's half of the B tile
        constexpr bool     kBf16   = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdesc  = ptx::idesc_f16(2 * BM, BN, kBf16, false, B_KN);
        constexpr int      kSlabs  = (BN + 63) / 64;
        constexpr uint32_t kRing   = kStages * (A_BYTES + B_BYTES);
        constexpr uint32_t kStage  = 4 * kPBlocks * 4096;

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sA    = base;
        const uint32_t sB    = base + kStages * A_BYTES;
        const uint32_t sOut  = base + kRing;
        const uint32_t sBar  = base + kRing + kStage; // full[kStages], empty[kStages], accFull[2], accEmpty[2], resid[4][kPBlocks]
        const uint32_t bAccF = sBar + 8 * (2 * kStages), bAccE = bAccF + 16, bRes = bAccE + 16;
        volatile int  *ctl   = (volatile int *) (gbase + kRing + kStage + 8 * (2 * kStages + 4 + 4 * kPBlocks)); // [0] tmem base, [1] abort
        const uint32_t sSlot = sBar + 8 * (2 * kStages + 4 + 4 * kPBlocks);
        float         *sbias = (float *) (gbase + kRing + kStage + 512); // [4 warps][BN]
        static_assert(8 * (2 * kStages + 4 + 4 * kPBlocks) + 16 <= 512, "barrier area");

        const int      warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const uint32_t rank = ptx::cluster_ctarank(); // 0 = leader
        const int      pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
        const int      num_kb = (int) ((p.K + BK - 1) / BK);

        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) {
                ptx::mbar_init(sBar + 8 * s, 1);
                ptx::mbar_init(sBar + 8 * (kStages + s), 1);
            }
            for (int b = 0; b < 2; ++b) {
                ptx::mbar_init(bAccF + 8 * b, 1);
                ptx::mbar_init(bAccE + 8 * b, 8); // one arrival per epilogue warp of both CTAs (used in the leader only)
            }
            for (int w = 0; w < 4 * kPBlocks; ++w) ptx::mbar_init(bRes + 8 * w, 1);
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmA);
            ptx::prefetch_tmap(&tmB);
            ptx::prefetch_tmap(&tmD);
        }
        if (warp == 1) {
            ptx::tmem_alloc_pair(sSlot, 2 * acc_stride(BN));
            ptx::tmem_relinquish_pair();
        }
        vkc_grid_dep_wait();
        vkc_grid_dep_launch();
        ptx::tc_fence_before();
        __syncthreads();
        ptx::cluster_sync(); // both CTAs' barriers exist before either side signals them
        ptx::tc_fence_after();
        const uint32_t tmem = (uint32_t) ctl[0];

        // tile t -> groups of kGroupM pair-row tiles; inside a group the row tile runs fastest, then the column tile; then the
        // next group, then the batch. The pairs that run at the same time then share a few hundred rows of A and columns of B
        // (for 8192^3: 8 x 9 tiles, 71 MB of operands) instead of a full column of row tiles, so the operands stay in L2.
        // m0 is this CTA's first row.
        constexpr int kGroupM = 8;
        auto tile_of = [&](int t, int &m0, int &n0, int &bz) {
            const int per_batch = m_tiles * n_tiles, tb = t % per_batch;
            const int grp = tb / (kGroupM * n_tiles), first = grp * kGroupM;
            const int gsz = m_tiles - first < kGroupM ? m_tiles - first : kGroupM;
            const int in_g = tb - grp * (kGroupM * n_tiles);
            m0 = (first + in_g % gsz) * (2 * BM) + (int) rank * BM;
            n0 = (in_g / gsz) * BN;
            bz = t / per_batch;
        };

        if (warp == 0) {
            if (ptx::elect_one()) {
                int  it = 0;
                bool ok = true;
                if (p.gate_flags) {
                    ok = vkc_gate_wait(p.gate_flags, p.gate_n, p.gate_state, gridDim.x, p.dev_err);
                    if (!ok) ctl[1] = 1;
                }
                for (int t = pair; t < total_tiles && ok; t += npairs) {
                    int m0, n0, bz;
                    tile_of(t, m0, n0, bz);
                    const int za = p.a_bcast ? 0 : bz, zb = p.b_bcast ? 0 : bz;
                    const int nb = n0 + (int) rank * (BN / 2); // this CTA's half of the tile's columns
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int      s  = it % kStages;
                        const uint32_t ph = (it / kStages) & 1;
                        const int      kx = kb * BK;
                        if (!ptx::mbar_wait(sBar + 8 * (kStages + s), ph ^ 1, ctl + 1, p.dev_err)) {
                            ok = false;
                            break;
                        }
                        const uint32_t full = ptx::mapa(sBar + 8 * s, 0);
                        if (rank == 0) ptx::mbar_expect_tx(sBar + 8 * s, 2 * (A_BYTES + B_BYTES)); // the bytes of both CTAs
                        ptx::tma_load_3d_pair(sA + s * A_BYTES, &tmA, kx, m0, za, full);
                        if (!B_KN) {
                            ptx::tma_load_3d_pair(sB + s * B_BYTES, &tmB, kx, nb, zb, full);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN / 128; ++c) ptx::tma_load_3d_pair(sB + s * B_BYTES + c * (BK * 128), &tmB, nb + c * 64, kx, zb, full);
                        }
                    }
                }
            }
        } else if (warp == 1) {
            if (rank == 0 && ptx::elect_one()) {
                int  it = 0, i = 0;
                bool ok = true;
                for (int t = pair; t < total_tiles && ok; t += npairs, ++i) {
                    const int      buf = i & 1;
                    const uint32_t acc = tmem + (uint32_t) (buf * acc_stride(BN));
                    // the epilogue warps of both CTAs have drained this accumulator (two tiles ago)
                    ok = ptx::mbar_wait_cluster(bAccE + 8 * buf, ((i >> 1) & 1) ^ 1, ctl + 1, p.dev_err);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    for (int kb = 0; kb < num_kb; ++kb, ++it) {
                        const int      s  = it % kStages;
                        const uint32_t ph = (it / kStages) & 1;
                        ok                = ptx::mbar_wait_cluster(sBar + 8 * s, ph, ctl + 1, p.dev_err);
                        if (!ok) break;
                        ptx::tc_fence_after();
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k) {
                            const uint64_t ad = ptx::smem_desc_sw128(sA + s * A_BYTES + k * 32, 16, 1024);
                            const uint64_t bd = B_KN ? ptx::smem_desc_sw128(sB + s * B_BYTES + k * (16 * 128), BK * 128, 1024)
                                                     : ptx::smem_desc_sw128(sB + s * B_BYTES + k * 32, 16, 1024);
                            ptx::mma_f16_ss_pair(acc, ad, bd, kIdesc, (kb | k) != 0 ? 1u : 0u);
                        }
                        // the stage is free in BOTH CTAs once these MMAs have read it
                        ptx::tc_commit_pair(sBar + 8 * (kStages + s));
                        ptx::tc_commit_pair(ptx::mapa(sBar + 8 * (kStages + s), 1));
                    }
                    if (ok) {
                        ptx::tc_commit_pair(bAccF + 8 * buf);
                        ptx::tc_commit_pair(ptx::mapa(bAccF + 8 * buf, 1));
                    }
                }
            }
        } else {
            const int      q      = warp & 3; // the TMEM lane quarter this warp may address
            float         *wbias  = sbias + q * BN;
            const uint32_t wOut   = sOut + (uint32_t) (q * kPBlocks) * 4096u;
            uint8_t       *gOut   = gbase + kRing + (q * kPBlocks) * 4096;
            const uint32_t wRes   = bRes + 8 * (q * kPBlocks);
            const bool     resid  = (p.epilogue & VKC_EPI_RESIDUAL) != 0;
            const uint32_t accE0  = ptx::mapa(bAccE, 0); // the leader's "accumulator empty" barriers
            auto           nslabs = [&](int n0) {
                int n = 0;
                for (int sl = 0; sl < kSlabs; ++sl)
                    if ((int64_t) n0 + sl * 64 < p.N) n = sl + 1;
                return n;
            };
            int  g  = 0; // running slab number of this warp: staging block g % kPBlocks, use (g / kPBlocks) of that block
            bool ok = true;
            if (resid && pair < total_tiles && lane == 0) {
                int m0, n0, bz;
                tile_of(pair, m0, n0, bz);
                ptx::mbar_expect_tx(wRes, 4096u);
                ptx::tma_load_3d(wOut, &tmR, n0, m0 + q * 32, bz, wRes);
            }
            int i = 0;
            for (int t = pair; t < total_tiles && ok; t += npairs, ++i) {
                int m0, n0, bz;
                tile_of(t, m0, n0, bz);
                const int  buf = i & 1, nslab = nslabs(n0), row0 = m0 + q * 32;
                const bool rows_in = row0 < p.M; // warp-uniform
                __syncwarp();
                if (p.epilogue & VKC_EPI_BIAS)
                    for (int j = lane; j < BN; j += 32) wbias[j] = (int64_t) n0 + j < p.N ? __ldg(p.bias + n0 + j) : 0.f;
                __syncwarp();
                ok = ptx::mbar_wait(bAccF + 8 * buf, (i >> 1) & 1, ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t acc = tmem + ((uint32_t) (q * 32) << 16) + (uint32_t) (buf * acc_stride(BN));
#pragma unroll 1
                for (int sl = 0; sl < nslab; ++sl, ++g) {
                    const int blk = g % kPBlocks;
                    if (lane == 0) {
                        ptx::bulk_wait_group_read_1();
                        if (resid) {
                            int  tm0 = m0, tn0 = n0 + (sl + 1) * 64, tbz = bz;
                            bool more = sl + 1 < nslab;
                            if (!more && t + npairs < total_tiles) {
                                tile_of(t + npairs, tm0, tn0, tbz);
                                more = true;
                            }
                            if (more) {
                                const int nb = (g + 1) % kPBlocks;
                                ptx::mbar_expect_tx(wRes + 8 * nb, 4096u);
                                ptx::tma_load_3d(wOut + nb * 4096, &tmR, tn0, tm0 + q * 32, tbz, wRes + 8 * nb);
                            }
                        }
                    }
                    __syncwarp();
                    uint32_t r2[2][32];
                    ptx::tmem_ld_x32(acc + (uint32_t) (sl * 64), r2[0]);
                    ptx::tmem_ld_x32(acc + (uint32_t) (sl * 64 + 32), r2[1]);
                    ptx::tc_wait_ld();
                    if (sl == nslab - 1) { // accumulator drained: the tensor pipe may overwrite it
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive_cluster(accE0 + 8 * buf);
                    }
                    if (resid) {
                        ok = ptx::mbar_wait(wRes + 8 * blk, (g / kPBlocks) & 1, ctl + 1, p.dev_err);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok) break;
                    }
                    uint8_t *blkp = gOut + blk * 4096 + lane * 128;
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r2[hf][j]);
                        if (p.epilogue & VKC_EPI_BIAS) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 bv = *reinterpret_cast<const float4 *>(wbias + sl * 64 + hf * 32 + j);
                                v[j] += bv.x, v[j + 1] += bv.y, v[j + 2] += bv.z, v[j + 3] += bv.w;
                            }
                        }
                        if (p.epilogue & VKC_EPI_GELU_ERF) {
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                const float2 g2 = gelu_erf_pair(make_float2(v[j], v[j + 1]));
                                v[j] = g2.x, v[j + 1] = g2.y;
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            uint4 *slot = reinterpret_cast<uint4 *>(blkp + (((hf * 4 + u) ^ (lane & 7)) << 4));
                            if (resid) {
                                const uint4 rv = *slot;
                                const T    *rt = reinterpret_cast<const T *>(&rv);
#pragma unroll
                                for (int j = 0; j < 8; ++j) v[u * 8 + j] += St<T>::ld(rt + j);
                            }
                            uint4 ov;
                            T    *ot = reinterpret_cast<T *>(&ov);
#pragma unroll
                            for (int j = 0; j < 8; ++j) St<T>::st(ot + j, v[u * 8 + j]);
                            *slot = ov;
                        }
                    }
                    ptx::fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (rows_in) ptx::tma_store_3d(&tmD, wOut + blk * 4096, n0 + sl * 64, row0, bz);
                        ptx::bulk_commit_group(); // committed even when empty: the rotation counts groups
                    }
                }
            }
            if (lane == 0) ptx::bulk_wait_group_read_0();
            __syncwarp();
        }
        if (ctl[1]) {
            // aborted: give copies still in flight time to land before the CTA releases its shared memory
            for (int i = 0; i < 50; ++i) __nanosleep(20000);
        }
        ptx::tc_fence_before();
        __syncthreads();
        ptx::cluster_sync(); // neither CTA leaves while the other may still touch its shared memory, barriers or tensor memory
        if (warp == 1) ptx::tmem_dealloc_pair(tmem, 2 * acc_stride(BN));
    }

    template <int BN, int kStages, typename T, bool B_KN>
    int launch_pair(vkc_ctx *ctx, const CUtensorMap &tmA, const CUtensorMap &tmB, const CUtensorMap &tmD, const CUtensorMap &tmR, const GemmParams &p,
                    int64_t batch, cudaStream_t st) {
        auto          kern = gemm_tcgen05_pair_kernel<BN, kStages, T, B_KN>;
        constexpr int smem = smem_bytes_pair<BN, kStages>();
        static_assert(smem <= 227 * 1024, "shared memory budget");
        if (int rc = vkc_configure_smem(ctx, kern, smem)) return rc;
        const int64_t mt = (p.M + 2 * BM - 1) / (2 * BM), nt = (p.N + BN - 1) / BN, total = mt * nt * batch;
        if (total > INT32_MAX) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: too many tiles");
        const int64_t pairs = total < ctx->sm_count / 2 ? total : ctx->sm_count / 2;
        vkc_launch_cluster(ctx, kern, dim3((unsigned) (2 * pairs)), dim3(kThreads), smem, st, 2u, tmA, tmB, tmD, tmR, p, (int) mt, (int) nt, (int) total);
        return vkc_post_launch(ctx, "gemm_tcgen05_pair");
    }

    // Tile width: fewest waves over the SMs first, then the least padded work. Wide tiles re-read A less often.
    // Configurations the launcher can pick: tile width, ring depth, CTAs per SM, split-K factor.
    enum TileConfig {
        kCfg256x4x1, // 256 wide, 4 stages, one CTA per SM: large problems
        kCfg256x2x2,
        kCfg192x2x2,
        kCfg128x3x2,
        kCfg64x4x2,
        kCfg192x5x1,   // deep ring, one CTA per SM: a single wave of long-K tiles
        kCfg128x6x1,
        kCfg192x4x1s2, // split-K over a cluster of two CTAs
        kCfg256x3x1s2,
        kCfg128x5x1s2,
        kCfgP256x3, // persistent, double-buffered accumulator: the epilogue overlaps the next tile's K loop
        kCfgP192x4,
        kCfgP128x5,
        kCfgPair256x5, // CTA pairs (cta_group::2), 256 x 256 tiles, persistent
        kCfgPair128x6, // CTA pairs, 256 x 128 tiles
        kNumConfigs
    };
    struct TileChoice {
        TileConfig cfg;
        int        bn;
    };
    // Measured behaviour behind the rules: a tile's K loop is fed at 55-85 bytes per clock per SM from L2, so long-K
    // problems that fit one wave want the deepest ring that fits (one CTA per SM); when even the widest tiles leave most
    // SMs idle, splitting K over a cluster of two fills them; short-K problems are dominated by prologue and epilogue
    // and run best as two co-resident CTAs per SM.
    // A GELU epilogue is arithmetic-bound (about as long as a short K loop); with several tiles per SM the persistent form
    // hides it behind the next tile's K loop.
    TileChoice choose_tile(int64_t M, int64_t N, int64_t K, int64_t batch, int sms, bool staged, int epilogue) {
        const int64_t mt     = (M + BM - 1) / BM;
        auto          tiles  = [&](int bn) { return mt * ((N + bn - 1) / bn) * batch; };
        const int64_t num_kb = (K + BK - 1) / BK;
        // large problems in every dimension: CTA pairs halve the B traffic per SM (4096^3: 97.8 us against 109)
        if (staged && M >= 2048 && N >= 2048 && K >= 2048) return {kCfgPair256x5, 256};
        if (tiles(256) >= 4 * (int64_t) sms) return {kCfg256x4x1, 256};
        if (staged && (epilogue & VKC_EPI_GELU_ERF) && tiles(128) >= 2 * (int64_t) sms) return {kCfgP128x5, 128};
        if (num_kb >= 16) {
            // one-wave candidates, scored by busy SMs (ties: wider tile = less operand traffic)
            struct Cand {
                TileConfig cfg;
                int        bn, split;
            };
            const Cand cands[5] = {{kCfg192x5x1, 192, 1}, {kCfg128x6x1, 128, 1}, {kCfg192x4x1s2, 192, 2}, {kCfg256x3x1s2, 256, 2}, {kCfg128x5x1s2, 128, 2}};
            int64_t    best_ctas = 0;
            int        best      = -1;
            for (int i = 0; i < 5; ++i) {
                if (cands[i].split > 1 && (!staged || num_kb < 8 * cands[i].split)) continue;
                const int64_t ctas = tiles(cands[i].bn) * cands[i].split;
                if (ctas > sms) continue;
                if (ctas > best_ctas) best_ctas = ctas, best = i;
            }
            if (best >= 0 && best_ctas * 10 >= (int64_t) sms * 6) return {cands[best].cfg, cands[best].bn};
            // a few row tiles and a very long K (the row shards of a token-sharded encoder: 342 x 1024 x 4096): half of K per CTA
            // still beats one narrow tile per CTA over the whole K (10.5 against 13.3 us)
            if (best >= 0 && cands[best].split == 2 && num_kb >= 32 && best_ctas * 10 >= (int64_t) sms * 3) return {cands[best].cfg, cands[best].bn};
        }
        TileChoice    best {kCfg128x3x2, 128};
        double        best_cost = 1e300;
        const int     cands[4]  = {256, 192, 128, 64};
        const TileConfig cfgs[4] = {kCfg256x2x2, kCfg192x2x2, kCfg128x3x2, kCfg64x4x2};
        for (int i = 0; i < 4; ++i) {
            // two co-resident CTAs share one tensor pipe: model a slot as half an SM
            const double waves = std::ceil((double) tiles(cands[i]) / (2.0 * sms));
            const double cost  = waves * (cands[i] + 48.0); // per-tile time ~ width + fixed prologue/epilogue
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best      = {cfgs[i], cands[i]};
            }
        }
        return best;
    }

} // namespace

extern "C" int vkc_gemm_config_count(void) { return kNumConfigs; }

// Returns VKC_ERR_UNSUPPORTED (without touching ctx->err semantics beyond the message) when the operands do not
// meet the TMA alignment rules; the caller then uses the SIMT kernel.
int vkc_gemm_tcgen05(vkc_ctx *ctx, const void *A, const void *B, const float *bias, const void *residual, void *D, int64_t M, int64_t N,
                     int64_t K, int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_d, int64_t lda, int64_t ldb, int64_t ldd,
                     int b_layout, int epilogue, int dtype, int config, const vkc_gate *gate, cudaStream_t st) {
    if (dtype != VKC_F16 && dtype != VKC_BF16) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: 16-bit storage only");
    if ((lda % 8) || (ldb % 8) || (stride_a % 8) || (stride_b % 8) || ((uintptr_t) A & 15) || ((uintptr_t) B & 15))
        return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: operand strides/bases must be multiples of 16 bytes");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > 65535) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: extent too large");

    const bool a_bcast = stride_a == 0 || batch == 1, b_bcast = stride_b == 0 || batch == 1;
    // split-K needs the staged (TMA) epilogue; its alignment conditions are the ones checked for tma_out below
    const bool can_stage = (ldd % 8 == 0) && (stride_d % 8 == 0) && (((uintptr_t) D & 15) == 0) &&
                           (!(epilogue & VKC_EPI_RESIDUAL) || (((uintptr_t) residual & 15) == 0));
    // output / residual maps for the staged epilogue (box = 64 columns x 32 rows, one per epilogue warp and slab)
    CUtensorMap tmD, tmR;
    memset(&tmD, 0, sizeof tmD);
    memset(&tmR, 0, sizeof tmR);
    bool tma_out = false;
    if (can_stage) {
        uint64_t dims[3] = {(uint64_t) N, (uint64_t) M, (uint64_t) batch};
        uint64_t str[2]  = {(uint64_t) ldd * 2, (uint64_t) (batch > 1 ? (uint64_t) stride_d * 2 : (uint64_t) ldd * 2 * (uint64_t) M)};
        uint32_t box[3]  = {64, 32, 1};
        int      rc      = vkc_make_tmap(ctx, &tmD, dtype, D, 3, dims, str, box);
        if (rc == VKC_OK && (epilogue & VKC_EPI_RESIDUAL)) rc = vkc_make_tmap(ctx, &tmR, dtype, residual, 3, dims, str, box);
        tma_out = rc == VKC_OK;
    }

    TileChoice tc = choose_tile(M, N, K, batch, ctx->sm_count, tma_out, epilogue);
    if (config >= 0) { // caller-chosen configuration (autotuning); refuse what this problem cannot run
        const int  bns[kNumConfigs] = {256, 256, 192, 128, 64, 192, 128, 192, 256, 128, 256, 192, 128, 256, 128};
        const int  split            = (config >= kCfg192x4x1s2 && config <= kCfg128x5x1s2) ? 2 : 1;
        if (((config >= kCfgP256x3 && config <= kCfgP128x5) || config >= kCfgPair256x5) && !tma_out)
            return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: persistent configuration %d needs a TMA-storable output", config);
        if (config >= kCfgPair256x5 && M <= BM)
            return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: CTA-pair configuration %d needs more than one 128-row tile", config);
        // every CTA of the cluster must get a non-empty K range: ceil(kb / split) * (split - 1) < kb
        const int64_t nkb = (K + BK - 1) / BK;
        if (split > 1 && (!tma_out || nkb < 2 * split || ((nkb + split - 1) / split) * (split - 1) >= nkb))
            return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "gemm_tcgen05: split-K configuration %d needs a TMA-storable output and at least %d k-steps", config, 2 * split);
        tc = {(TileConfig) config, bns[config]};
    }
    const int        BN = tc.bn;

    CUtensorMap tmA, tmB;
    {
        uint64_t dims[3] = {(uint64_t) K, (uint64_t) M, (uint64_t) (a_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) lda * 2, (uint64_t) (a_bcast ? (uint64_t) lda * 2 * (uint64_t) M : (uint64_t) stride_a * 2)};
        uint32_t box[3]  = {BK, BM, 1};
        int      rc      = vkc_make_tmap(ctx, &tmA, dtype, A, 3, dims, str, box);
        if (rc) return rc;
    }
    if (b_layout == VKC_B_NK) {
        uint64_t dims[3] = {(uint64_t) K, (uint64_t) N, (uint64_t) (b_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) ldb * 2, (uint64_t) (b_bcast ? (uint64_t) ldb * 2 * (uint64_t) N : (uint64_t) stride_b * 2)};
        uint32_t box[3]  = {BK, (uint32_t) (tc.cfg >= kCfgPair256x5 ? BN / 2 : BN), 1}; // a CTA of a pair loads half of the tile's columns
        int      rc      = vkc_make_tmap(ctx, &tmB, dtype, B, 3, dims, str, box);
        if (rc) return rc;
    } else {
        uint64_t dims[3] = {(uint64_t) N, (uint64_t) K, (uint64_t) (b_bcast ? 1 : batch)};
        uint64_t str[2]  = {(uint64_t) ldb * 2, (uint64_t) (b_bcast ? (uint64_t) ldb * 2 * (uint64_t) K : (uint64_t) stride_b * 2)};
        uint32_t box[3]  = {64, BK, 1};
        int      rc      = vkc_make_tmap(ctx, &tmB, dtype, B, 3, dims, str, box);
        if (rc) return rc;
    }
    GemmParams p;
    p.bias     = bias;
    p.residual = residual;
    p.D        = D;
    p.M        = M;
    p.N        = N;
    p.K        = K;
    p.ldd      = ldd;
    p.stride_d = stride_d;
    p.epilogue = epilogue;
    p.a_bcast  = a_bcast;
    p.b_bcast  = b_bcast;
    p.dev_err  = ctx->dev_err;
    p.tma_out  = tma_out ? 1 : 0;
    p.gate_flags = gate ? gate->flags : nullptr;
    p.gate_n     = gate ? gate->n : 0;
    p.gate_state = gate ? gate->state : nullptr;
#define VKC_GEMM_LAUNCH(BN_, ST_, C_, T_)                                                                       \
    (b_layout == VKC_B_KN ? launch<BN_, ST_, C_, T_, true>(ctx, tmA, tmB, tmD, tmR, p, batch, st) \
                          : launch<BN_, ST_, C_, T_, false>(ctx, tmA, tmB, tmD, tmR, p, batch, st))
#define VKC_GEMM_LAUNCH_S(BN_, ST_, C_, T_, S_)                                                                    \
    (b_layout == VKC_B_KN ? launch<BN_, ST_, C_, T_, true, S_>(ctx, tmA, tmB, tmD, tmR, p, batch, st) \
                          : launch<BN_, ST_, C_, T_, false, S_>(ctx, tmA, tmB, tmD, tmR, p, batch, st))
#define VKC_GEMM_LAUNCH_P(BN_, ST_, T_)                                                                      \
    (b_layout == VKC_B_KN ? launch_persistent<BN_, ST_, T_, true>(ctx, tmA, tmB, tmD, tmR, p, batch, st) \
                          : launch_persistent<BN_, ST_, T_, false>(ctx, tmA, tmB, tmD, tmR, p, batch, st))
#define VKC_GEMM_LAUNCH_2(BN_, ST_, T_)                                                                \
    (b_layout == VKC_B_KN ? launch_pair<BN_, ST_, T_, true>(ctx, tmA, tmB, tmD, tmR, p, batch, st) \
                          : launch_pair<BN_, ST_, T_, false>(ctx, tmA, tmB, tmD, tmR, p, batch, st))
#define VKC_GEMM_BY_TILE(T_)                                                         \
    do {                                                                             \
        switch (tc.cfg) {                                                            \
            case kCfg256x4x1: return VKC_GEMM_LAUNCH(256, 4, 1, T_);                 \
            case kCfg256x2x2: return VKC_GEMM_LAUNCH(256, 2, 2, T_);                 \
            case kCfg192x2x2: return VKC_GEMM_LAUNCH(192, 2, 2, T_);                 \
            case kCfg128x3x2: return VKC_GEMM_LAUNCH(128, 3, 2, T_);                 \
            case kCfg64x4x2: return VKC_GEMM_LAUNCH(64, 4, 2, T_);                   \
            case kCfg192x5x1: return VKC_GEMM_LAUNCH(192, 5, 1, T_);                 \
            case kCfg128x6x1: return VKC_GEMM_LAUNCH(128, 6, 1, T_);                 \
            case kCfg192x4x1s2: return VKC_GEMM_LAUNCH_S(192, 4, 1, T_, 2);          \
            case kCfg256x3x1s2: return VKC_GEMM_LAUNCH_S(256, 3, 1, T_, 2);          \
            case kCfgP256x3: return VKC_GEMM_LAUNCH_P(256, 3, T_);                   \
            case kCfgP192x4: return VKC_GEMM_LAUNCH_P(192, 4, T_);                   \
            case kCfgP128x5: return VKC_GEMM_LAUNCH_P(128, 5, T_);                   \
            case kCfgPair256x5: return VKC_GEMM_LAUNCH_2(256, 5, T_);                \
            case kCfgPair128x6: return VKC_GEMM_LAUNCH_2(128, 6, T_);                \
            default: return VKC_GEMM_LAUNCH_S(128, 5, 1, T_, 2);                     \
        }                                                                            \
    } while (0)
    if (dtype == VKC_F16) VKC_GEMM_BY_TILE(__half);
    VKC_GEMM_BY_TILE(__nv_bfloat16);
#undef VKC_GEMM_BY_TILE
#undef VKC_GEMM_LAUNCH
#undef VKC_GEMM_LAUNCH_S
#undef VKC_GEMM_LAUNCH_P
#undef VKC_GEMM_LAUNCH_2
}
