// K2 — fused prefill attention on the 5th-generation tensor cores (flash style: the score matrix never leaves
// the SM). A CTA works on TWO 128-row query tiles (A and B) of one (batch, head) at a time — a unit — and walks the
// key/value sequence in tiles of 128 keys; while the softmax warps of one query tile work, the tensor core runs the
// MMAs of the other. For head size 64 and only a few units a one-tile form runs instead, two CTAs per SM: the same overlap
// happens between the co-resident CTAs.
// Work distribution: with per-sequence lengths (or a causal mask on a small or ragged problem) one CTA per unit. Otherwise the
// work comes in blocks of equal length — a unit without a mask; with a causal mask the pair of query groups (n-1-k, k) of a
// head — and the CTAs are persistent (one per SM): whole blocks round-robin, then the blocks left over cut into equal pieces of
// their key range, one piece per CTA, whose normalised partial rows a merge kernel joins with their (maximum, sum) weights
// (AttnParams says how). A persistent CTA runs its items back to back: the next item's Q tiles are fetched before the
// current one ends, barrier phases and ring stages simply continue, and the output rows leave through a staging area of
// their own.
// Warp numbers below are those of the two-tile form.
//
//   warp 8     TMA producer: both Q tiles once, then K and V tiles through two independent 2-stage
//              shared-memory rings (128-byte swizzle, plain per-CTA tiled loads; rows past the end read as zeros).
//   warp 9     MMA issuer (the warp runs the loop, one elected lane issues) and owner of the tensor-memory allocation (512 columns):
//                S_t (128 fp32 columns)  = Q_t . K_j^T     both operands from shared memory (K-major)
//                O_t (D fp32 columns)   += P_t . V_j       P_t from tensor memory, V_j MN-major from its row-major tile
//              issue order per key tile j:  P.V_A(j), Q.K_A(j+1), P.V_B(j), Q.K_B(j+1).
//   warps 0-3  softmax of tile A, warps 4-7 softmax of tile B; thread r owns row r of its tile. The row of S is
//              read from TMEM once into registers; P = exp2(S*scale*log2e - m) in fp32 is packed to the storage
//              type and written over the first 64 columns of S_t (tcgen05.st), which the P.V MMA reads as its A
//              operand. P_t is handed over in two column groups (keys 0-63, 64-127), each on its own mbarrier with
//              one arrival per warp, so the first four P.V MMA steps run while the second half is exponentiated.
//              The exponentials are the scarce resource (16 per clock per SM): the row is processed as a software
//              pipeline written in issue order, packed fp32 arithmetic (f32x2) around the MUFU ex2, and every fourth
//              column pair takes a cubic-polynomial 2^x on the FMA pipes instead. The running maximum is raised
//              only when it grows by more than 8 (factor 256), so O_t in TMEM is rescaled rarely; row sums stay in
//              fp32. After the last key tile of an item the same warps read O_t, divide by the row sum and store.
//   warps 8-11 form the control warpgroup (8 = TMA, 9 = MMA); it gives registers up (setmaxnreg) so that the two
//              softmax warpgroups hold a whole score row plus the packed probabilities without spilling.
// Ordering notes: tcgen05.commit covers every MMA issued before it, so "S_t(j) ready" also means P.V_t(j-1) has
// finished and O_t may be rescaled; Q.K_t(j+1) overwrites the columns P_t(j) lives in and is issued after
// P.V_t(j) by the same thread, which the tensor pipe executes in order.
// Masking: keys >= kv_len[b] (or >= Skv) and, for causal, keys > row + (Skv - Sq) get probability 0; key tiles
// entirely above a query tile's diagonal are skipped for that tile.
#include <type_traits>
#include "common.cuh"
#include <cstdlib>
#include "ptx.cuh"
#include "tensormap.cuh"

namespace {

    constexpr int BM = 128, BN = 128; // rows per query tile, keys per key tile
    // QT = query tiles per CTA: 2 (one CTA per SM, the two tiles' softmax and MMAs overlap inside the CTA) or, for
    // head size 64 where two CTAs fit an SM, 1 (the overlap happens between the two co-resident CTAs and the hardware
    // block scheduler balances single tiles over the SMs: 176 two-tile CTAs on 148 SMs take two rounds, 352 one-tile CTAs
    // on 296 slots a little over one).
    __host__ __device__ constexpr int threads_for(int qt) { return 128 + qt * 128; } // QT softmax warpgroups, then the control warpgroup
    constexpr float kRescaleThreshold = 8.0f;
    constexpr int   kPParts = 2; // P_t is handed to the MMA issuer in this many column groups (BN / kPParts keys each)

    using FanOut = VkcFanDev;
    __device__ __forceinline__ void fanout_signal(const FanOut &f, unsigned total) { vkc_fanout_signal(f, total); }

    struct AttnParams {
        void          *O;
        int64_t        os[3];
        int64_t        Sq, Skv, Hq, Hkv;
        float          scale_log2;
        int            causal;
        const int32_t *kv_len;
        int           *dev_err;
        // Work distribution. A unit is one group of QT query tiles of one (batch, head), unit u = (b * Hq + h) * nq + group; it
        // needs `steps` key tiles.
        // balanced == 0: one CTA per unit, grid (groups, Hq, B).
        // balanced == 1 (no per-sequence lengths): a one-dimensional grid of persistent CTAs over blocks of work of equal length,
        // `steps` key tiles each. Without a causal mask every unit needs the same number of key tiles and a block is a unit.
        // With one (pairing == 1, Sq = Skv) the groups of a head differ, and a block is the pair of groups (nq - 1 - k, k), the
        // long one first: their lengths add up to the same for every k (the launcher checks it). "Unit" below then reads
        // "block" for the distribution; an item still lies in ONE unit. CTA c first takes `rounds` whole units, c, c + grid, c + 2 grid, ... (at any
        // moment the CTAs work on neighbouring units, so the K and V tiles they stream are the same few heads' and stay in
        // L2). The units left over, fewer than the grid has CTAs, are each cut into as many equal pieces of `quota` key tiles as
        // there are CTAs for: they are laid out on a line, unit r at [r * ustride, r * ustride + steps) with ustride a multiple
        // of quota (so every cut falls on a piece boundary and the tail of a stride is padding), and CTA c takes the steps
        // [c * quota, (c + 1) * quota) of the line. The stretch of a CTA's range that lies in one unit is an item. An item that
        // covers its whole unit stores final rows; otherwise it leaves a partial per row — the normalised output in the storage
        // type and (running maximum, row sum) — in the CTA's slot 0 (the unit began in an earlier CTA's range) or slot 1 (it
        // began in this one), and the merge kernel joins the partials of each left-over unit.
        int     balanced, pairing, nq, steps, quota, rounds, ustride;
        int     total;   // length of the line of left-over units
        void   *part_o;  // [CTAs][2][QT * BM][D] storage type
        float  *part_ml; // [CTAs][2][QT * BM][2]
        // output fan-out (n_dest > 0): every output row goes to dest[0..n_dest) instead of O; when the grid's last block has
        // stored (of the merge kernel in the balanced form), flag[d] (a word in destination d's memory) receives this rank's
        // count of completed fan-outs
        FanOut fan;
    };

    // Key tiles the 128-row query tile that starts at row `first` needs when `len` keys are visible to the sequence.
    __host__ __device__ inline int tile_steps(int64_t Sq, int64_t Skv, int causal, int64_t first, int64_t len) {
        int64_t kend = len;
        if (first >= Sq) kend = 0; // tile entirely past the end of the query sequence
        if (causal && kend > 0) {
            int64_t last = first + BM - 1;
            if (last > Sq - 1) last = Sq - 1;
            const int64_t lim = last + (Skv - Sq) + 1;
            if (lim < kend) kend = lim;
            if (kend < 0) kend = 0;
        }
        return (int) ((kend + BN - 1) / BN);
    }
    // ... and the group of QT tiles number `qg` (its longest tile), all Skv keys visible
    template <int QT> __host__ __device__ inline int unit_steps(int64_t Sq, int64_t Skv, int causal, int qg) {
        int n = 0;
#pragma unroll
        for (int t = 0; t < QT; ++t) {
            const int nt = tile_steps(Sq, Skv, causal, (int64_t) qg * (QT * BM) + (int64_t) t * BM, Skv);
            n            = nt > n ? nt : n;
        }
        return n;
    }

    // One item of a CTA's work and what each of its query tiles has to do in it.
    template <int QT> struct Work {
        bool    valid, last; // last: the CTA has nothing to do after this item
        int     b, h, qg;    // the unit
        int     j0;       // first key tile of the item; tile counts below are relative to it
        int     slot;     // partial slot of this CTA (0 or 1), or -1: the item covers the whole unit and stores final rows
        int     adv;      // how far the item moves the CTA along the line
        int64_t m0, len;  // first query row of the unit, visible key length
        int     n_t[QT], n_max;
    };
    // Which CTA of which grid (the kernel passes blockIdx / gridDim.x; the host walks the same arithmetic for its plan report).
    struct CtaId {
        int x, y, z, nx;
    };
    // `pos`: the key-tile steps the CTA has behind it when the item starts.
    template <int QT> __host__ __device__ __forceinline__ Work<QT> work_at(const AttnParams &p, int pos, const CtaId c) {
        Work<QT> w;
        int      cnt;
        if (p.balanced) {
            int       blk, j, room, bstart;                  // block, step inside it, steps left of the CTA's claim, block start in the line
            const int lp0 = c.x * p.quota; // this CTA's stretch of the line of left-over blocks: [lp0, lp1)
            const int lp1 = lp0 + p.quota < p.total ? lp0 + p.quota : p.total;
            const bool whole = pos < p.rounds * p.steps; // a whole block of the round-robin part
            if (whole) {
                const int k = pos / p.steps;
                blk         = k * c.nx + c.x;
                j           = pos - k * p.steps;
                room        = p.steps - j;
                bstart      = 0;
            } else {
                const int lp = lp0 + (pos - p.rounds * p.steps);
                w.valid      = lp < lp1;
                if (!w.valid) return w;
                const int br = lp / p.ustride;
                j            = lp - br * p.ustride;
                w.valid      = j < p.steps; // (else: the padding behind the block's last piece)
                if (!w.valid) return w;
                room   = lp1 - lp;
                bstart = br * p.ustride;
                blk    = p.rounds * c.nx + br;
            }
            // the unit of the block that step j lies in: [uoff, uoff + nu)
            const int nb = p.pairing ? p.nq / 2 : p.nq; // blocks per (batch, head)
            const int bh = blk / nb, k2 = blk - bh * nb;
            int       nu = p.steps, uoff = 0;
            w.qg         = k2;
            if (p.pairing) {
                const int n_hi = unit_steps<QT>(p.Sq, p.Skv, 1, p.nq - 1 - k2);
                if (j < n_hi) w.qg = p.nq - 1 - k2, nu = n_hi;
                else uoff = n_hi, nu = p.steps - n_hi;
            }
            w.j0           = j - uoff;
            const int left = nu - w.j0;
            cnt            = left < room ? left : room;
            w.slot         = (w.j0 == 0 && cnt == nu) ? -1 : (whole || bstart + uoff >= lp0 ? 1 : 0);
            w.valid        = true;
            w.adv          = cnt;
            // what comes after this item: more of this block or another whole block, a piece of a left-over block, or nothing
            // (the item ends j + cnt steps into its block's stride: at the stride's end the next block begins, past `steps` lies
            // padding)
            const int np = pos + cnt - p.rounds * p.steps, nj = j + cnt;
            w.last       = !(np < 0 || (lp0 + np < lp1 && (np == 0 || nj == p.ustride || nj < p.steps)));
            w.h          = bh % (int) p.Hq;
            w.b          = bh / (int) p.Hq;
        } else {
            w.valid = pos < 1;
            if (!w.valid) return w;
            w.b = c.z, w.h = c.y;
            w.qg   = p.causal ? c.nx - 1 - c.x : c.x; // heavy (late) query tiles first when causal
            w.j0   = 0;
            cnt    = INT32_MAX;
            w.slot = -1;
            w.adv  = 1;
            w.last = true;
        }
        w.m0  = (int64_t) w.qg * (QT * BM);
        w.len = p.Skv;
#ifdef __CUDA_ARCH__
        if (p.kv_len) w.len = (int64_t) p.kv_len[w.b];
#endif
        if (w.len > p.Skv) w.len = p.Skv;
        if (w.len < 0) w.len = 0;
        w.n_max = 0;
#pragma unroll
        for (int t = 0; t < QT; ++t) {
            int n    = tile_steps(p.Sq, p.Skv, p.causal, w.m0 + (int64_t) t * BM, w.len) - w.j0; // key tiles the query tile needs, from the item's first on
            n        = n < 0 ? 0 : (n > cnt ? cnt : n);
            w.n_t[t] = n;
            w.n_max  = n > w.n_max ? n : w.n_max;
        }
        return w;
    }

    template <int D, int KS, int VS, int QT> struct Smem {
        static constexpr uint32_t Q_BYTES  = BM * D * 2; // per query tile
        static constexpr uint32_t KV_BYTES = BN * D * 2;
        static constexpr uint32_t oQ   = 0;
        static constexpr uint32_t oK   = oQ + QT * Q_BYTES;
        static constexpr uint32_t oV   = oK + KS * KV_BYTES;
        static constexpr uint32_t oStage = oV + VS * KV_BYTES; // output staging: 32 rows x 128 bytes per softmax warp
        static constexpr uint32_t oBar = oStage + QT * 4 * 4096;
        // barriers: q_full, q_read, k_full[KS], k_empty[KS], v_full[VS], v_empty[VS], s_full[QT], p_full[QT][kPParts], o_final[QT]
        static constexpr int nBar = 2 + 2 * KS + 2 * VS + QT * (2 + kPParts);
        static constexpr uint32_t oCtl  = oBar + 8 * nBar;
        static constexpr uint32_t total = oCtl + 16 + 1024;
    };

    __device__ __forceinline__ float fast_exp2(float x) {
        float y;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
        return y;
    }
    // Polynomial 2^x (its steps are written inline in the softmax loop): every fourth column pair is exponentiated on
    // the fp32 pipes, so that the exponentials of a score tile are shared between the special-function unit and the FMA pipes: x = n + f with n = round(x) taken by the magic-number addition
    // (1.5 * 2^23) and f in [-0.5, 0.5]; 2^f by a cubic with relative error < 7.5e-5 (below half an ulp of either
    // 16-bit storage type); n is added into the exponent field. Inputs are clamped at -125, so a masked score
    // (-inf) yields 2^-125 rather than 0: invisible next to any visible key, and rows with no visible key are
    // detected by their running maximum instead of by a zero sum.
    template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
    template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }

    // Order-pinned (volatile) forms of the softmax arithmetic, operating on 32-bit registers in place.
    __device__ __forceinline__ void v_ex2(uint32_t &x) { asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+r"(x)); }
    __device__ __forceinline__ void v_max(uint32_t &x, float lo) { asm volatile("max.f32 %0, %0, %1;" : "+r"(x) : "f"(lo)); }
    // {dx,dy} = {ax,ay} * b + c
    __device__ __forceinline__ void v_ffma2(uint32_t &dx, uint32_t &dy, uint32_t ax, uint32_t ay, float2 b, float2 c) {
        asm volatile("{.reg .b64 a, d; mov.b64 a, {%2, %3}; fma.rn.f32x2 d, a, %4, %5; mov.b64 {%0, %1}, d;}"
                     : "=r"(dx), "=r"(dy)
                     : "r"(ax), "r"(ay), "l"(reinterpret_cast<const unsigned long long &>(b)), "l"(reinterpret_cast<const unsigned long long &>(c)));
    }
    // {dx,dy} = a * {bx,by} + c
    __device__ __forceinline__ void v_ffma2to(uint32_t &dx, uint32_t &dy, float2 a, uint32_t bx, uint32_t by, float2 c) {
        asm volatile("{.reg .b64 b, d; mov.b64 b, {%2, %3}; fma.rn.f32x2 d, %4, b, %5; mov.b64 {%0, %1}, d;}"
                     : "=r"(dx), "=r"(dy)
                     : "r"(bx), "r"(by), "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(c)));
    }
    // {px,py} = {px,py} * {fx,fy} + c
    __device__ __forceinline__ void v_ffma2acc(uint32_t &px, uint32_t &py, uint32_t fx, uint32_t fy, float2 c) {
        asm volatile("{.reg .b64 p, f; mov.b64 p, {%0, %1}; mov.b64 f, {%2, %3}; fma.rn.f32x2 p, p, f, %4; mov.b64 {%0, %1}, p;}"
                     : "+r"(px), "+r"(py)
                     : "r"(fx), "r"(fy), "l"(reinterpret_cast<const unsigned long long &>(c)));
    }
    // {dx,dy} = {ax,ay} + b
    __device__ __forceinline__ void v_fadd2to(uint32_t &dx, uint32_t &dy, uint32_t ax, uint32_t ay, float2 b) {
        asm volatile("{.reg .b64 a, d; mov.b64 a, {%2, %3}; add.rn.f32x2 d, a, %4; mov.b64 {%0, %1}, d;}"
                     : "=r"(dx), "=r"(dy)
                     : "r"(ax), "r"(ay), "l"(reinterpret_cast<const unsigned long long &>(b)));
    }
    // acc += {ax,ay}
    __device__ __forceinline__ void v_fadd2(float2 &acc, uint32_t ax, uint32_t ay) {
        asm volatile("{.reg .b64 a; mov.b64 a, {%1, %2}; add.rn.f32x2 %0, %0, a;}"
                     : "+l"(reinterpret_cast<unsigned long long &>(acc))
                     : "r"(ax), "r"(ay));
    }
    // d = bits(p) + (bits(t) << 23): the integer part held in the low bits of t goes into the exponent of p
    __device__ __forceinline__ void v_expo(uint32_t &d, uint32_t p, uint32_t t) {
        asm volatile("{.reg .b32 e; shl.b32 e, %2, 23; add.u32 %0, %1, e;}" : "=r"(d) : "r"(p), "r"(t));
    }
    template <typename T> __device__ __forceinline__ uint32_t v_pack2(uint32_t lo, uint32_t hi);
    template <> __device__ __forceinline__ uint32_t v_pack2<__half>(uint32_t lo, uint32_t hi) {
        uint32_t d;
        asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
        return d;
    }
    template <> __device__ __forceinline__ uint32_t v_pack2<__nv_bfloat16>(uint32_t lo, uint32_t hi) {
        uint32_t d;
        asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(hi)), "f"(__uint_as_float(lo)));
        return d;
    }

    template <typename T, int D, int kMode, int QT>
    __global__ void __launch_bounds__(threads_for(QT), QT == 1 ? 2 : 1)
        attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                            AttnParams p) {
        constexpr int KS = 2, VS = 2; // the MMA issuer selects ring stages by the parity of the key tile
        static_assert(KS == 2 && VS == 2, "stage selection assumes two-stage rings");
        using L               = Smem<D, KS, VS, QT>;
        constexpr int kQTiles = QT, kThreads = threads_for(QT);
        constexpr int kWarpTma = 4 * QT, kWarpMma = 4 * QT + 1; // the other two warps of the control warpgroup only give up registers
        constexpr int kTmemCols = QT == 2 ? 512 : 256;
        // Register re-partitioning. The CTA is launched with kRegsBase registers per thread (what the launch bounds allow);
        // setmaxnreg.inc blocks in hardware until the CTA's own pool holds the registers, so the control warpgroup must
        // give up at least what the softmax warpgroups take (checked here: a shortfall would hang the kernel).
        constexpr int kRegsBase    = (65536 / (threads_for(QT) * (QT == 1 ? 2 : 1))) / 8 * 8;
        constexpr int kRegsControl = QT == 2 ? 88 : 56;
        constexpr int kRegsSoftmax = QT == 2 ? 208 : 200;
        static_assert(QT * (kRegsSoftmax - kRegsBase) <= kRegsBase - kRegsControl, "softmax warpgroups would wait forever for registers");
        (void) kThreads;
        constexpr bool kBf16  = std::is_same<T, __nv_bfloat16>::value;
        constexpr uint32_t kIdescQK = ptx::idesc_f16(BM, BN, kBf16, false, false);
        constexpr uint32_t kIdescPV = ptx::idesc_f16(BM, D, kBf16, false, true);
        constexpr int      DCH      = D / 64; // 64-element (128-byte) spans per row
        constexpr int      kColS    = 0;      // S_A at 0, S_B at 128; P_t aliases the first 64 columns of S_t
        constexpr int      kColO    = QT * 128; // O_A behind the S tiles, O_B at + D

        extern __shared__ uint8_t smem_raw[];
        const uint32_t raw   = ptx::smem_u32(smem_raw);
        const uint32_t base  = (raw + 1023u) & ~1023u;
        uint8_t       *gbase = smem_raw + (base - raw);
        const uint32_t sQ = base + L::oQ, sK = base + L::oK, sV = base + L::oV, sBar = base + L::oBar;
        volatile int  *ctl = (volatile int *) (gbase + L::oCtl); // ctl[0] = tmem base, ctl[1] = abort flag
        auto           bar = [&](int i) { return sBar + 8u * (uint32_t) i; };
        constexpr int  bQ = 0, bQE = 1, bKF = 2, bKE = bKF + KS, bVF = bKE + KS, bVE = bVF + VS, bSF = bVE + VS, bPF = bSF + QT,
                      bOF = bPF + QT * kPParts;

        const int   warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const CtaId cta {(int) blockIdx.x, (int) blockIdx.y, (int) blockIdx.z, (int) gridDim.x};

        if (threadIdx.x == (kWarpMma + 1) * 32) { // a thread of an idle warp, so that the set-up runs beside the look-up above
            for (int i = 0; i < L::nBar; ++i) ptx::mbar_init(bar(i), (i >= bPF && i < bOF) ? 4 : 1); // p_full: one arrival per softmax warp of the tile
            ctl[1] = 0;
            ptx::fence_mbar_init();
            ptx::prefetch_tmap(&tmQ);
            ptx::prefetch_tmap(&tmK);
            ptx::prefetch_tmap(&tmV);
        }
        if (warp == kWarpMma) {
            ptx::tmem_alloc(base + L::oCtl, kTmemCols);
            ptx::tmem_relinquish();
        }
        const Work<QT> w_first = work_at<QT>(p, 0, cta); // the first item, looked up while the barriers are being set up
        // the item after `cur` (which began at step `pos` minus its length); none behind the CTA's last
        auto next_work = [&](const Work<QT> &cur, int pos) {
            if (!cur.last) return work_at<QT>(p, pos, cta);
            Work<QT> none;
            none.valid = false;
            return none;
        };
        ptx::tc_fence_before();
        __syncthreads();
        ptx::tc_fence_after();
        const uint32_t tmem = (uint32_t) ctl[0];
        vkc_grid_dep_wait(); // set-up above overlaps the previous kernel's tail; global memory from here on
        vkc_grid_dep_launch();

        if (warp >= kWarpTma) {
          ptx::setmaxnreg_dec<kRegsControl>();
          if (warp == kWarpTma) {
            // ------------------------------------------------------------------ TMA producer
            // Key tiles are numbered g = 0, 1, ... over all items of the CTA; ring stage g & 1, phase g >> 1. The Q tiles of the
            // next item are loaded as soon as every Q.K^T MMA of the current one has read them (q_read) — normally a whole key
            // tile before the current item ends.
            if (ptx::elect_one()) {
                int  cq = 0; // Q loads issued
                int  g  = 0;
                bool ok = true;
                const int hq_per_kv = (int) (p.Hq / p.Hkv);
                Work<QT>  w = w_first;
                for (int pos = 0; ok; w = next_work(w, pos)) {
                    if (!w.valid) break;
                    pos += w.adv;
                    const int hk = w.h / hq_per_kv;
                    for (int j = 0; j < w.n_max; ++j, ++g) {
                        const int      st = g & 1;
                        const uint32_t ph = (uint32_t) ((g >> 1) & 1);
                        if (!(ok = ptx::mbar_wait(bar(bKE + st), ph ^ 1, ctl + 1, p.dev_err))) break;
                        ptx::mbar_expect_tx(bar(bKF + st), L::KV_BYTES);
#pragma unroll
                        for (int c = 0; c < DCH; ++c) ptx::tma_load_4d(sK + st * L::KV_BYTES + c * (BN * 128), &tmK, c * 64, (w.j0 + j) * BN, hk, w.b, bar(bKF + st));
                        if (j == 0) {
                            if (cq > 0) {
                                const uint32_t pq = (uint32_t) ((cq - 1) & 1);
                                if (!(ok = ptx::mbar_wait(bar(bQE), pq, ctl + 1, p.dev_err))) break;
                            }
                            ptx::mbar_expect_tx(bar(bQ), kQTiles * L::Q_BYTES);
#pragma unroll
                            for (int t = 0; t < kQTiles; ++t)
#pragma unroll
                                for (int c = 0; c < DCH; ++c)
                                    ptx::tma_load_4d(sQ + t * L::Q_BYTES + c * (BM * 128), &tmQ, c * 64, (int) (w.m0 + t * BM), w.h, w.b, bar(bQ));
                            ++cq;
                        }
                        if (!(ok = ptx::mbar_wait(bar(bVE + st), ph ^ 1, ctl + 1, p.dev_err))) break;
                        ptx::mbar_expect_tx(bar(bVF + st), L::KV_BYTES);
#pragma unroll
                        for (int c = 0; c < DCH; ++c) ptx::tma_load_4d(sV + st * L::KV_BYTES + c * (BN * 128), &tmV, c * 64, (w.j0 + j) * BN, hk, w.b, bar(bVF + st));
                    }
                }
            }
          } else if (warp == kWarpMma) {
            // ------------------------------------------------------------------ MMA issuer
            // The whole warp runs the loop (waits, descriptor arithmetic) convergently and one elected lane issues the
            // tcgen05 instructions. One issuer serves both query tiles in strict alternation: that alternation is what
            // keeps the two tiles half a period apart, so that one tile's exponentials run under the other's MMAs
            // (an issuer per tile lets the tiles fall into step and share the exponential unit: 949 vs 1265 TFLOP/s).
            const bool leader = ptx::elect_one();
            {
                // Base descriptors once; a step along K only moves the 14-bit start-address field (16-byte units).
                const uint64_t dQ0 = ptx::smem_desc_sw128(sQ, 16, 1024), dQ1 = ptx::smem_desc_sw128(sQ + L::Q_BYTES, 16, 1024);
                const uint64_t dK0 = ptx::smem_desc_sw128(sK, 16, 1024), dK1 = ptx::smem_desc_sw128(sK + L::KV_BYTES, 16, 1024);
                const uint64_t dV0 = ptx::smem_desc_sw128(sV, BN * 128, 1024), dV1 = ptx::smem_desc_sw128(sV + L::KV_BYTES, BN * 128, 1024);
                auto wait = [&](int barIdx, uint32_t parity) { return __all_sync(0xffffffffu, ptx::mbar_wait(bar(barIdx), parity, ctl + 1, p.dev_err)); };
                auto issue_qk = [&](int t, int g) { // g: the key tile's number in the CTA (selects the ring stage)
                    const uint64_t aq = t ? dQ1 : dQ0, bk = (g & 1) ? dK1 : dK0;
                    const uint32_t d  = tmem + kColS + t * BN;
#pragma unroll
                    for (int k = 0; k < D / 16; ++k) {
                        const uint32_t off = ((uint32_t) (k / 4) * (BM * 128) + (uint32_t) (k % 4) * 32) >> 4;
                        if (leader) ptx::mma_f16_ss(d, aq + off, bk + off, kIdescQK, k != 0 ? 1u : 0u);
                    }
                    if (leader) ptx::tc_commit(bar(bSF + t));
                };
                auto issue_pv = [&](int t, int j, int g, int part) { // j: key tile within the item (0 starts a new O_t)
                    // V tile: D/64 spans of [128 keys x 128 B]; 16 keys per MMA step = 2048 B; `part` selects BN / kPParts keys
                    const uint64_t bv = (g & 1) ? dV1 : dV0;
                    const uint32_t d = tmem + kColO + t * D, a = tmem + kColS + t * BN;
#pragma unroll
                    for (int k = part * (8 / kPParts); k < (part + 1) * (8 / kPParts); ++k)
                        if (leader) ptx::mma_f16_ts(d, a + k * 8, bv + (uint64_t) (k * 128), kIdescPV, (j | k) != 0 ? 1u : 0u);
                };
                int  cq = 0;      // items with work so far (phase of the Q barriers)
                int  cs[kQTiles]; // key tiles each query tile has been through (phase of its S and P barriers)
                int  g0 = 0;      // key tiles before this item
                bool ok = true;
#pragma unroll
                for (int t = 0; t < kQTiles; ++t) cs[t] = 0;
                Work<QT> w = w_first;
                for (int pos = 0; ok; w = next_work(w, pos)) {
                    if (!w.valid) break;
                    pos += w.adv;
                    if (w.n_max == 0) continue;
                    const int n_max = w.n_max;
                    ok = wait(bKF + (g0 & 1), (uint32_t) ((g0 >> 1) & 1)) && wait(bQ, (uint32_t) (cq & 1));
                    if (!ok) break;
                    ptx::tc_fence_after();
                    // O_t and S_t of the previous item are free: its P.V MMAs were issued before these, and the softmax warps
                    // have read O_t before they can hand over the first P_t of this item.
#pragma unroll
                    for (int t = 0; t < kQTiles; ++t)
                        if (w.n_t[t] > 0) issue_qk(t, g0);
                    if (leader) {
                        ptx::tc_commit(bar(bKE + (g0 & 1)));
                        if (n_max == 1) ptx::tc_commit(bar(bQE));
                    }
                    for (int j = 0; j < n_max && ok; ++j) {
                        const int g = g0 + j, vs = g & 1;
                        ok = wait(bVF + vs, (uint32_t) ((g >> 1) & 1));
                        const bool more = j + 1 < n_max;
#pragma unroll
                        for (int t = 0; t < kQTiles && ok; ++t) {
                            if (j < w.n_t[t]) {
                                const uint32_t pp = (uint32_t) (cs[t] & 1);
                                ok = wait(bPF + kPParts * t, pp);
                                if (!ok) break;
                                ptx::tc_fence_after();
                                issue_pv(t, j, g, 0);
#pragma unroll
                                for (int part = 1; part < kPParts && ok; ++part) {
                                    ok = wait(bPF + kPParts * t + part, pp);
                                    if (ok) {
                                        ptx::tc_fence_after();
                                        issue_pv(t, j, g, part);
                                    }
                                }
                                if (!ok) break;
                                ++cs[t];
                                if (j + 1 < w.n_t[t]) {
                                    ok = wait(bKF + ((g + 1) & 1), (uint32_t) (((g + 1) >> 1) & 1));
                                    if (!ok) break;
                                    ptx::tc_fence_after();
                                    issue_qk(t, g + 1);
                                } else if (leader) {
                                    ptx::tc_commit(bar(bOF + t)); // O_t complete
                                }
                            }
                        }
                        if (!ok) break;
                        if (leader) {
                            ptx::tc_commit(bar(bVE + vs));
                            if (more) {
                                ptx::tc_commit(bar(bKE + ((g + 1) & 1)));
                                if (j + 2 == n_max) ptx::tc_commit(bar(bQE)); // the item's last Q.K^T MMAs are issued: Q may be replaced
                            }
                        }
                    }
                    g0 += n_max;
                    ++cq;
                }
            }
          }
        } else {
            ptx::setmaxnreg_inc<kRegsSoftmax>();
            // ------------------------------------------------------------------ softmax + epilogue (thread = row)
            const int      t      = warp >> 2;             // query tile of this warpgroup
            const int      q      = warp & 3;              // TMEM lane quarter this warp may address
            const int      r      = q * 32 + lane;
            const uint32_t tS     = tmem + ((uint32_t) (q * 32) << 16) + kColS + t * BN;
            const uint32_t tO     = tmem + ((uint32_t) (q * 32) << 16) + kColO + t * D;
            int            cs = 0, co = 0; // key tiles / items with work this query tile has been through (barrier phases)
            bool           ok = true;
            // What the key-tile loop needs of an item is boiled down to four numbers, so that the item's description does not
            // occupy registers next to a whole row of scores; the epilogue looks the item up again.
            int  n = 0, kbase = 0, jm = 0, lim_row = 0;
            int  iadv = 0, ib = 0, ih = 0, imisc = 0; // the item's length along the line and what the epilogue needs: batch, head, and group | (slot + 1) << 26 | last << 28 | (n_max > 0) << 29
            bool have = false;
            auto prepare = [&](const Work<QT> &w) {
                have = w.valid;
                if (!have) return;
                iadv = w.adv, ib = w.b, ih = w.h, imisc = w.qg | ((w.slot + 1) << 26) | (w.last ? 1 << 28 : 0) | (w.n_max > 0 ? 1 << 29 : 0);
                n     = t ? w.n_t[QT - 1] : w.n_t[0]; // (a run-time index would put the whole description into local memory)
                kbase = w.j0 * BN; // first key of the item
                const int64_t first = w.m0 + (int64_t) t * BM, off = p.Skv - p.Sq;
                // keys < lim_row are visible to this thread's row
                int64_t lim = w.len;
                if (p.causal && first + r + off + 1 < lim) lim = first + r + off + 1;
                lim_row = lim < 0 ? 0 : (int) lim;
                // key tiles from jm on (counted within the item) straddle kv_len or the causal diagonal and take the masked body
                jm = (int) (w.len / BN) - w.j0;
                if (p.causal) {
                    const int64_t f1 = first + off + 1 < 0 ? 0 : first + off + 1;
                    const int     j2 = (int) (f1 / BN) - w.j0;
                    jm = j2 < jm ? j2 : jm;
                }
            };
            prepare(w_first);
          for (int pos = 0; ok && have;) {
            float          m_used = -INFINITY, l = 0.f;
            // One key tile; kMask selects the body that replaces invisible scores by -inf (only the tiles that
            // straddle kv_len or the causal diagonal take it, every other tile runs free of any mask arithmetic).
            auto tile = [&](auto mask_tag, int j) -> bool {
                constexpr bool kMask = decltype(mask_tag)::value;
                ok = ptx::mbar_wait(bar(bSF + t), (uint32_t) (cs & 1), ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) return false;
                ++cs;
                ptx::tc_fence_after();
                uint32_t s[4][32];
#pragma unroll
                for (int c = 0; c < 4; ++c) ptx::tmem_ld_x32(tS + c * 32, s[c]);
                ptx::tc_wait_ld();
                if (kMask) {
                    // visible columns of this row in this tile: [0, nvis)
                    const int lim  = lim_row - (kbase + j * BN);
                    const int nvis = lim < 0 ? 0 : (lim > BN ? BN : lim);
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (c * 32 + i >= nvis) s[c][i] = 0xff800000u; // -inf
                }
                // row maximum: 16 independent chains over 8 columns each (3-input max), then a short tree
                float mx[16];
#pragma unroll
                for (int k = 0; k < 16; ++k)
                    mx[k] = ptx::fmax3(__uint_as_float(s[k >> 2][(k & 3) * 8]), __uint_as_float(s[k >> 2][(k & 3) * 8 + 1]),
                                       __uint_as_float(s[k >> 2][(k & 3) * 8 + 2]));
#pragma unroll
                for (int u = 3; u < 7; u += 2)
#pragma unroll
                    for (int k = 0; k < 16; ++k)
                        mx[k] = ptx::fmax3(mx[k], __uint_as_float(s[k >> 2][(k & 3) * 8 + u]), __uint_as_float(s[k >> 2][(k & 3) * 8 + u + 1]));
#pragma unroll
                for (int k = 0; k < 8; ++k) mx[k] = ptx::fmax3(mx[k], mx[k + 8], __uint_as_float(s[k >> 1][(k & 1) * 16 + 7]));
#pragma unroll
                for (int k = 0; k < 8; ++k) mx[k] = fmaxf(mx[k], __uint_as_float(s[k >> 1][(k & 1) * 16 + 15]));
                mx[0] = ptx::fmax3(mx[0], mx[1], mx[2]);
                mx[3] = ptx::fmax3(mx[3], mx[4], mx[5]);
                mx[6] = fmaxf(mx[6], mx[7]);
                const float mxs = ptx::fmax3(mx[0], mx[3], mx[6]) * p.scale_log2; // scale > 0
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
                const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(neg_m, neg_m);
                float2       ls  = make_float2(0.f, 0.f);
                // P for column group `part` of this row is in TMEM: one arrival per warp on that group's barrier
                auto p_ready = [&](int part) {
                    ptx::tc_wait_st();
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar(bPF + kPParts * t + part));
                };
                if (kMode == 0) {
#pragma unroll
                    for (int c = 0; c < 4; c += 2) {
                        uint32_t pk[32];
#pragma unroll
                        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                const float2 x = ptx::ffma2(make_float2(__uint_as_float(s[c + cc][i]), __uint_as_float(s[c + cc][i + 1])), sc2, nm2);
                                const float2 e = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                                ls             = ptx::fadd2(ls, e);
                                pk[cc * 16 + i / 2] = pack2<T>(e.x, e.y);
                            }
                        ptx::tmem_st_x32(tS + (c / 2) * 32, pk);
#pragma unroll
                        for (int part = (c / 2) * (kPParts / 2); part < (c / 2 + 1) * (kPParts / 2); ++part)
                            if (part != kPParts - 1) p_ready(part);
                    }
                } else {
                    // The 64 column pairs of the row as a three-stage software pipeline written out in issue order, so
                    // that the two exponentials of a pair (special-function unit, 8 cycles per warp instruction) always
                    // sit between fp32-pipe instructions of other pairs: stage 0 scales (x = s*scale*log2e - m), stage 1
                    // exponentiates in place, stage 2 adds to the row sum and packs to 16 bits. In mode 2 every fourth
                    // pair takes the polynomial 2^x, whose steps are spread between the exponentials of the other three.
                    constexpr int kPairs = 64 / kPParts; // column pairs per hand-off group
                    uint32_t      pk[32];
                    auto     X  = [&](int g) -> uint32_t & { return s[g >> 4][(g & 15) * 2]; };
                    auto     Y  = [&](int g) -> uint32_t & { return s[g >> 4][(g & 15) * 2 + 1]; };
                    auto     S0 = [&](int g) {
                        if (g < 64) v_ffma2(X(g), Y(g), X(g), Y(g), sc2, nm2);
                    };
                    auto S2 = [&](int g) {
                        if (g >= 0) {
                            v_fadd2(ls, X(g), Y(g));
                            pk[g & 31] = v_pack2<T>(X(g), Y(g));
                            if (kPairs == 16 && (g & 15) == 15) {
                                if (g & 16) ptx::tmem_st_x16(tS + (g >> 4) * 16, *reinterpret_cast<uint32_t(*)[16]>(pk + 16));
                                else ptx::tmem_st_x16(tS + (g >> 4) * 16, *reinterpret_cast<uint32_t(*)[16]>(pk));
                            }
                            if (kPairs == 32 && (g & 31) == 31) ptx::tmem_st_x32(tS + (g >> 5) * 32, pk);
                            // signal a group a few pairs after its store was issued
                            if (g >= kPairs && g < 64 && (g % kPairs) == 3) p_ready(g / kPairs - 1);
                        }
                    };
                    const float2 kMagic = make_float2(12582912.0f, 12582912.0f), kNegMagic = make_float2(-12582912.0f, -12582912.0f);
                    const float2 kNegOne = make_float2(-1.f, -1.f);
                    const float2 kC3 = make_float2(5.517164618e-02f, 5.517164618e-02f), kC2 = make_float2(2.426111251e-01f, 2.426111251e-01f);
                    const float2 kC1 = make_float2(6.932609677e-01f, 6.932609677e-01f), kC0 = make_float2(9.999280572e-01f, 9.999280572e-01f);
                    uint32_t     tx, ty, nx, ny, px, py; // the polynomial pair in flight
                    S0(0), S0(1), S0(2), S0(3);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int m0 = 4 * i, m1 = m0 + 1, m2 = m0 + 2, q = m0 + 3;
                        v_ex2(X(m0));
                        S0(m0 + 4);
                        if (kMode == 2) v_max(X(q), -125.0f), v_max(Y(q), -125.0f);
                        v_ex2(Y(m0));
                        if (kMode == 2) {
                            v_fadd2to(tx, ty, X(q), Y(q), kMagic);
                            v_fadd2to(nx, ny, tx, ty, kNegMagic);
                        }
                        S2(m0 - 4);
                        v_ex2(X(m1));
                        S0(m1 + 4);
                        if (kMode == 2) {
                            v_ffma2(nx, ny, nx, ny, kNegOne, make_float2(__uint_as_float(X(q)), __uint_as_float(Y(q)))); // f = x - n
                            v_ffma2to(px, py, kC3, nx, ny, kC2);
                        }
                        v_ex2(Y(m1));
                        if (kMode == 2) v_ffma2acc(px, py, nx, ny, kC1);
                        S2(m1 - 4);
                        v_ex2(X(m2));
                        S0(m2 + 4);
                        if (kMode == 2) {
                            v_ffma2acc(px, py, nx, ny, kC0);
                            v_expo(X(q), px, tx);
                        } else {
                            v_ex2(X(q));
                        }
                        v_ex2(Y(m2));
                        S0(q + 4);
                        if (kMode == 2) {
                            v_expo(Y(q), py, ty);
                        } else {
                            v_ex2(Y(q));
                        }
                        S2(m2 - 4);
                        S2(q - 4);
                    }
                    S2(60), S2(61), S2(62), S2(63);
                }
                l += ls.x + ls.y;
                p_ready(kPParts - 1);
                return true;
            };
            for (int j = 0; j < n; ++j) {
                if (!(j >= jm ? tile(std::true_type{}, j) : tile(std::false_type{}, j))) break;
            }
            if (!ok) break;
            struct { int slot; bool last; int n_max; } w; // (n_max: only whether the item had work)
            w.slot = ((imisc >> 26) & 3) - 1, w.last = (imisc >> 28) & 1, w.n_max = (imisc >> 29) & 1;
            pos += iadv;
            const int      b = ib, h = ih;
            const int64_t  m0 = (int64_t) (imisc & ((1 << 26) - 1)) * (QT * BM), row = m0 + (int64_t) t * BM + r;
            const int      ndest  = w.slot >= 0 ? 0 : p.fan.n_dest; // fan-out of final rows only (the launcher checked alignment)
            // epilogue of the item
            if (n > 0) {
                ok = ptx::mbar_wait(bar(bOF + t), (uint32_t) (co & 1), ctl + 1, p.dev_err);
                ok = __all_sync(0xffffffffu, ok);
                ++co;
            }
            if (!ok) break;
            {
                ptx::tc_fence_after();
                // a row with no visible key stores NaN like the reference's 0/0
                float       inv    = (n > 0 && m_used == -INFINITY) ? __int_as_float(0x7fc00000) : 1.0f / l;
                const int64_t ooff  = (int64_t) b * p.os[0] + (int64_t) h * p.os[1] + row * p.os[2];
                T          *orow   = (T *) p.O + ooff;
                bool        vec_ok = (p.os[0] % 8 == 0) && (p.os[1] % 8 == 0) && (p.os[2] % 8 == 0) && (((uintptr_t) p.O & 15) == 0);
                const bool  partial = w.slot >= 0;
                // rows of a partial: [CTA][slot][QT * BM]
                const int64_t prow0 = ((int64_t) blockIdx.x * 2 + (partial ? w.slot : 0)) * (kQTiles * BM) + (int64_t) t * BM;
                if (partial) {
                    // partial of this stretch of the keys: O / l in the storage type (bounded by max |v|, so 16 bits do not
                    // overflow), weight data (m, l) in fp32; a stretch without a visible key for this row has weight 0
                    const bool none = n == 0 || m_used == -INFINITY;
                    inv    = none ? 0.f : 1.0f / l;
                    orow   = (T *) p.part_o + (prow0 + r) * D;
                    vec_ok = true;
                    if (row < p.Sq) {
                        p.part_ml[(prow0 + r) * 2]     = none ? -INFINITY : m_used;
                        p.part_ml[(prow0 + r) * 2 + 1] = none ? 0.f : l;
                    }
                }
                if (vec_ok) {
                    // Coalesced stores. Thread = row would write 16 bytes per row and instruction: 32 scattered segments per warp
                    // store (partly filled sectors in local memory, and each its own NVLink packet when the destination is a
                    // peer). The warp therefore stages 64 columns of its 32 rows (128 bytes per row) in its own 4 KB of shared
                    // memory, in 16-byte chunks XOR-swizzled by the row, and then writes whole 128-byte lines: 4 rows per
                    // instruction.
                    const uint32_t sStage = base + L::oStage + (uint32_t) (t * 4 + q) * 4096;
                    // partial rows are dense [.., QT * BM, D]; final rows follow the caller's output strides
                    const int64_t row_stride = partial ? (int64_t) D : p.os[2];
                    const int64_t base_off   = partial ? (prow0 - (m0 + (int64_t) t * BM)) * D : (int64_t) b * p.os[0] + (int64_t) h * p.os[1];
                    T *const      obase      = partial ? (T *) p.part_o : (T *) p.O;
#pragma unroll 1
                    for (int c = 0; c < D / 64; ++c) {
                        uint32_t v[64];
                        if (n > 0) {
                            ptx::tmem_ld_x32(tO + c * 64, *reinterpret_cast<uint32_t(*)[32]>(v));
                            ptx::tmem_ld_x32(tO + c * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(v + 32));
                            ptx::tc_wait_ld();
                        } else {
#pragma unroll
                            for (int i = 0; i < 64; ++i) v[i] = 0u;
                        }
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            uint32_t o32[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                o32[i] = pack2<T>(__uint_as_float(v[g * 8 + 2 * i]) * inv, __uint_as_float(v[g * 8 + 2 * i + 1]) * inv);
                            ptx::st_shared_v4(sStage + (uint32_t) lane * 128 + (uint32_t) ((g ^ (lane & 7)) << 4), o32[0], o32[1], o32[2], o32[3]);
                        }
                        __syncwarp();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int     rr   = i * 4 + (lane >> 3), ch = lane & 7;
                            const int64_t grow = m0 + (int64_t) t * BM + q * 32 + rr;
                            const uint4   o4   = ptx::ld_shared_v4(sStage + (uint32_t) rr * 128 + (uint32_t) ((ch ^ (rr & 7)) << 4));
                            if (grow < p.Sq) {
                                const int64_t off = base_off + grow * row_stride + c * 64 + ch * 8;
                                if (ndest == 0) *reinterpret_cast<uint4 *>(obase + off) = o4;
                                else vkc_fanout_store16<T>(p.fan, off, o4);
                            }
                        }
                        __syncwarp(); // the staging lines are rewritten by the next 64 columns
                    }
                } else {
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
#pragma unroll
                            for (int i = 0; i < 32; ++i) St<T>::st(orow + c * 32 + i, __uint_as_float(v[i]) * inv);
                        }
                    }
                }
                // O_t has been read: order those reads before the P_t hand-over of the next item, after which the tensor
                // pipe starts a new O_t
                ptx::tc_fence_before();
            }
            if (w.last) break;
            prepare(work_at<QT>(p, pos, cta));
          }
        }
        if (ctl[1]) {
            for (int i = 0; i < 50; ++i) __nanosleep(20000); // aborted: let copies in flight land
        }
        ptx::tc_fence_before();
        __syncthreads();
        if (warp == kWarpMma) ptx::tmem_dealloc(tmem, kTmemCols);
        if (!p.balanced && p.fan.n_dest > 0) fanout_signal(p.fan, gridDim.x * gridDim.y * gridDim.z);
    }

    // Merge kernel of the balanced form: one thread per 16 bytes of an output row of the units in the left-over blocks
    // (`main_ctas` = grid size of the attention kernel, `left` = number of left-over blocks). A unit that one CTA covered alone
    // already has its final rows. The others were cut at CTA boundaries: CTA c of the run [first, last] holds the unit's
    // partial in its slot 0, except the first if the unit began inside that CTA's range (slot 1). Each row gets the weights
    // l_s * 2^(m_s - m) over their sum (m_s are in the log2 domain the kernel works in); a row without any visible key gets NaN
    // like the reference's 0/0.
    template <typename T, int D, int QT>
    __global__ void __launch_bounds__(256) attn_prefill_merge_kernel(const AttnParams p, int main_ctas, int left) {
        constexpr int TPRW = D / 8, ROWS = QT * BM; // threads per row (8 elements each), rows per unit
        const int     upb  = p.pairing ? 2 : 1;     // units per block
        const int64_t gid  = (int64_t) blockIdx.x * blockDim.x + threadIdx.x;
        const int     ui   = (int) (gid / (ROWS * TPRW)), rr = (int) (gid / TPRW) % ROWS, c = (int) (gid % TPRW) * 8;
        const int     br = ui / upb, which = ui - br * upb;
        vkc_grid_dep_wait(); // launched with programmatic serialization: the partials are complete only after this
        vkc_grid_dep_launch();
        if (br < left) {
            const int     nb  = p.pairing ? p.nq / 2 : p.nq;
            const int64_t blk = (int64_t) p.rounds * main_ctas + br, bh = blk / nb;
            const int     k2  = (int) (blk - bh * nb);
            int           qg = k2, nu = p.steps, uoff = 0;
            if (p.pairing) {
                const int n_hi = unit_steps<QT>(p.Sq, p.Skv, 1, p.nq - 1 - k2);
                if (which == 0) qg = p.nq - 1 - k2, nu = n_hi;
                else uoff = n_hi, nu = p.steps - n_hi;
            }
            const int64_t s0 = (int64_t) br * p.ustride + uoff, s1 = s0 + nu - 1; // the unit's steps in the line
            const int64_t ca = s0 / p.quota, cb = s1 / p.quota;
            const int64_t h = bh % p.Hq, b = bh / p.Hq, grow = (int64_t) qg * ROWS + rr;
            if (nu > 0 && ca != cb && grow < p.Sq) {
                const T *part_o = (const T *) p.part_o;
                float    m      = -INFINITY;
                for (int64_t cc = ca; cc <= cb; ++cc) {
                    const int64_t prow = (cc * 2 + (s0 < cc * p.quota ? 0 : 1)) * ROWS + rr;
                    m                  = fmaxf(m, p.part_ml[prow * 2]);
                }
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, wsum = 0.f;
                for (int64_t cc = ca; cc <= cb; ++cc) {
                    const int64_t prow = (cc * 2 + (s0 < cc * p.quota ? 0 : 1)) * ROWS + rr;
                    const float   ms = p.part_ml[prow * 2], ls = p.part_ml[prow * 2 + 1];
                    const float   wt = ms == -INFINITY ? 0.f : ls * exp2f(ms - m);
                    wsum += wt;
                    const uint4 pv = *reinterpret_cast<const uint4 *>(part_o + prow * D + c);
                    const T    *pt = reinterpret_cast<const T *>(&pv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += wt * St<T>::ld(pt + i);
                }
                const float   inv  = 1.0f / wsum; // 0/0 -> NaN for a row with no visible key
                const int64_t ooff = b * p.os[0] + h * p.os[1] + grow * p.os[2] + c;
                if (p.fan.n_dest == 0) {
                    T *orow = (T *) p.O + ooff;
#pragma unroll
                    for (int i = 0; i < 8; ++i) St<T>::st(orow + i, acc[i] * inv);
                } else {
                    uint4 ov; // the launcher checked that every destination takes 16-byte stores
                    T    *ot = reinterpret_cast<T *>(&ov);
#pragma unroll
                    for (int i = 0; i < 8; ++i) St<T>::st(ot + i, acc[i] * inv);
                    vkc_fanout_store16<T>(p.fan, ooff, ov);
                }
            }
        }
        // every thread of every block; the rows that the attention kernel itself fanned out were complete before this kernel began
        if (p.fan.n_dest > 0) fanout_signal(p.fan, gridDim.x);
    }

    // How the balanced form would distribute `units` units of `steps` key tiles over `slots` resident CTAs, and a rough cost of
    // both forms in key-tile steps of one CTA (a unit run by a CTA of its own pays about two steps for launch, set-up, first
    // loads and the final stores; an item of a persistent CTA about one; cut units pay about three more for the merge pass).
    struct Plan {
        int64_t ctas, rounds, left, total, quota, ustride, pieces;
        double  cost_balanced, cost_per_unit;
    };
    inline Plan plan_balanced(int64_t units, int64_t steps, int64_t slots) {
        Plan pl;
        pl.rounds = units / slots, pl.left = units - pl.rounds * slots;
        pl.pieces = 1, pl.quota = steps, pl.ustride = steps;
        if (pl.left > 0) { // pieces of at least three key tiles, as many per unit as there are CTAs for
            int64_t want = slots / pl.left;
            if (want > steps / 3) want = steps / 3;
            if (want < 1) want = 1;
            pl.quota   = (steps + want - 1) / want;
            pl.pieces  = (steps + pl.quota - 1) / pl.quota;
            pl.ustride = pl.pieces * pl.quota;
        }
        pl.total = pl.left * pl.ustride;
        pl.ctas  = pl.rounds > 0 ? slots : pl.left * pl.pieces;
        if (pl.ctas < 1) pl.ctas = 1;
        pl.cost_balanced = (double) pl.rounds * (steps + 1.0) + (pl.left > 0 ? (double) pl.quota + (pl.pieces > 1 ? 2.0 + 3.0 : 1.0) : 0.0);
        pl.cost_per_unit = (double) ((units + slots - 1) / slots) * (steps + 2.0);
        return pl;
    }

    // The distribution of one call: which form, and the fields of AttnParams that describe it (everything but the scratch
    // pointers). Pure arithmetic on the shape and the SM count, shared by the launcher and by vkc_attn_prefill_plan / _items.
    struct Distribution {
        int     qt;       // query tiles per CTA
        bool    balanced; // persistent CTAs over blocks (else one CTA per unit on a (groups, Hq, B) grid)
        Plan    pl;       // meaningful when balanced
        int64_t nq;       // query groups per (batch, head)
    };
    // fills p.balanced / pairing / nq / steps / quota / rounds / ustride / total for `qt` query tiles per CTA
    template <int QT> Distribution distribute_qt(AttnParams &p, int64_t B, bool want_balanced, int64_t sms) {
        Distribution d;
        d.qt = QT, d.balanced = false;
        d.nq = (p.Sq + QT * BM - 1) / (QT * BM);
        const int64_t slots = sms * (QT == 1 ? 2 : 1);
        // blocks of equal length: the units themselves, or with a causal mask the pairs of groups (nq - 1 - k, k)
        const int     pairing = want_balanced && p.causal ? 1 : 0;
        const int64_t units   = (pairing ? d.nq / 2 : d.nq) * p.Hq * B;
        const int64_t steps   = pairing ? unit_steps<QT>(p.Sq, p.Skv, 1, (int) d.nq - 1) + unit_steps<QT>(p.Sq, p.Skv, 1, 0) : (p.Skv + BN - 1) / BN;
        p.balanced = 0, p.pairing = 0;
        p.nq = (int) d.nq, p.steps = (int) steps, p.quota = 1, p.total = 0, p.rounds = 0, p.ustride = (int) steps;
        if (want_balanced) {
            d.pl = plan_balanced(units, steps, slots);
            if (!(d.pl.rounds == 0 && d.pl.pieces == 1)) { // (one whole unit per CTA in a single round: the three-dimensional grid does the same)
                d.balanced = true;
                p.balanced = 1, p.pairing = pairing;
                p.rounds = (int) d.pl.rounds, p.quota = (int) d.pl.quota, p.ustride = (int) d.pl.ustride, p.total = (int) d.pl.total;
            }
        }
        return d;
    }
    // which form for the shape in p (Sq, Skv, Hq, causal, kv_len) and head size D
    Distribution distribute(AttnParams &p, int64_t B, int D, int64_t sms) {
        const int64_t pairs = ((p.Sq + 2 * BM - 1) / (2 * BM)) * p.Hq * B, steps = (p.Skv + BN - 1) / BN;
        // Head size 64: two one-tile CTAs fit an SM and their softmax and MMA phases overlap like the two tiles of the two-tile
        // form do, at finer granularity; unless the grid is many rounds deep anyway (then sharing K/V between two tiles wins).
        const bool one_tile = D == 64 && pairs < 6 * sms;
        // The balanced form (no per-sequence lengths) when its estimate is clearly the lower one.
        bool balanced = false, one_tile_balanced = false;
        if (p.causal && !p.kv_len && !one_tile && p.Sq == p.Skv && pairs > 0 && pairs * steps < (1ll << 29)) {
            // Causal: blocks are pairs of query groups (nq - 1 - k, k). The form needs every pair to add up to the same number of
            // key tiles (true whenever the sequence is a multiple of 256 rows) and an even number of groups.
            const int64_t nq = (p.Sq + 2 * BM - 1) / (2 * BM);
            int64_t       lo = INT64_MAX, hi = 0, work = 0, longest = unit_steps<2>(p.Sq, p.Skv, 1, (int) nq - 1);
            for (int64_t k = 0; k < nq / 2; ++k) {
                const int64_t sum = unit_steps<2>(p.Sq, p.Skv, 1, (int) (nq - 1 - k)) + unit_steps<2>(p.Sq, p.Skv, 1, (int) k);
                lo = sum < lo ? sum : lo, hi = sum > hi ? sum : hi, work += sum;
            }
            if (nq % 2 == 0 && nq >= 2 && lo == hi) {
                const Plan   pl = plan_balanced((nq / 2) * p.Hq * B, hi, sms);
                // one CTA per unit: the heavy units start first, which leaves about half of the longest unit as a tail
                const double pu = (double) (work * p.Hq * B) / (double) sms + 2.0 * (double) ((pairs + sms - 1) / sms) + 0.5 * (double) longest;
                // (a block holds two items; measured: 1171 -> 1227 TFLOP/s at S = 8192 and 1207 -> 1289 at 16384 with six and
                // more rounds of blocks, nothing at three, and a loss when the blocks do not even fill the SMs twice)
                balanced = pl.rounds >= 2 && pl.cost_balanced + (double) pl.rounds < 0.985 * pu;
            }
        }
        if (!p.causal && !p.kv_len && pairs > 0 && steps >= 1 && pairs * steps < (1ll << 29)) {
            const Plan pl = plan_balanced(pairs, steps, sms);
            double     pu = pl.cost_per_unit, bal = pl.cost_balanced;
            if (one_tile) { // one-tile units, two CTAs per SM, each about as fast as a two-tile CTA alone
                const int64_t tiles = ((p.Sq + BM - 1) / BM) * p.Hq * B;
                const Plan    p1    = plan_balanced(tiles, steps, 2 * sms);
                pu                  = p1.cost_per_unit;
                // (on a tie the two-tile form when whole rounds of units dominate, the one-tile form for a handful of units)
                if (p1.cost_balanced < bal || (p1.cost_balanced == bal && p1.rounds == 0)) bal = p1.cost_balanced, one_tile_balanced = true;
            }
            balanced = bal < 0.985 * pu;
        }
        if (one_tile && (!balanced || one_tile_balanced)) return distribute_qt<1>(p, B, balanced, sms);
        return distribute_qt<2>(p, B, balanced, sms);
    }

    template <typename T, int D, int QT>
    int launch_attn_qt(vkc_ctx *ctx, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, AttnParams &p, int64_t B, Distribution d,
                       cudaStream_t st) {
        auto          kern = attn_prefill_kernel<T, D, 2, QT>;
        constexpr int smem = (int) Smem<D, 2, 2, QT>::total;
        static_assert(smem * (QT == 1 && D == 64 ? 2 : 1) <= 227 * 1024, "shared memory budget");
        if (int rc = vkc_configure_smem(ctx, kern, smem)) return rc;
        if (d.balanced) {
            const Plan  &pl       = d.pl;
            const size_t prows    = (size_t) pl.ctas * 2 * QT * BM;
            const size_t ml_bytes = (prows * 2 * sizeof(float) + 255) & ~(size_t) 255;
            if (vkc_ensure_scratch(ctx, ml_bytes + prows * D * 2 + 256, st) == VKC_OK) {
                p.part_ml = (float *) ctx->scratch;
                p.part_o  = (char *) ctx->scratch + ml_bytes;
                vkc_launch(ctx, kern, dim3((unsigned) pl.ctas), dim3(threads_for(QT)), smem, st, tq, tk, tv, p);
                if (int rc = vkc_post_launch(ctx, "attn_prefill_tcgen05")) return rc;
                if ((pl.left == 0 || pl.pieces == 1) && p.fan.n_dest == 0) return VKC_OK; // nothing was cut
                // (with a fan-out the merge kernel also publishes the flags, so it runs even when it has nothing to join)
                const int64_t threads = pl.left * (p.pairing ? 2 : 1) * QT * BM * (D / 8);
                vkc_launch(ctx, attn_prefill_merge_kernel<T, D, QT>, dim3((unsigned) (threads > 0 ? (threads + 255) / 256 : 1)), dim3(256), 0, st, p,
                           (int) pl.ctas, (int) pl.left);
                return vkc_post_launch(ctx, "attn_prefill_merge");
            }
            distribute_qt<QT>(p, B, false, ctx->sm_count); // no scratch to be had: one CTA per unit
        }
        dim3 grid((unsigned) d.nq, (unsigned) p.Hq, (unsigned) B);
        vkc_launch(ctx, kern, grid, dim3(threads_for(QT)), smem, st, tq, tk, tv, p);
        return vkc_post_launch(ctx, "attn_prefill_tcgen05");
    }
    template <typename T, int D>
    int launch_attn(vkc_ctx *ctx, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, AttnParams &p, int64_t B, cudaStream_t st) {
        const Distribution d = distribute(p, B, D, ctx->sm_count);
        if (D == 64 && d.qt == 1) return launch_attn_qt<T, 64, 1>(ctx, tq, tk, tv, p, B, d, st);
        return launch_attn_qt<T, D, 2>(ctx, tq, tk, tv, p, B, d, st);
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
                             int causal, const int32_t *kv_len, int dtype, const vkc_fanout *fan, cudaStream_t st) {
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
    p.balanced = 0;
    if (int frc = vkc_fan_to_dev(ctx, fan, &p.fan, "attn_prefill_fanout")) return frc;
    if (fan) {
        if ((os[0] % 8) || (os[1] % 8) || (os[2] % 8)) return vkc_fail(ctx, VKC_ERR_UNSUPPORTED, "attn_prefill_fanout: output strides must be multiples of 16 bytes");
        p.O = fan->dest[0];
    }
    p.part_o     = nullptr;
    p.part_ml    = nullptr;
    if (dtype == VKC_F16) return D == 64 ? launch_attn<__half, 64>(ctx, tq, tk, tv, p, B, st) : launch_attn<__half, 128>(ctx, tq, tk, tv, p, B, st);
    return D == 64 ? launch_attn<__nv_bfloat16, 64>(ctx, tq, tk, tv, p, B, st) : launch_attn<__nv_bfloat16, 128>(ctx, tq, tk, tv, p, B, st);
}

// ---- introspection of the work distribution (host arithmetic only: no device, no context) -------------------------------
namespace {
    void plan_params(AttnParams &p, int64_t Hq, int64_t Sq, int64_t Skv, int causal, int has_kv_len) {
        p = AttnParams();
        p.Sq = Sq, p.Skv = Skv, p.Hq = Hq, p.Hkv = Hq;
        p.causal = causal;
        p.kv_len = has_kv_len ? reinterpret_cast<const int32_t *>(uintptr_t(1)) : nullptr; // only ever tested for null on the host
    }
} // namespace

extern "C" int vkc_attn_prefill_plan(int sm_count, int64_t B, int64_t Hq, int64_t Sq, int64_t Skv, int64_t D, int causal, int has_kv_len,
                                      int32_t *plan) {
    if (sm_count < 1 || B < 1 || Hq < 1 || Sq < 1 || Skv < 0 || (D != 64 && D != 128) || !plan) return VKC_ERR_INVALID;
    AttnParams p;
    plan_params(p, Hq, Sq, Skv, causal, has_kv_len);
    const Distribution d = distribute(p, B, (int) D, sm_count);
    plan[0] = d.balanced ? 1 : 0;
    plan[1] = d.qt;
    plan[2] = d.balanced ? (int32_t) d.pl.ctas : (int32_t) (d.nq * Hq * B);
    plan[3] = p.rounds;
    plan[4] = d.balanced ? (int32_t) d.pl.left : 0;
    plan[5] = d.balanced ? (int32_t) d.pl.pieces : 1;
    plan[6] = p.quota;
    plan[7] = p.steps;
    return VKC_OK;
}

extern "C" int vkc_attn_prefill_items(int sm_count, int64_t B, int64_t Hq, int64_t Sq, int64_t Skv, int64_t D, int causal, int has_kv_len, int cta,
                                       int32_t *items, int max_items) {
    if (sm_count < 1 || B < 1 || Hq < 1 || Sq < 1 || Skv < 0 || (D != 64 && D != 128) || cta < 0 || (!items && max_items > 0)) return VKC_ERR_INVALID;
    AttnParams p;
    plan_params(p, Hq, Sq, Skv, causal, has_kv_len);
    const Distribution d = distribute(p, B, (int) D, sm_count);
    p.kv_len = nullptr; // (per-sequence lengths only shorten the items of the one-CTA-per-unit form)
    CtaId c;
    if (d.balanced) {
        if (cta >= d.pl.ctas) return VKC_ERR_INVALID;
        c = CtaId {cta, 0, 0, (int) d.pl.ctas};
    } else {
        if (cta >= d.nq * Hq * B) return VKC_ERR_INVALID;
        c = CtaId {(int) (cta % d.nq), (int) ((cta / d.nq) % Hq), (int) (cta / (d.nq * Hq)), (int) d.nq};
    }
    int n = 0;
    for (int pos = 0;;) {
        int32_t row[8];
        bool    last;
        int     adv;
        if (d.qt == 1) {
            const Work<1> w = work_at<1>(p, pos, c);
            if (!w.valid) break;
            row[0] = w.b, row[1] = w.h, row[2] = w.qg, row[3] = w.j0, row[4] = w.n_t[0], row[5] = 0, row[6] = w.slot, row[7] = w.last;
            last = w.last, adv = w.adv;
        } else {
            const Work<2> w = work_at<2>(p, pos, c);
            if (!w.valid) break;
            row[0] = w.b, row[1] = w.h, row[2] = w.qg, row[3] = w.j0, row[4] = w.n_t[0], row[5] = w.n_t[1], row[6] = w.slot, row[7] = w.last;
            last = w.last, adv = w.adv;
        }
        if (n < max_items)
            for (int i = 0; i < 8; ++i) items[n * 8 + i] = row[i];
        ++n;
        pos += adv;
        if (last) break;
    }
    return n;
}
