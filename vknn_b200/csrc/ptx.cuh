// Inline-PTX wrappers for the sm_100a features the kernels use: mbarriers, TMA tiled bulk copies (plain,
// per-CTA form only), tensor memory (TMEM) management and 5th-generation tensor-core MMAs (tcgen05).
//
// Every wait on an mbarrier is BOUNDED: after ~1 s of spinning it records VKC_DEVERR_WAIT_TIMEOUT in the
// context's device error word, raises a CTA-wide abort flag in shared memory and returns false, so a kernel
// can drain, release its tensor memory and exit instead of hanging the GPU.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace ptx {

    __device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t) __cvta_generic_to_shared(p); }

    __device__ __forceinline__ bool elect_one() {
        uint32_t pred;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "elect.sync _|p, 0xffffffff;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(pred));
        return pred != 0;
    }

    // ---- mbarrier ---------------------------------------------------------------------------------------
    __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
    }
    __device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    __device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
    __device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    }
    __device__ __forceinline__ void mbar_arrive(uint32_t bar) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
    }
    __device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        return ok != 0;
    }

    constexpr long long kWaitLimitCycles = 2000000000LL; // ~1 s at 2 GHz

    // Bounded wait. `abort_flag` lives in shared memory and is shared by every waiter of the CTA.
    __device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *dev_err) {
        if (mbar_try_wait(bar, parity)) return true;
        const long long t0 = clock64();
        for (;;) {
            if (mbar_try_wait(bar, parity)) return true;
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                atomicCAS(dev_err, 0, 1 /* VKC_DEVERR_WAIT_TIMEOUT */);
                return false;
            }
        }
    }

    // ---- TMA tiled loads (global -> this CTA's shared memory, completion on an mbarrier) ----------------
    __device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                     "l"(map), "r"(x), "r"(y), "r"(bar)
                     : "memory");
    }
    __device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                     "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                     : "memory");
    }
    __device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, int w, uint32_t bar) {
        asm volatile(
            "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
            "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
            : "memory");
    }
    // Tiled store shared memory -> global (clipped at the tensor bounds); completion is tracked per thread in bulk groups.
    __device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int x, int y, int z) {
        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src), "r"(x), "r"(y),
                     "r"(z)
                     : "memory");
    }
    __device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
    __device__ __forceinline__ void bulk_wait_group_0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
    // Waits only until the committed bulk stores have read their shared-memory source (enough before the CTA exits or
    // reuses the staging area; the global writes complete on their own).
    __device__ __forceinline__ void bulk_wait_group_read_0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
    // Same, but leaves the most recently committed group in flight.
    __device__ __forceinline__ void bulk_wait_group_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
    // Untiled bulk copy of `bytes` contiguous bytes (both addresses 16-byte aligned, size a multiple of 16).
    __device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                     "r"(bar)
                     : "memory");
    }
    // Packed fp32 pair arithmetic (two independent fp32 FMAs per instruction).
    __device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
        float2 d;
        asm("fma.rn.f32x2 %0, %1, %2, %3;"
            : "=l"(reinterpret_cast<unsigned long long &>(d))
            : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)),
              "l"(reinterpret_cast<const unsigned long long &>(c)));
        return d;
    }
    __device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
        float2 d;
        asm("mul.rn.f32x2 %0, %1, %2;"
            : "=l"(reinterpret_cast<unsigned long long &>(d))
            : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)));
        return d;
    }
    __device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
        float2 d;
        asm("add.rn.f32x2 %0, %1, %2;"
            : "=l"(reinterpret_cast<unsigned long long &>(d))
            : "l"(reinterpret_cast<const unsigned long long &>(a)), "l"(reinterpret_cast<const unsigned long long &>(b)));
        return d;
    }
    __device__ __forceinline__ float fmax3(float a, float b, float c) {
        float d;
        asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
        return d;
    }
    // Register re-partitioning between warpgroups (all four warps of a warpgroup execute the same one).
    template <int N> __device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
    template <int N> __device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
    __device__ __forceinline__ void prefetch_tmap(const CUtensorMap *map) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
    }

    // ---- tensor memory ----------------------------------------------------------------------------------
    // Allocation is warp-collective; the base address is written to shared memory at `slot`.
    __device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t ncols) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
    }
    __device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
    __device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    }
    __device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
    __device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
    __device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
    __device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

    // Arrive on an mbarrier once every MMA issued so far by this thread has completed.
    __device__ __forceinline__ void tc_commit(uint32_t bar) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }

    // Shared-memory operand descriptor, 128-byte swizzle. For a K-major operand (K contiguous, rows of 64
    // 16-bit elements = 128 B, groups of 8 rows = 1024 B): sbo = 1024, lbo unused (encoded 1).
    // For an MN-major operand (MN contiguous in spans of 64 elements): lbo = byte stride between 64-element
    // MN spans, sbo = byte stride between groups of 8 K rows (1024 for densely stacked rows).
    __device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
        uint64_t d = 0;
        d |= (uint64_t) ((saddr & 0x3FFFFu) >> 4);
        d |= (uint64_t) ((lbo_bytes >> 4) & 0x3FFFu) << 16;
        d |= (uint64_t) ((sbo_bytes >> 4) & 0x3FFFu) << 32;
        d |= 1ull << 46; // descriptor version for sm_100
        d |= 2ull << 61; // SWIZZLE_128B
        return d;
    }

    // Instruction descriptor for kind::f16 with fp32 accumulation.
    __host__ __device__ constexpr uint32_t idesc_f16(int M, int N, bool bf16, bool a_mn_major, bool b_mn_major) {
        return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
               ((uint32_t) (N >> 3) << 17) | ((uint32_t) (M >> 4) << 24);
    }

    // D[tmem] (+)= A[smem] * B[smem]
    __device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
    // D[tmem] (+)= A[tmem] * B[smem]
    __device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
            "}\n" ::"r"(d_tmem),
            "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }

    // ---- CTA pairs (cluster of two CTAs driving one cta_group::2 MMA) ------------------------------------
    __device__ __forceinline__ uint32_t cluster_ctarank() {
        uint32_t r;
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
        return r;
    }
    // Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
    __device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
        uint32_t r;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
        return r;
    }
    __device__ __forceinline__ void cluster_sync() {
        asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    // Split-K reduction through distributed shared memory: 16-byte store into a peer CTA's shared memory, arrival on a
    // peer's mbarrier with cluster-scope release, and the matching bounded wait with cluster-scope acquire.
    __device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
        asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
    }
    __device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
        uint4 v;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
        return v;
    }
    __device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
    }
    __device__ __forceinline__ void fence_acq_rel_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
    __device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
    }
    // Bulk copy from this CTA's shared memory into a peer CTA's (shared::cluster addresses for destination and barrier);
    // the bytes are credited to the peer's mbarrier. Addresses and size are multiples of 16.
    __device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes, uint32_t bar_cluster) {
        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_cluster), "r"(src_cta),
                     "r"(bytes), "r"(bar_cluster)
                     : "memory");
    }
    // The two halves of a cluster barrier, so that work can sit between the arrival and the wait.
    __device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
    __device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
    __device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        return ok != 0;
    }
    __device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *dev_err) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        const long long t0 = clock64();
        for (;;) {
            if (mbar_try_wait_cluster(bar, parity)) return true;
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                atomicCAS(dev_err, 0, 1 /* VKC_DEVERR_WAIT_TIMEOUT */);
                return false;
            }
        }
    }
    // Tiled load issued by either CTA of a pair; the completion bytes go to the mbarrier at `bar`, which may live in
    // the other CTA of the pair (a shared::cluster address).
    __device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
            "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
            : "memory");
    }
    __device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t ncols) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(ncols) : "memory");
    }
    __device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
    __device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    }
    // Arrive on the mbarrier at `bar` (a shared::cluster address, own or peer CTA) once every pair MMA issued so far
    // by this thread has completed.
    __device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }
    // D[tmem of both CTAs, 256 rows] (+)= A[smem of both CTAs] * B[smem halves of both CTAs]; issued by the leader CTA.
    __device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem),
            "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }

    // TMEM -> registers: each thread of the warp reads its own lane (row), N consecutive 32-bit columns.
    __device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
              "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
              "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr)
            : "memory");
    }
    __device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
              "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr)
            : "memory");
    }
    // registers -> TMEM, same thread-to-lane mapping
    __device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
            "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
            "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
            "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
            "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
            "r"(r[31])
            : "memory");
    }
    __device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
            "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
            "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
            : "memory");
    }

} // namespace ptx
