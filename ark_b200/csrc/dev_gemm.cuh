// Tiled matmul on the 5th-generation tensor cores (sm_100a).
//
// Replaces the reference's matmul -> gemm_cutlass -> CUTLASS 2.x mma.sync path
// (ark/include/kernels/matmul.h:36-115, gemm_cutlass.h:900-965). One CTA runs a
// list of 128 x tile_n output tiles with three warp roles:
//   warp 4      : TMA producer  — cp.async.bulk.tensor loads of A and B
//                 k-blocks (64 elements of K) into a 4-deep shared-memory ring;
//   warp 5      : MMA issuer    — one elected lane issues tcgen05.mma
//                 (M=128, N=tile_n, K=16, fp32 accumulators in TMEM);
//   warps 0..3  : epilogue      — tcgen05.ld of the accumulator (each warp owns
//                 the 32 TMEM lanes of its quarter), activation / bias, one
//                 rounding to the storage type, 128-bit stores.
// Two accumulators (2 x 256 TMEM columns) let the epilogue of tile i overlap
// the mainloop of tile i+1. No cluster launch, no multicast: every CTA loads
// its own operands, so the same code runs on any number of GPUs.
//
// Every wait is bounded; on expiry the CTA records a status and leaves.
#pragma once
#include "dev_common.cuh"
#include "dev_funcs.h"

namespace arkb {

constexpr int kGemmBK = 64;                       // K elements per stage (128 bytes of fp16/bf16)
constexpr int kGemmTileM = 128;                   // accumulator rows per CTA
constexpr int kGemmABytes = kGemmTileM * kGemmBK * 2;   // 16 KiB
// One CTA per tile: B tile up to 256 columns (32 KiB), 4 stages.
// CTA pair per tile (cta_group::2, 256 x tile_n): each CTA stages its 128 rows
// of A and half of the B columns (16 KiB), 6 stages.
template <bool PAIR>
struct GemmCfg {
    static constexpr int kStages = PAIR ? 6 : 4;
    static constexpr int kBBytes = (PAIR ? 128 : 256) * kGemmBK * 2;
    static constexpr int kStageBytes = kGemmABytes + kBBytes;
};
constexpr int kGemmMaxStages = 12;  // skinny (swapped) problems stage small B blocks and use more, smaller stages
constexpr int kGemmPipeBytes = 4 * (kGemmABytes + 256 * kGemmBK * 2);  // 192 KiB of operand stages in both modes
// epilogue staging: per epilogue warp two 32-row x 64-byte blocks (64-byte swizzle)
constexpr int kEpiBlockBytes = 32 * 64;
constexpr int kEpiStageBytes = 4 * 2 * kEpiBlockBytes;                  // 16 KiB
constexpr int kGemmSmemBytes = kGemmPipeBytes + kEpiStageBytes;
static_assert(kGemmSmemBytes >= kSwappedRingBytes, "ring of the swapped form must fit the kernel's shared memory");
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 4, kProducerWarp = 4, kMmaWarp = 5, kProducerWarpB = 6;  // warp 4 loads A, warp 6 loads B

struct GemmPipe {
    unsigned long long full[kGemmMaxStages];
    unsigned long long empty[kGemmMaxStages];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned int use[kGemmMaxStages];  // completed uses of each ring slot since launch (gives the barrier phase)
    unsigned int tile_count;  // tiles this CTA has finished since launch
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(void *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void *bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void *bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// Bounded wait on an mbarrier phase; false when `limit_ns` nanoseconds ran out.
__device__ __forceinline__ bool mbar_wait(void *bar, uint32_t parity, unsigned long long limit_ns) {
    const uint32_t a = smem_u32(bar);
    unsigned long long t0 = 0;
    for (unsigned long long i = 1;; ++i) {
        uint32_t ok;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((i & 255) == 0) {
            const unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit_ns) return false;
        }
    }
}

__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *tm, void *bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tma_load_5d(void *smem_dst, const CUtensorMap *tm, void *bar, int c0, int c1, int c2,
                                            int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
// Bits: [0,14) start>>4, [16,30) leading byte offset>>4, [32,46) stride byte
// offset>>4, [46,48) version = 1, [61,64) layout = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A/B fp16 or bf16.
__device__ __forceinline__ uint32_t umma_idesc(int bf16, int a_mn, int b_mn, int n, int m = kGemmTileM) {
    uint32_t d = 0;
    d |= 1u << 4;                        // D format: F32
    d |= (uint32_t)(bf16 ? 1 : 0) << 7;  // A format
    d |= (uint32_t)(bf16 ? 1 : 0) << 10; // B format
    d |= (uint32_t)(a_mn ? 1 : 0) << 15; // A major: 0 K, 1 MN
    d |= (uint32_t)(b_mn ? 1 : 0) << 16; // B major
    d |= (uint32_t)(n >> 3) << 17;       // N / 8
    d |= (uint32_t)(m >> 4) << 24;       // M / 16
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void umma_commit(void *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// TMA store of a staged block (shared -> global), tracked by bulk async-groups.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *tm, const void *smem_src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tm),
                 "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until at most N of this thread's bulk groups are still reading shared memory / still in flight.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// TMEM allocation for the whole CTA lifetime (one warp executes these).
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, int cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, int cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// pair == true: the accumulator-empty barrier of the leader CTA collects the
// epilogue warps of both CTAs.
// ---- CTA-pair (cta_group::2) variants --------------------------------------------------
// Address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void tma_load_4d_pair(void *smem_dst, const CUtensorMap *tm, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2, int c3) {
    // data lands in this CTA's shared memory, the byte count is credited to the
    // leader CTA's barrier; no multicast: every CTA loads its own operands
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tm), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d_pair(void *smem_dst, const CUtensorMap *tm, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tm), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
// Arrive on a barrier (given as a shared::cluster address, own or peer CTA) when
// the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, int cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, int cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void gemm_pipe_init(GemmPipe *pp, bool pair) {
    for (int s = 0; s < kGemmMaxStages; ++s) {
        mbar_init(&pp->full[s], 2);  // one arrival per producer warp (A and B)
        mbar_init(&pp->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
        mbar_init(&pp->acc_full[a], 1);
        mbar_init(&pp->acc_empty[a], pair ? 2 * kEpiWarps : kEpiWarps);
    }
    for (int s = 0; s < kGemmMaxStages; ++s) pp->use[s] = 0;
    pp->tile_count = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

}  // namespace arkb
