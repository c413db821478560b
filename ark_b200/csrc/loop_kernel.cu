// The persistent loop kernel: one CTA per processor walks the stage list of a
// lowered plan, once per iteration, and in loop mode stays resident waiting
// for run requests on a host-mapped flag. Counterpart of the reference's
// generated ark_loop_kernel / ark_kernel
// (ark/include/kernels/kernel_template.in:40-78).
#include "dev_comm.cuh"
#include "dev_common.cuh"
#include "dev_funcs.h"
#include "dev_gemm.cuh"
#include "loop_kernel.h"

#include <algorithm>
#include <cstring>

namespace arkb {

__device__ __forceinline__ bool in_range(const Stage &S, int cta, int &p, int &Pn) {
    const int b = S.proc_b, e = S.proc_e, s = S.proc_s;
    Pn = (e - b + s - 1) / s;
    if (cta < b || cta >= e) return false;
    const int d = cta - b;
    if (d % s) return false;
    p = d / s;
    return true;
}

// One pass over the stage list. iter_local counts iterations since this
// launch (barrier phases); iter_no is the 1-based iteration number over the
// executor's life (cross-rank epochs and channel flags).
// Stage records are read through a two-slot cache in shared memory: while a CTA works on stage s the
// record of stage s+1 (of stage 0 after the last one) is copied asynchronously into the other slot, so
// the global-memory latency of fetching a record is off the path between two stages.
struct StageCache {
    Stage slot[2];
};

__device__ __forceinline__ void stage_fetch(StageCache *sc, int slot, const Stage *src) {
    constexpr int kWords = sizeof(Stage) / 16;
    static_assert(sizeof(Stage) % 16 == 0 && kWords <= kThreads, "stage record is copied 16 bytes per thread");
    if (threadIdx.x < kWords) {
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(reinterpret_cast<char *>(&sc->slot[slot]) + threadIdx.x * 16);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(reinterpret_cast<const char *>(src) + threadIdx.x * 16)
                     : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void stage_fetch_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <bool PAIR>
__device__ __forceinline__ void run_body(const LaunchParams &P, char *smem, GemmPipe *pipe, CtaCtl *ctl, StageCache *sc,
                                         int &cur, unsigned long long iter_local, unsigned long long iter_no) {
    const int cta = blockIdx.x;
    for (int s = 0; s < P.n_stages; ++s) {
        stage_fetch_wait();
        __syncthreads();  // the record of stage s has landed; every thread is done with stage s-1
        // `cur` (the slot holding stage s) is the same in every thread: all threads of a CTA walk the same stages
        const Stage &S = sc->slot[cur];
        stage_fetch(sc, cur ^ 1, &P.stages[s + 1 == P.n_stages ? 0 : s + 1]);
        cur ^= 1;
        int p = 0, Pn = 1;
        if (!in_range(S, cta, p, Pn)) continue;
        if (ctl->abort) return;
        unsigned long long *stamp = P.stage_times ? P.stage_times + ((size_t)s * gridDim.x + cta) * 2 : nullptr;
        if (stamp && threadIdx.x == 0) stamp[0] = globaltimer();
        switch (S.kind) {
            case SK_SYNC: {
                // while this CTA waits, the L2 fetches its share of operands that stages behind the barrier will stream
                if (threadIdx.x >= 32 && (int)threadIdx.x < 32 + S.sy.n_pf) {
                    const int e = threadIdx.x - 32;
                    const unsigned long long bytes = S.sy.pf_bytes[e];
                    const unsigned long long per = ((bytes + Pn - 1) / Pn + 127ull) & ~127ull;
                    const unsigned long long off = (unsigned long long)p * per;
                    if (off < bytes) {
                        const unsigned long long len = (bytes - off < per ? bytes - off : per) & ~15ull;
                        if (len) l2_prefetch(reinterpret_cast<const char *>(S.sy.pf_ptr[e]) + off, (uint32_t)len);
                    }
                }
                const unsigned long long k = iter_local * (unsigned long long)P.syncs_per_iter[S.sync_group] + S.sync_ord;
                if (!grid_barrier(&P.state->barrier[S.sync_group], k * (unsigned long long)S.sync_count, P.spin_limit,
                                  ctl, P.state, s))
                    return;
                break;
            }
            case SK_EWISE: run_ewise(S.ew, p, Pn, iter_no); break;
            case SK_REDUCE: run_reduce(S.rd, p, Pn, smem); break;
            case SK_ROWOP: run_rowop(S.ro, p, Pn, smem, ctl, P.state, s, P.spin_limit); break;
            case SK_GEMM:
                if constexpr (PAIR) run_gemm_pair(S.gm, &P.stages[s].gm, p, Pn, smem, pipe, ctl, P.state, s, P.spin_limit);
                else run_gemm(S.gm, &P.stages[s].gm, p, Pn, smem, pipe, ctl, P.state, s, P.spin_limit);
                break;
            case SK_GEMV: run_gemv(S.gv, p, Pn, smem, P, iter_no); break;
            case SK_DECODE_ATTN: run_decode_attn(S.da, p, Pn, smem); break;
            case SK_PREFILL_ATTN:
                if constexpr (!PAIR) run_prefill_attn(S.pa, &P.stages[s].pa, p, Pn, smem, ctl, P.state, s, P.spin_limit);
                break;
            case SK_GEMM_SIMT: run_gemm_simt(S.gs, p, Pn, smem); break;
            case SK_SPLITK_REDUCE: run_splitk_reduce(S.sr, p, Pn); break;
            case SK_TRANSPOSE: run_transpose(S.tp, p, Pn, smem); break;
            case SK_EMBED: run_embed(S.em, p, Pn); break;
            case SK_PUT: run_put(S.put, p, Pn, iter_no); break;
            case SK_SIGNAL: if (p == 0) run_signal(P, S.sg, iter_no); break;
            case SK_WAITFLAG: if (p == 0) run_wait(P, S.wt, iter_no, ctl, s); break;
            case SK_PEERSYNC: {
                const unsigned long long epoch = (iter_no - 1) * (unsigned long long)P.peersyncs_per_iter + S.ps.ord;
                if (!S.ps.with_grid) {
                    if (p == 0) run_peersync(P, epoch, ctl, s);
                    break;
                }
                unsigned long long *ctr = &P.state->barrier[S.sync_group];
                const unsigned long long k = iter_local * (unsigned long long)P.syncs_per_iter[S.sync_group] + S.sync_ord;
                const unsigned long long done = k * (unsigned long long)S.sync_count;
                __syncthreads();
                if (threadIdx.x == 0) red_release_gpu_add(ctr, 1ull);
                if (p == 0) {
                    if (threadIdx.x == 0) counter_wait(ctr, done - 1, P.spin_limit, ctl, P.state, s);  // every CTA has arrived
                    __syncthreads();
                    if (!ctl->abort) run_peersync(P, epoch, ctl, s);
                    // a failed exchange releases nobody: the other CTAs give up at this barrier, not on incomplete data
                    if (threadIdx.x == 0 && !ctl->abort) red_release_gpu_add(ctr, 1ull);
                }
                if (threadIdx.x == 0) counter_wait(ctr, done, P.spin_limit, ctl, P.state, s);
                __syncthreads();
                if (ctl->abort) return;
                break;
            }
            case SK_ALLREDUCE: run_allreduce(P, S.ar, p, Pn, iter_no); break;
            case SK_PACKET: run_packet(P, S.pk, p, Pn, iter_no, ctl, s); break;
            case SK_PACKET_REDUCE: run_packet_reduce(P, S.pr, p, Pn, iter_no, ctl, s); break;
            default: break;
        }
        if (stamp) {
            __syncthreads();
            if (threadIdx.x == 0) stamp[1] = globaltimer();
        }
    }
}

template <bool PAIR>
__device__ __forceinline__ void loop_main(const LaunchParams &P) {
    extern __shared__ __align__(1024) char dyn_smem[];
    __shared__ CtaCtl ctl;
    __shared__ GemmPipe pipe;
    __shared__ StageCache stage_cache;
    // dynamic shared memory base rounded up to 1 KiB (128-byte swizzle atoms)
    char *smem = reinterpret_cast<char *>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~(uintptr_t)1023);

    if (threadIdx.x == 0) {
        ctl.abort = 0;
        ctl.run_iters = 0;
        gemm_pipe_init(&pipe, PAIR);
    }
    if (threadIdx.x < 32) {
        if constexpr (PAIR) tmem_alloc_pair(&ctl.tmem_base, kTmemCols);
        else tmem_alloc(&ctl.tmem_base, kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // the partner's barriers are initialised before anything signals them
    tc_fence_after();

    int cache_slot = 0;
    if (P.n_stages > 0) stage_fetch(&stage_cache, 0, &P.stages[0]);

    DeviceState *st = P.state;
    const int whole = kMaxSyncGroups - 1;  // barrier counter reserved for the run protocol
    unsigned long long whole_k = 0;        // whole-grid barriers passed since launch
    unsigned long long run_seq = 0;        // run requests seen since launch
    unsigned long long iter_local = 0;
    unsigned long long iter_no = st->iter_total;  // stable: only advanced after the last barrier of a run

    for (;;) {
        int iters = P.iters;
        if (P.loop_mode) {
            // CTA 0 polls the host's run flag and publishes each request (sequence number +
            // iteration count) in device memory; the other CTAs poll that word. Waiting for work
            // is not a failure: it is bounded by the idle limit, not by the wait limit.
            ++run_seq;
            if (threadIdx.x == 0) {
                const unsigned long long t0 = globaltimer();
                if (blockIdx.x == 0) {
                    int v;
                    for (;;) {
                        v = *P.run_flag;
                        if (v != 0) break;
                        if (globaltimer() - t0 > P.idle_limit_ns) {
                            v = -2;  // idle for too long: leave, the host relaunches on the next run
                            break;
                        }
                        __nanosleep(200);
                    }
                    st->run_iters = v;
                    __threadfence();
                    st_release_gpu(&st->run_seq, run_seq);
                    ctl.run_iters = v;
                } else {
                    int v = -2;
                    for (;;) {
                        if (ld_acquire_gpu(&st->run_seq) >= run_seq) {
                            v = *reinterpret_cast<volatile int32_t *>(&st->run_iters);
                            break;
                        }
                        if (globaltimer() - t0 > P.idle_limit_ns + P.spin_limit) break;
                        __nanosleep(500);
                    }
                    ctl.run_iters = v;
                }
            }
            __syncthreads();
            iters = ctl.run_iters;
            if (iters < 0) {
                // (an idle limit of 0 means one launch per request: leaving is then the normal end, not worth a note)
                if (iters == -2 && P.idle_limit_ns != 0 && blockIdx.x == 0 && threadIdx.x == 0) atomicCAS(&st->status, ST_OK, ST_IDLE_EXIT);
                break;
            }
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) st->t_begin = globaltimer();
        bool ok = true;
        for (int i = 0; i < iters && ok; ++i) {
            run_body<PAIR>(P, smem, &pipe, &ctl, &stage_cache, cache_slot, iter_local, iter_no + 1);
            ++whole_k;
            ok = grid_barrier(&st->barrier[whole], whole_k * gridDim.x, P.spin_limit, &ctl, st, -2);
            ++iter_local;
            ++iter_no;
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            st->t_end = globaltimer();
            st->iter_total = iter_no;
            if (st->host_iters) *st->host_iters = iter_no;  // the host checks this count against what it asked for
            __threadfence_system();
            if (P.loop_mode) *P.run_flag = 0;
        }
        if (!ok || !P.loop_mode) break;
    }

    stage_fetch_wait();
    __syncthreads();
    if (ctl.abort && threadIdx.x == 0) {
        // give bulk copies still in flight time to land before the CTA's shared memory goes away
        for (int i = 0; i < 64; ++i) __nanosleep(2000);
        if (P.loop_mode && blockIdx.x == 0) *P.run_flag = 0;
    }
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();  // neither CTA of a pair leaves while the other may still touch it
    tc_fence_after();
    if (threadIdx.x < 32) {
        if constexpr (PAIR) tmem_dealloc_pair(ctl.tmem_base, kTmemCols);
        else tmem_dealloc(ctl.tmem_base, kTmemCols);
    }
}

// One CTA per processor, tcgen05 cta_group::1.
extern "C" __global__ void __launch_bounds__(kThreads, 1) arkb_loop_kernel(const __grid_constant__ LaunchParams P) {
    loop_main<false>(P);
}
// Processors 2q and 2q+1 form a cluster (one SM pair); matmul tiles are shared by the pair (cta_group::2).
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    arkb_loop_kernel_pair(const __grid_constant__ LaunchParams P) {
    loop_main<true>(P);
}

}  // namespace arkb

// ---- host-side launch shim (keeps <<<>>> syntax inside the .cu file) ----------------
namespace arkb {
size_t loop_kernel_smem_bytes() { return kGemmSmemBytes + 1024; }

cudaError_t loop_kernel_prepare() {
    cudaError_t e = cudaFuncSetAttribute(arkb_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)loop_kernel_smem_bytes());
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(arkb_loop_kernel_pair, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)loop_kernel_smem_bytes());
}

// The grid barriers need every CTA resident at once, so the launch is cooperative: it is refused
// (cudaErrorCooperativeLaunchTooLarge) or queued behind other work instead of deadlocking when the grid
// does not fit beside what already runs on the device.
cudaError_t loop_kernel_launch(const LaunchParams &P, int grid, cudaStream_t stream, size_t smem_bytes) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    // + 1 KiB: the kernel rounds its base up to 1 KiB (128-byte swizzle atoms)
    cfg.dynamicSmemBytes = smem_bytes ? std::min(smem_bytes + 1024, loop_kernel_smem_bytes()) : loop_kernel_smem_bytes();
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = P.pair_mode ? cudaLaunchKernelEx(&cfg, arkb_loop_kernel_pair, P) : cudaLaunchKernelEx(&cfg, arkb_loop_kernel, P);
    if (e == cudaErrorNotSupported || e == cudaErrorInvalidValue) {
        // a driver that cannot combine the attribute with this kernel: plain launch (the caller keeps the grid <= #SMs)
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        e = P.pair_mode ? cudaLaunchKernelEx(&cfg, arkb_loop_kernel_pair, P) : cudaLaunchKernelEx(&cfg, arkb_loop_kernel, P);
    }
    return e;
}
}  // namespace arkb
