// In-kernel communication over peer-mapped memory (NVLink): put + signal /
// wait (send / recv), cross-rank barrier (device_sync) and all_reduce.
//
// Replaces the MSCCL++ proxy / SM channel layer of the reference
// (ark/include/kernels/comm.h:314-439): no host proxy thread, no packets —
// 128-bit peer stores and loads, flags written with st.release.sys and read
// with ld.acquire.sys. Every wait is bounded and reports a status.
#pragma once
#include "dev_common.cuh"
#include "dev_funcs.h"

namespace arkb {

__device__ __forceinline__ CommBlock *comm_block(const LaunchParams &P, int r) {
    return reinterpret_cast<CommBlock *>(P.comm[r]);
}

__device__ __forceinline__ bool wait_flag_ge(const unsigned long long *flag, unsigned long long want,
                                             unsigned long long limit) {
    unsigned long long spins = 0, t0 = 0;
    while (ld_acquire_sys(flag) < want) {
        ++spins;
        if ((spins & 255) == 0) {
            const unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit) return false;  // limit is in nanoseconds
        }
        if (spins > 32) __nanosleep(64);
    }
    return true;
}

// Raise channel flag on the receiver. Runs on one CTA after a grid barrier has
// collected the put's stores.
__device__ __forceinline__ void run_signal(const LaunchParams &P, const SignalArgs &a, unsigned long long iter_no) {
    if (threadIdx.x == 0) {
        __threadfence_system();
        st_release_sys(&comm_block(P, a.peer)->chan_flag[P.rank * kChannels + a.channel], iter_no);
    }
}

__device__ __forceinline__ void run_wait(const LaunchParams &P, const WaitArgs &a, unsigned long long iter_no,
                                         CtaCtl *ctl, int stage) {
    if (threadIdx.x == 0) {
        if (!wait_flag_ge(&comm_block(P, P.rank)->chan_flag[a.peer * kChannels + a.channel], iter_no, P.spin_limit)) {
            ctl->abort = 1;
            report(P.state, ST_PEER_TIMEOUT, stage);
        }
    }
}

// Cross-rank barrier: every rank writes its epoch into slot [rank] of every
// peer's block, then waits until all slots of its own block reached the epoch.
// One CTA runs it, between two grid barriers.
__device__ __forceinline__ void run_peersync(const LaunchParams &P, unsigned long long epoch, CtaCtl *ctl, int stage) {
    const int t = threadIdx.x;
    if (t == 0) __threadfence_system();
    __syncthreads();
    if (t < P.nranks && t != P.rank) st_release_sys(&comm_block(P, t)->barrier_flag[P.rank], epoch);
    if (t < P.nranks && t != P.rank) {
        if (!wait_flag_ge(&comm_block(P, P.rank)->barrier_flag[t], epoch, P.spin_limit)) {
            ctl->abort = 1;
            report(P.state, ST_PEER_TIMEOUT, stage);
        }
    }
    __syncthreads();
}

}  // namespace arkb
