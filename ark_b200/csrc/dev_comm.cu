// Data movers of the in-kernel communication layer (see dev_comm.cuh).
#include "dev_comm.cuh"

namespace arkb {

// Dense byte copy local -> peer by all CTAs of the stage.
__device__ void run_put(const PutArgs &a, int p, int P) {
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x, nth = (int64_t)P * kThreads;
    const char *s = reinterpret_cast<const char *>(a.src);
    char *d = reinterpret_cast<char *>(a.dst);
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d) | (uintptr_t)a.bytes) & 15) == 0) {
        const int64_t n = a.bytes / 16;
        for (int64_t i = tid; i < n; i += nth) reinterpret_cast<uint4 *>(d)[i] = reinterpret_cast<const uint4 *>(s)[i];
    } else {
        for (int64_t i = tid; i < a.bytes; i += nth) d[i] = s[i];
    }
}

template <typename T>
__device__ void allreduce_typed(const LaunchParams &P, const AllReduceArgs &a, int p, int Pn, unsigned long long iter_no) {
    constexpr int V = 16 / sizeof(T);
    const int R = P.nranks, me = P.rank;
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x, nth = (int64_t)Pn * kThreads;
    const int64_t nv = a.nelem / V;  // host guarantees nelem % V == 0 and 16-byte alignment
    if (a.algo == 0) {
        const uint64_t par = (iter_no * (unsigned long long)a.per_iter + (unsigned long long)a.ord) & 1;
        const uint64_t base = kCommDataOff + par * a.stage_bytes;
        const uint64_t slot_bytes = a.stage_bytes / kMaxPeers;
        if (a.phase == 0) {
            const uint4 *src = reinterpret_cast<const uint4 *>(P.arena[me] + a.buf_off[me]);
            for (int64_t i = tid; i < nv; i += nth) {
                const uint4 v = src[i];
                for (int q = 0; q < R; ++q)
                    reinterpret_cast<uint4 *>(P.comm[q] + base + me * slot_bytes)[i] = v;
            }
        } else {
            T *dst = a.sum_out ? reinterpret_cast<T *>(a.sum_out) : reinterpret_cast<T *>(P.arena[me] + a.buf_off[me]);
            const T *res = reinterpret_cast<const T *>(a.residual);
            for (int64_t i = tid; i < nv; i += nth) {
                float acc[V];
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = 0.0f;
                for (int q = 0; q < R; ++q) {
                    float x[V];
                    load_vec<T, V>(reinterpret_cast<const T *>(P.comm[me] + base + q * slot_bytes) + i * V, x);
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] += x[k];
                }
                if (res) {  // the sum is rounded where the all_reduce would have stored it, then the residual is added
                    float r[V];
                    load_vec<T, V>(res + i * V, r);
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] = to_f32(from_f32<T>(acc[k])) + r[k];
                }
                store_vec<T, V>(dst + i * V, acc);
            }
        }
        return;
    }
    // two-shot and slots: this rank owns vectors [lo, hi). Two-shot reads the partial of every rank from that
    // rank's tensor; slots (algo 2) finds them in its own staging slots, where the peers' matmul epilogues put them.
    const int64_t per = (nv + R - 1) / R;
    const int64_t lo = per * me, hi = min(nv, lo + per);
    const bool slots = a.algo == 2;
    for (int64_t i = lo + tid; i < hi; i += nth) {
        float acc[V];
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] = 0.0f;
        uint4 raw[kMaxPeers];
#pragma unroll
        for (int q = 0; q < kMaxPeers; ++q)
            if (q < R)
                raw[q] = slots ? reinterpret_cast<const uint4 *>(P.arena[me] + a.stage_off + q * a.stage_bytes)[i - lo]
                               : reinterpret_cast<const uint4 *>(P.arena[q] + a.buf_off[q])[i];
#pragma unroll
        for (int q = 0; q < kMaxPeers; ++q)
            if (q < R) {
                const T *e = reinterpret_cast<const T *>(&raw[q]);
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] += to_f32(e[k]);
            }
        union { uint4 q; T e[V]; } o;
#pragma unroll
        for (int k = 0; k < V; ++k) o.e[k] = from_f32<T>(acc[k]);
#pragma unroll
        for (int q = 0; q < kMaxPeers; ++q)
            if (q < R) reinterpret_cast<uint4 *>(P.arena[q] + a.buf_off[q])[i] = o.q;
    }
}

__device__ void run_allreduce(const LaunchParams &P, const AllReduceArgs &a, int p, int Pn,
                                           unsigned long long iter_no) {
    switch (a.dtype) {
        case DT_F32: allreduce_typed<float>(P, a, p, Pn, iter_no); break;
        case DT_F16: allreduce_typed<__half>(P, a, p, Pn, iter_no); break;
        case DT_BF16: allreduce_typed<__nv_bfloat16>(P, a, p, Pn, iter_no); break;
        default: break;
    }
}

}  // namespace arkb
