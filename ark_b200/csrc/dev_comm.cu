// Data movers of the in-kernel communication layer (see dev_comm.cuh).
#include "dev_comm.cuh"

namespace arkb {

// Dense byte copy local -> peer by all CTAs of the stage.
__device__ __noinline__ void run_put(const PutArgs &a, int p, int P, unsigned long long iter_no) {
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x, nth = (int64_t)P * kThreads;
    const int64_t slot = a.iter_slots > 1 ? (int64_t)((iter_no - 1) % (unsigned long long)a.iter_slots) : 0;
    const char *s = reinterpret_cast<const char *>(a.src) + slot * a.src_iter_bytes;
    char *d = reinterpret_cast<char *>(a.dst);
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d) | (uintptr_t)a.bytes) & 15) == 0) {
        const int64_t n = a.bytes / 16;
        for (int64_t i = tid; i < n; i += nth) reinterpret_cast<uint4 *>(d)[i] = reinterpret_cast<const uint4 *>(s)[i];
    } else {
        for (int64_t i = tid; i < a.bytes; i += nth) d[i] = s[i];
    }
}

// ---- NVSwitch multicast (NVLS) -------------------------------------------------------------------------
// One 16-byte vector summed over the copies that all ranks hold at this multicast address (fp32 accumulation in the
// switch for the 16-bit types), and one 16-byte store that lands in every rank's copy.
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce_add(const void *mc);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<__half>(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<__nv_bfloat16>(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce_add<float>(const void *mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
}
__device__ __forceinline__ void multimem_st16(void *mc, const uint4 &v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

template <typename T>
__device__ void allreduce_typed(const LaunchParams &P, const AllReduceArgs &a, int p, int Pn, unsigned long long iter_no) {
    constexpr int V = 16 / sizeof(T);
    const int R = P.nranks, me = P.rank;
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x, nth = (int64_t)Pn * kThreads;
    const int64_t nv = a.nelem / V;  // host guarantees nelem % V == 0 and 16-byte alignment
    if (a.algo == 3) {
        // the tensor sits at the same offset in every rank's arena (checked by the host): one multicast address
        char *mc = P.mc_arena + a.buf_off[me];
        const int64_t per = (nv + R - 1) / R;
        const int64_t lo = per * me, hi = min(nv, lo + per);
        for (int64_t i = lo + tid; i < hi; i += nth) {
            const uint4 v = multimem_ld_reduce_add<T>(mc + i * 16);
            multimem_st16(mc + i * 16, v);
        }
        return;
    }
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
        if (a.no_gather) {
            reinterpret_cast<uint4 *>(P.arena[me] + a.buf_off[me])[i] = o.q;
            continue;
        }
        if (a.mc_store) {  // one store, replicated by the switch into every rank's tensor
            multimem_st16(P.mc_arena + a.buf_off[me] + i * 16, o.q);
            continue;
        }
#pragma unroll
        for (int q = 0; q < kMaxPeers; ++q)
            if (q < R) reinterpret_cast<uint4 *>(P.arena[q] + a.buf_off[q])[i] = o.q;
    }
}

// ---- packets ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t packet_flag(uint32_t flag, unsigned long long iter_no) {
    return (uint32_t)((iter_no & 0xffffffull) << 8) | (flag & 0xffu);  // iter_no >= 1: never 0, the value of untouched memory
}
__device__ __forceinline__ void st_packet(void *p, uint32_t d0, uint32_t d1, uint32_t f) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(f), "r"(d1), "r"(f) : "memory");
}
// Polls one packet until both flag words carry `f`; false when the wait limit ran out.
__device__ __forceinline__ bool ld_packet(const void *p, uint32_t f, unsigned long long limit, uint32_t &d0, uint32_t &d1) {
    unsigned long long spins = 0, t0 = 0;
    for (;;) {
        uint32_t a, b, c, d;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(p) : "memory");
        if (b == f && d == f) {
            d0 = a;
            d1 = c;
            return true;
        }
        if ((++spins & 255) == 0) {
            const unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit) return false;
        }
        if (spins > 16) __nanosleep(64);
    }
}

__device__ __noinline__ void run_packet(const LaunchParams &P, const PacketArgs &a, int p, int Pn, unsigned long long iter_no, CtaCtl *ctl, int stage) {
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x, nth = (int64_t)Pn * kThreads;
    const int64_t n = a.payload_bytes / 8;
    const uint32_t f = packet_flag(a.flag, iter_no);
    if (!a.get) {
        const uint2 *src = reinterpret_cast<const uint2 *>(a.src);
        uint4 *dst = reinterpret_cast<uint4 *>(a.dst);
        for (int64_t i = tid; i < n; i += nth) {
            const uint2 v = src[i];
            st_packet(dst + i, v.x, v.y, f);
        }
        return;
    }
    const uint4 *src = reinterpret_cast<const uint4 *>(a.src);
    uint2 *dst = reinterpret_cast<uint2 *>(a.dst);
    bool ok = true;
    for (int64_t i = tid; i < n && ok; i += nth) {
        uint2 v;
        ok = ld_packet(src + i, f, P.spin_limit, v.x, v.y);
        if (ok) dst[i] = v;
    }
    if (!ok) {
        ctl->abort = 1;
        report(P.state, ST_PEER_TIMEOUT, stage);
    }
}

template <typename T>
__device__ void packet_reduce_typed(const LaunchParams &P, const PacketReduceArgs &a, int p, int Pn, unsigned long long iter_no, CtaCtl *ctl,
                                    int stage) {
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x, nth = (int64_t)Pn * kThreads;
    const T *in = reinterpret_cast<const T *>(a.in);
    T *out = reinterpret_cast<T *>(a.out);
    if (a.packets) {
        constexpr int V = 8 / sizeof(T);  // elements in one packet's payload
        const int64_t n = a.nelem / V;
        const uint32_t f = packet_flag(a.flag, iter_no);
        const uint4 *scratch = reinterpret_cast<const uint4 *>(a.scratch);
        bool ok = true;
        for (int64_t i = tid; i < n && ok; i += nth) {
            float acc[V];
            load_vec<T, V>(in + i * V, acc);
            for (int q = 0; q < a.npeers && ok; ++q) {
                union { uint2 u; T e[V]; } v;
                ok = ld_packet(scratch + (int64_t)q * n + i, f, P.spin_limit, v.u.x, v.u.y);
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] += to_f32(v.e[k]);
            }
            if (!ok) break;
            union { uint2 u; T e[V]; } o;
#pragma unroll
            for (int k = 0; k < V; ++k) o.e[k] = from_f32<T>(acc[k]);
            *reinterpret_cast<uint2 *>(out + i * V) = o.u;
            for (int q = 0; q < a.npeers; ++q) st_packet(reinterpret_cast<uint4 *>(a.peer_out[q]) + i, o.u.x, o.u.y, f);
        }
        if (!ok) {
            ctl->abort = 1;
            report(P.state, ST_PEER_TIMEOUT, stage);
        }
        return;
    }
    constexpr int V = 16 / sizeof(T);
    const int64_t n = a.nelem / V;
    const T *scratch = reinterpret_cast<const T *>(a.scratch);
    for (int64_t i = tid; i < n; i += nth) {
        float acc[V];
        load_vec<T, V>(in + i * V, acc);
        for (int q = 0; q < a.npeers; ++q) {
            float x[V];
            load_vec<T, V>(scratch + (int64_t)q * a.nelem + i * V, x);
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] += x[k];
        }
        union { uint4 u; T e[V]; } o;
#pragma unroll
        for (int k = 0; k < V; ++k) o.e[k] = from_f32<T>(acc[k]);
        reinterpret_cast<uint4 *>(out)[i] = o.u;
        for (int q = 0; q < a.npeers; ++q) reinterpret_cast<uint4 *>(a.peer_out[q])[i] = o.u;
    }
}

__device__ __noinline__ void run_packet_reduce(const LaunchParams &P, const PacketReduceArgs &a, int p, int Pn, unsigned long long iter_no, CtaCtl *ctl,
                                  int stage) {
    switch (a.dtype) {
        case DT_F32: packet_reduce_typed<float>(P, a, p, Pn, iter_no, ctl, stage); break;
        case DT_F16: packet_reduce_typed<__half>(P, a, p, Pn, iter_no, ctl, stage); break;
        case DT_BF16: packet_reduce_typed<__nv_bfloat16>(P, a, p, Pn, iter_no, ctl, stage); break;
        default: break;
    }
}

__device__ __noinline__ void run_allreduce(const LaunchParams &P, const AllReduceArgs &a, int p, int Pn,
                                           unsigned long long iter_no) {
    switch (a.dtype) {
        case DT_F32: allreduce_typed<float>(P, a, p, Pn, iter_no); break;
        case DT_F16: allreduce_typed<__half>(P, a, p, Pn, iter_no); break;
        case DT_BF16: allreduce_typed<__nv_bfloat16>(P, a, p, Pn, iter_no); break;
        default: break;
    }
}

}  // namespace arkb
