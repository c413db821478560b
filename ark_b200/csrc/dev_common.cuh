// Device helpers shared by all op implementations of the loop kernel:
// typed 128-bit loads/stores with fp32 conversion, warp/CTA reductions,
// bounded waits and the device-scope barrier.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "program.h"

namespace arkb {

// ---- per-CTA control block in shared memory ---------------------------------
struct CtaCtl {
    int abort;        // set when any bounded wait in this CTA gave up
    int run_iters;    // broadcast of the run request
    uint32_t tmem_base;
    int pad;
};

__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void report(DeviceState *st, int code, int stage) {
    if (atomicCAS(&st->status, ST_OK, code) == ST_OK) {
        st->status_stage = stage;
        st->status_cta = blockIdx.x;
        if (st->host_status) *st->host_status = code;
    }
    __threadfence_system();
}

__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(unsigned long long *p, unsigned long long v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Asks the L2 to fetch [p, p + bytes) (16-byte aligned, a multiple of 16 bytes) from HBM; returns at once.
__device__ __forceinline__ void l2_prefetch(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Barrier over `count` CTAs on a monotonic counter: the k-th barrier of a
// group completes when the counter reaches k*count. Replaces the reference's
// sense-reversing sync_gpu (ark/include/kernels/common/sync.h:36-66); the wait
// is bounded (`spin_limit` nanoseconds) and reports instead of spinning forever.
// Returns false on abort.
// One thread waits until the counter reaches `target` (acquire); bounded.
__device__ __forceinline__ void counter_wait(unsigned long long *ctr, unsigned long long target, unsigned long long spin_limit,
                                             CtaCtl *ctl, DeviceState *st, int stage) {
    unsigned long long spins = 0, t0 = 0;
    while (ld_acquire_gpu(ctr) < target) {
        ++spins;
        if ((spins & 1023) == 0) {
            const unsigned long long now = globaltimer();
            if (t0 == 0) t0 = now;
            if (now - t0 > spin_limit) {
                ctl->abort = 1;
                report(st, ST_BARRIER_TIMEOUT, stage);
                break;
            }
        }
        if (spins > 64) __nanosleep(spins > 4096 ? 256 : 32);
    }
}

__device__ __forceinline__ bool grid_barrier(unsigned long long *ctr, unsigned long long target,
                                             unsigned long long spin_limit, CtaCtl *ctl, DeviceState *st,
                                             int stage) {
    __syncthreads();
    if (threadIdx.x == 0) {
        red_release_gpu_add(ctr, 1ull);
        counter_wait(ctr, target, spin_limit, ctl, st, stage);
    }
    __syncthreads();
    return ctl->abort == 0;
}

// ---- typed vector access -------------------------------------------------------
template <typename T>
struct VecOf {
    static constexpr int N = 16 / sizeof(T);
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(int32_t v) { return (float)v; }
__device__ __forceinline__ float to_f32(uint32_t v) { return (float)v; }
__device__ __forceinline__ float to_f32(int8_t v) { return (float)v; }
__device__ __forceinline__ float to_f32(uint8_t v) { return (float)v; }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ int32_t from_f32<int32_t>(float v) { return (int32_t)v; }
template <>
__device__ __forceinline__ uint32_t from_f32<uint32_t>(float v) { return (uint32_t)v; }
template <>
__device__ __forceinline__ int8_t from_f32<int8_t>(float v) { return (int8_t)v; }
template <>
__device__ __forceinline__ uint8_t from_f32<uint8_t>(float v) { return (uint8_t)v; }

// 16-byte global load that does not allocate a line in L1. The loop kernel gives
// almost all of the SM's L1/shared storage to shared memory, so the few L1 lines
// that are left would otherwise bound the number of loads in flight.
__device__ __forceinline__ uint4 ldg16_stream(const void *p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Load N consecutive elements (N*sizeof(T) is 4, 8, 16 or 32 bytes, address
// aligned to min(16, N*sizeof(T))) and widen to fp32.
template <typename T, int N>
__device__ __forceinline__ void load_vec(const T *p, float (&f)[N]) {
    constexpr int BYTES = N * sizeof(T);
    union {
        uint4 q[(BYTES + 15) / 16];
        T e[N];
    } u;
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) u.q[i] = ldg16_stream(reinterpret_cast<const uint4 *>(p) + i);
    } else if constexpr (BYTES == 8) {
        uint2 v = *reinterpret_cast<const uint2 *>(p);
        u.q[0].x = v.x;
        u.q[0].y = v.y;
    } else if constexpr (BYTES == 4) {
        u.q[0].x = *reinterpret_cast<const uint32_t *>(p);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) u.e[i] = p[i];
    }
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f32(u.e[i]);
}

// Same as load_vec but through L1: for small operands that are re-read many times
// (norm weights, broadcast rows).
template <typename T, int N>
__device__ __forceinline__ void load_vec_cached(const T *p, float (&f)[N]) {
    constexpr int BYTES = N * sizeof(T);
    union {
        uint4 q[(BYTES + 15) / 16];
        T e[N];
    } u;
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) u.q[i] = reinterpret_cast<const uint4 *>(p)[i];
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) u.e[i] = p[i];
    }
#pragma unroll
    for (int i = 0; i < N; ++i) f[i] = to_f32(u.e[i]);
}

template <typename T, int N>
__device__ __forceinline__ void store_vec(T *p, const float (&f)[N]) {
    constexpr int BYTES = N * sizeof(T);
    union {
        uint4 q[(BYTES + 15) / 16];
        T e[N];
    } u;
#pragma unroll
    for (int i = 0; i < N; ++i) u.e[i] = from_f32<T>(f[i]);
    if constexpr (BYTES >= 16) {
#pragma unroll
        for (int i = 0; i < BYTES / 16; ++i) reinterpret_cast<uint4 *>(p)[i] = u.q[i];
    } else if constexpr (BYTES == 8) {
        *reinterpret_cast<uint2 *>(p) = make_uint2(u.q[0].x, u.q[0].y);
    } else if constexpr (BYTES == 4) {
        *reinterpret_cast<uint32_t *>(p) = u.q[0].x;
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) p[i] = u.e[i];
    }
}

// Eight 16-bit elements held in one 16-byte register quad, widened to fp32.
template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &q, float (&f)[8]) {
    const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32(e[i]);
}

// Element offset of 4-D index (n,c,h,w) in a view.
__device__ __forceinline__ int64_t tref_off(const TRef &t, int64_t n, int64_t c, int64_t h, int64_t w) {
    return n * t.stride[0] + c * t.stride[1] + h * t.stride[2] + w * t.stride[3];
}

// ---- reductions -----------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Named barrier over a sub-group of warps of the CTA (ids 1..15; 0 is
// __syncthreads). Counterpart of the reference's sync_warps
// (ark/include/kernels/common/sync.h:80-104).
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// The tanh form of GeLU used by the reference (ark/include/kernels/math_functions.h:24-46,
// host baseline ark/ops/ops_math_test.cpp:10-12), evaluated in fp32.
__device__ __forceinline__ float gelu_f(float x) {
    // 0.5 * (1 + tanh(u)) == 1 / (1 + exp(-2u)): no cancellation in the negative tail
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    float u = k0 * (x + k1 * x * x * x);
    return x / (1.0f + expf(-2.0f * u));
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// Activations for 16-bit outputs (GEMM epilogue): hardware exp2 / reciprocal
// approximations, relative error ~1e-6, far below the storage rounding.
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float apply_act_fast(int act, float v) {
    switch (act) {
        case ACT_RELU: return fmaxf(v, 0.0f);
        case ACT_GELU: {
            const float k0 = 0.7978845608028654f, k1 = 0.044715f;
            const float u = k0 * (v + k1 * v * v * v);
            return v * fast_sigmoid(2.0f * u);
        }
        case ACT_SIGMOID: return fast_sigmoid(v);
        case ACT_SILU: return v * fast_sigmoid(v);
        default: return v;
    }
}

__device__ __forceinline__ float apply_act(int act, float v) {
    switch (act) {
        case ACT_RELU: return fmaxf(v, 0.0f);
        case ACT_GELU: return gelu_f(v);
        case ACT_SIGMOID: return sigmoid_f(v);
        case ACT_SILU: return v * sigmoid_f(v);
        default: return v;
    }
}

}  // namespace arkb
