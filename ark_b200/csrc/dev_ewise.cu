// Elementwise stages: unary math, binary arithmetic with NumPy broadcast,
// scalar ops, cast, copy and rope. One implementation replaces the
// reference's Broadcast1/Broadcast2 tile walkers
// (ark/include/kernels/common/broadcast.h:22-553, arithmetic.h, math_functions.h,
// cast.h, copy.h, scalar.h, embedding.h:14-37): every thread moves 128-bit
// vectors, the arithmetic is fp32 and the result is rounded once.
#include "dev_common.cuh"
#include "dev_funcs.h"

namespace arkb {

// FAST: results are rounded to a 16-bit type, so the hardware exp2 / reciprocal
// approximations (relative error ~1e-6) are used for gelu / sigmoid / silu.
template <int N, bool FAST>
__device__ __forceinline__ void ewise_math(int op, float scalar, const float (&x)[N], const float (&y)[N],
                                           float (&r)[N]) {
    switch (op) {
        case EW_GELU:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = FAST ? apply_act_fast(ACT_GELU, x[i]) : gelu_f(x[i]);
            break;
        case EW_EXP:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = expf(x[i]);
            break;
        case EW_RELU:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] > 0.0f ? x[i] : 0.0f;
            break;
        case EW_RSQRT:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = 1.0f / sqrtf(x[i]);
            break;
        case EW_SIGMOID:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = FAST ? fast_sigmoid(x[i]) : sigmoid_f(x[i]);
            break;
        case EW_SILU:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] * (FAST ? fast_sigmoid(x[i]) : sigmoid_f(x[i]));
            break;
        case EW_SQRT:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = sqrtf(x[i]);
            break;
        case EW_ADD:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] + y[i];
            break;
        case EW_SUB:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] - y[i];
            break;
        case EW_MUL:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] * y[i];
            break;
        case EW_DIV:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] / y[i];
            break;
        case EW_SCALAR_ASSIGN:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = scalar;
            break;
        case EW_SCALAR_ADD:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] + scalar;
            break;
        case EW_SCALAR_MUL:
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i] * scalar;
            break;
        case EW_ROPE:
            // complex multiply on adjacent pairs (ark/include/kernels/embedding.h:14-37)
            if constexpr (N >= 2) {
#pragma unroll
                for (int i = 0; i < N; i += 2) {
                    r[i] = x[i] * y[i] - x[i + 1] * y[i + 1];
                    r[i + 1] = x[i] * y[i + 1] + x[i + 1] * y[i];
                }
            }
            break;
        default:  // EW_COPY / EW_CAST
#pragma unroll
            for (int i = 0; i < N; ++i) r[i] = x[i];
            break;
    }
}

__device__ __forceinline__ bool ewise_is_binary(int op) { return (op >= EW_ADD && op <= EW_DIV) || op == EW_ROPE; }
__device__ __forceinline__ bool ewise_reads_in0(int op) { return op != EW_SCALAR_ASSIGN; }


// Same-type path: TIn == TOut, V elements per access.
template <typename TI, typename TO, int V>
__device__ void ewise_walk(const EwiseArgs &a, int p, int P) {
    const int op = a.op;
    const bool bin = ewise_is_binary(op);
    const bool rd0 = ewise_reads_in0(op);
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x;
    const int64_t nth = (int64_t)P * kThreads;
    TO *out = reinterpret_cast<TO *>(a.out.ptr);
    const TI *in0 = reinterpret_cast<const TI *>(a.in0.ptr);
    const TI *in1 = reinterpret_cast<const TI *>(a.in1.ptr);
    if (a.flat) {
        const int64_t n_units = a.n_units;
        const float scalar = a.scalar;
        if constexpr (V * sizeof(TI) == 16) {
            // 16-byte units kept packed in registers until they are consumed, so that eight
            // (unary) or six (binary) loads per operand are in flight per thread: with one
            // 512-thread CTA per SM the bytes in flight, not the issue rate, bound the bandwidth
            if (!bin) {
                constexpr int U = 8;
                for (int64_t u0 = tid; u0 < n_units; u0 += nth * U) {
                    uint4 rx[U];
#pragma unroll
                    for (int j = 0; j < U; ++j)
                        if (rd0 && u0 + j * nth < n_units) rx[j] = ldg16_stream(in0 + (u0 + j * nth) * V);
#pragma unroll
                    for (int j = 0; j < U; ++j) {
                        const int64_t u = u0 + j * nth;
                        if (u < n_units) {
                            float x[V], r[V];
                            const TI *e = reinterpret_cast<const TI *>(&rx[j]);
#pragma unroll
                            for (int i = 0; i < V; ++i) x[i] = to_f32(e[i]);
                            ewise_math<V, sizeof(TO) == 2>(op, scalar, x, x, r);
                            store_vec<TO, V>(out + u * V, r);
                        }
                    }
                }
            } else {
                constexpr int U = 6;
                for (int64_t u0 = tid; u0 < n_units; u0 += nth * U) {
                    uint4 rx[U], ry[U];
#pragma unroll
                    for (int j = 0; j < U; ++j)
                        if (u0 + j * nth < n_units) {
                            rx[j] = ldg16_stream(in0 + (u0 + j * nth) * V);
                            ry[j] = ldg16_stream(in1 + (u0 + j * nth) * V);
                        }
#pragma unroll
                    for (int j = 0; j < U; ++j) {
                        const int64_t u = u0 + j * nth;
                        if (u < n_units) {
                            float x[V], y[V], r[V];
                            const TI *ex = reinterpret_cast<const TI *>(&rx[j]);
                            const TI *ey = reinterpret_cast<const TI *>(&ry[j]);
#pragma unroll
                            for (int i = 0; i < V; ++i) {
                                x[i] = to_f32(ex[i]);
                                y[i] = to_f32(ey[i]);
                            }
                            ewise_math<V, sizeof(TO) == 2>(op, scalar, x, y, r);
                            store_vec<TO, V>(out + u * V, r);
                        }
                    }
                }
            }
            return;
        }
        for (int64_t u = tid; u < n_units; u += nth) {
            float x[V], y[V], r[V];
            if (rd0) load_vec<TI, V>(in0 + u * V, x);
            if (bin) load_vec<TI, V>(in1 + u * V, y);
            ewise_math<V, sizeof(TO) == 2>(op, scalar, x, y, r);
            store_vec<TO, V>(out + u * V, r);
        }
        return;
    }
    // strided / broadcast walk. The host has collapsed the dimensions, so the common
    // cases are two-dimensional ([rows, W]); index arithmetic is 32-bit whenever the unit
    // count allows it (64-bit division costs ~4x as many instructions).
    const int64_t n_units = a.n_units;
    const float scalar = a.scalar;
    const uint32_t WV = (uint32_t)((a.out.shape[3] + V - 1) / V), H = (uint32_t)a.out.shape[2], C = (uint32_t)a.out.shape[1];
    const bool two_d = a.out.shape[0] == 1 && a.out.shape[1] == 1 && n_units <= 0xffffffffll;
    const int64_t so2 = a.out.stride[2], s02 = a.in0.stride[2], s12 = a.in1.stride[2];
    const int64_t s03 = a.in0.stride[3], s13 = a.in1.stride[3];
    // an operand with a broadcast dimension is re-read many times: keep it in L1
    const bool bc0 = !(s02 && s03), bc1 = !(s12 && s13);
    constexpr int U = 4;
    for (int64_t u0 = tid; u0 < n_units; u0 += nth * U) {
        int64_t oo[U], o0[U], o1[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            const int64_t u = u0 + k * nth;
            if (two_d) {
                const uint32_t uu = (uint32_t)u;
                const uint32_t row = uu / WV;
                const int64_t w = (int64_t)(uu - row * WV) * V;
                oo[k] = row * so2 + w;
                o0[k] = row * s02 + (s03 ? w : 0);
                o1[k] = row * s12 + (s13 ? w : 0);
            } else {
                const int64_t wv = u % WV;
                int64_t row = u / WV;
                const int64_t h = row % H;
                row /= H;
                const int64_t c = row % C, n = row / C;
                const int64_t w = wv * V;
                oo[k] = tref_off(a.out, n, c, h, w);
                o0[k] = tref_off(a.in0, n, c, h, s03 ? w : 0);
                o1[k] = tref_off(a.in1, n, c, h, s13 ? w : 0);
            }
        }
        if constexpr (V * sizeof(TI) == 16) {
            // operands stay packed (one 16-byte register quad per unit) until they are used
            uint4 rx[U], ry[U];
            float sx[U], sy[U];
#pragma unroll
            for (int k = 0; k < U; ++k) {
                if (u0 + k * nth >= n_units) continue;
                if (rd0) {
                    if (!s03) sx[k] = to_f32(in0[o0[k]]);
                    else rx[k] = bc0 ? *reinterpret_cast<const uint4 *>(in0 + o0[k]) : ldg16_stream(in0 + o0[k]);
                }
                if (bin) {
                    if (!s13) sy[k] = to_f32(in1[o1[k]]);
                    else ry[k] = bc1 ? *reinterpret_cast<const uint4 *>(in1 + o1[k]) : ldg16_stream(in1 + o1[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < U; ++k) {
                if (u0 + k * nth >= n_units) continue;
                float x[V], y[V], r[V];
                const TI *ex = reinterpret_cast<const TI *>(&rx[k]);
                const TI *ey = reinterpret_cast<const TI *>(&ry[k]);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    x[i] = s03 ? to_f32(ex[i]) : sx[k];
                    y[i] = s13 ? to_f32(ey[i]) : sy[k];
                }
                ewise_math<V, sizeof(TO) == 2>(op, scalar, x, y, r);
                store_vec<TO, V>(out + oo[k], r);
            }
        } else {
#pragma unroll
            for (int k = 0; k < U; ++k) {
                if (u0 + k * nth >= n_units) continue;
                float x[V], y[V], r[V];
                if (rd0) load_vec_cached<TI, V>(in0 + o0[k], x);
                if (bin) load_vec_cached<TI, V>(in1 + o1[k], y);
                ewise_math<V, sizeof(TO) == 2>(op, scalar, x, y, r);
                store_vec<TO, V>(out + oo[k], r);
            }
        }
    }
}

template <typename TI, typename TO>
__device__ __forceinline__ void ewise_typed(const EwiseArgs &a, int p, int P) {
    constexpr int VS = 16 / (sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO));
    if (a.vec > 1)
        ewise_walk<TI, TO, VS>(a, p, P);
    else
        ewise_walk<TI, TO, 1>(a, p, P);
}

// Raw copy of integer data (no fp32 round trip): 16 or 1 bytes per access.
__device__ void ewise_bytes(const EwiseArgs &a, int p, int P, int esize, unsigned long long iter_no) {
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x;
    const int64_t nth = (int64_t)P * kThreads;
    const int64_t slot = a.iter_slots > 1 ? (int64_t)((iter_no - 1) % (unsigned long long)a.iter_slots) : 0;
    const char *in_base = reinterpret_cast<const char *>(a.in0.ptr) + slot * a.in_iter_bytes;
    char *out_base = reinterpret_cast<char *>(a.out.ptr) + slot * a.out_iter_bytes;
    if (a.flat && a.vec > 1) {
        const uint4 *s = reinterpret_cast<const uint4 *>(in_base);
        uint4 *d = reinterpret_cast<uint4 *>(out_base);
        const int64_t n = a.n_units;
        constexpr int U = 8;
        for (int64_t u0 = tid; u0 < n; u0 += nth * U) {
            uint4 r[U];
#pragma unroll
            for (int j = 0; j < U; ++j)
                if (u0 + j * nth < n) r[j] = ldg16_stream(s + u0 + j * nth);
#pragma unroll
            for (int j = 0; j < U; ++j)
                if (u0 + j * nth < n) d[u0 + j * nth] = r[j];
        }
        return;
    }
    // generic strided element copy
    const int64_t W = a.out.shape[3], H = a.out.shape[2], C = a.out.shape[1];
    const int64_t total = (int64_t)a.out.shape[0] * C * H * W;
    const char *s = in_base;
    char *d = out_base;
    for (int64_t i = tid; i < total; i += nth) {
        int64_t w = i % W, r = i / W;
        int64_t h = r % H;
        r /= H;
        int64_t c = r % C, n = r / C;
        int64_t so = tref_off(a.in0, n, c, h, w) * esize, dof = tref_off(a.out, n, c, h, w) * esize;
        for (int b = 0; b < esize; ++b) d[dof + b] = s[so + b];
    }
}

// Conversions between any two storage types go through one generic walker
// whose loads and stores dispatch on the runtime dtype (keeps the code size
// additive in the number of types instead of quadratic).
template <int V>
__device__ __forceinline__ void load_any(const void *base, int dt, int64_t e, float (&f)[V]) {
    switch (dt) {
        case DT_F32: load_vec<float, V>(reinterpret_cast<const float *>(base) + e, f); break;
        case DT_F16: load_vec<__half, V>(reinterpret_cast<const __half *>(base) + e, f); break;
        case DT_BF16: load_vec<__nv_bfloat16, V>(reinterpret_cast<const __nv_bfloat16 *>(base) + e, f); break;
        case DT_I32: load_vec<int32_t, V>(reinterpret_cast<const int32_t *>(base) + e, f); break;
        case DT_U32: load_vec<uint32_t, V>(reinterpret_cast<const uint32_t *>(base) + e, f); break;
        case DT_I8: load_vec<int8_t, V>(reinterpret_cast<const int8_t *>(base) + e, f); break;
        default: load_vec<uint8_t, V>(reinterpret_cast<const uint8_t *>(base) + e, f); break;
    }
}
template <int V>
__device__ __forceinline__ void store_any(void *base, int dt, int64_t e, const float (&f)[V]) {
    switch (dt) {
        case DT_F32: store_vec<float, V>(reinterpret_cast<float *>(base) + e, f); break;
        case DT_F16: store_vec<__half, V>(reinterpret_cast<__half *>(base) + e, f); break;
        case DT_BF16: store_vec<__nv_bfloat16, V>(reinterpret_cast<__nv_bfloat16 *>(base) + e, f); break;
        case DT_I32: store_vec<int32_t, V>(reinterpret_cast<int32_t *>(base) + e, f); break;
        case DT_U32: store_vec<uint32_t, V>(reinterpret_cast<uint32_t *>(base) + e, f); break;
        case DT_I8: store_vec<int8_t, V>(reinterpret_cast<int8_t *>(base) + e, f); break;
        default: store_vec<uint8_t, V>(reinterpret_cast<uint8_t *>(base) + e, f); break;
    }
}

template <int V>
__device__ void ewise_convert(const EwiseArgs &a, int p, int P) {
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x;
    const int64_t nth = (int64_t)P * kThreads;
    const int idt = a.in0.dtype, odt = a.out.dtype;
    if (a.flat) {
        for (int64_t u = tid; u < a.n_units; u += nth) {
            float x[V];
            load_any<V>(a.in0.ptr, idt, u * V, x);
            store_any<V>(a.out.ptr, odt, u * V, x);
        }
        return;
    }
    const int64_t WV = (a.out.shape[3] + V - 1) / V;
    const int64_t H = a.out.shape[2], C = a.out.shape[1];
    for (int64_t u = tid; u < a.n_units; u += nth) {
        int64_t wv = u % WV, row = u / WV;
        int64_t h = row % H;
        row /= H;
        int64_t c = row % C, n = row / C;
        float x[V];
        load_any<V>(a.in0.ptr, idt, tref_off(a.in0, n, c, h, wv * V), x);
        store_any<V>(a.out.ptr, odt, tref_off(a.out, n, c, h, wv * V), x);
    }
}

// The full walkers above keep many loads in flight and need most of the register file; a function that uses many
// registers saves and restores them on every call (they live in the caller's hands by the calling convention),
// which costs ~2 us per stage whatever the tensor size. Small problems (a few units per thread: decode) therefore
// take a walker written for few registers; the dispatcher itself stays tiny.
__device__ __noinline__ void ewise_heavy(const EwiseArgs &a, int p, int P, unsigned long long iter_no) {
    const int idt = (a.op == EW_SCALAR_ASSIGN) ? a.out.dtype : a.in0.dtype;
    if (a.op == EW_COPY && idt == a.out.dtype) {
        const int es = (idt == DT_F32 || idt == DT_I32 || idt == DT_U32) ? 4 : (idt == DT_F16 || idt == DT_BF16) ? 2 : 1;
        ewise_bytes(a, p, P, es, iter_no);
        return;
    }
    if (a.op == EW_CAST || idt != a.out.dtype) {
        // vector mode moves 4 elements per access (16 bytes of the widest type)
        if (a.vec > 1) ewise_convert<4>(a, p, P);
        else ewise_convert<1>(a, p, P);
        return;
    }
    switch (idt) {
        case DT_F32: ewise_typed<float, float>(a, p, P); break;
        case DT_F16: ewise_typed<__half, __half>(a, p, P); break;
        case DT_BF16: ewise_typed<__nv_bfloat16, __nv_bfloat16>(a, p, P); break;
        default: break;
    }
}

template <typename T, int V>
__device__ __forceinline__ void ewise_light_walk(const EwiseArgs &a, int p, int P) {
    const int op = a.op;
    const bool bin = ewise_is_binary(op), rd0 = ewise_reads_in0(op);
    T *out = reinterpret_cast<T *>(a.out.ptr);
    const T *in0 = reinterpret_cast<const T *>(a.in0.ptr);
    const T *in1 = reinterpret_cast<const T *>(a.in1.ptr);
    const int nth = P * kThreads;
    const int n_units = (int)a.n_units;
    const int WV = (a.out.shape[3] + V - 1) / V, H = a.out.shape[2], C = a.out.shape[1];
    for (int u = p * kThreads + threadIdx.x; u < n_units; u += nth) {
        int64_t oo, o0, o1;
        if (a.flat) {
            oo = o0 = o1 = (int64_t)u * V;
        } else {
            const int wv = u % WV;
            int row = u / WV;
            const int h = row % H;
            row /= H;
            const int c = row % C, n = row / C;
            const int w = wv * V;
            oo = tref_off(a.out, n, c, h, w);
            o0 = tref_off(a.in0, n, c, h, a.in0.stride[3] ? w : 0);
            o1 = tref_off(a.in1, n, c, h, a.in1.stride[3] ? w : 0);
        }
        float x[V], y[V], r[V];
        if (rd0) {
            if (a.flat || a.in0.stride[3]) load_vec_cached<T, V>(in0 + o0, x);
            else {
                const float s = to_f32(in0[o0]);
#pragma unroll
                for (int i = 0; i < V; ++i) x[i] = s;
            }
        }
        if (bin) {
            if (a.flat || a.in1.stride[3]) load_vec_cached<T, V>(in1 + o1, y);
            else {
                const float s = to_f32(in1[o1]);
#pragma unroll
                for (int i = 0; i < V; ++i) y[i] = s;
            }
        }
        ewise_math<V, sizeof(T) == 2>(op, a.scalar, x, y, r);
        store_vec<T, V>(out + oo, r);
    }
}

// Integer tensors: Add / Sub / Mul / Div and the scalar forms in the tensors' own arithmetic (wrapping, truncating
// division), never through fp32, so that results are exact over the whole range of the type.
template <typename T>
__device__ __forceinline__ T int_math(int op, T x, T y, T s) {
    switch (op) {
        case EW_ADD: return (T)(x + y);
        case EW_SUB: return (T)(x - y);
        case EW_MUL: return (T)(x * y);
        case EW_DIV: return y != 0 ? (T)(x / y) : (T)0;
        case EW_SCALAR_ASSIGN: return s;
        case EW_SCALAR_ADD: return (T)(x + s);
        case EW_SCALAR_MUL: return (T)(x * s);
        case EW_RELU: return x > 0 ? x : (T)0;
        default: return x;
    }
}

template <typename T>
__device__ __noinline__ void ewise_int(const EwiseArgs &a, int p, int P) {
    const int op = a.op;
    T *out = reinterpret_cast<T *>(a.out.ptr);
    const T *in0 = reinterpret_cast<const T *>(a.in0.ptr);
    const T *in1 = reinterpret_cast<const T *>(a.in1.ptr);
    const bool bin = ewise_is_binary(op), rd0 = ewise_reads_in0(op);
    const T s = (T)a.scalar;
    const int64_t W = a.out.shape[3], H = a.out.shape[2], C = a.out.shape[1];
    const int64_t total = (int64_t)a.out.shape[0] * C * H * W;
    for (int64_t i = (int64_t)p * kThreads + threadIdx.x; i < total; i += (int64_t)P * kThreads) {
        int64_t oo = i, o0 = i, o1 = i;
        if (!a.flat) {
            const int64_t w = i % W;
            int64_t r = i / W;
            const int64_t h = r % H;
            r /= H;
            const int64_t c = r % C, n = r / C;
            oo = tref_off(a.out, n, c, h, w);
            o0 = tref_off(a.in0, n, c, h, w);
            o1 = tref_off(a.in1, n, c, h, w);
        }
        out[oo] = int_math<T>(op, rd0 ? in0[o0] : (T)0, bin ? in1[o1] : (T)0, s);
    }
}

// Part of an operator's tasks only (see EwiseArgs::task_b): an element walk over the un-collapsed 4-D output
// that keeps the elements whose tile belongs to the task range. Correct for every operator and type; plans use
// partial ranges to spread one operator over several processor groups, each part is small.
__device__ __noinline__ void ewise_masked(const EwiseArgs &a, int p, int P) {
    const int op = a.op;
    const bool bin = ewise_is_binary(op), rd0 = ewise_reads_in0(op);
    const int idt = rd0 ? a.in0.dtype : a.out.dtype, odt = a.out.dtype;
    const bool integer = idt >= DT_I32 && idt == odt && op != EW_COPY && op != EW_CAST;
    const int64_t W = a.out.shape[3], H = a.out.shape[2], C = a.out.shape[1];
    const int64_t total = (int64_t)a.out.shape[0] * C * H * W;
    for (int64_t i = (int64_t)p * kThreads + threadIdx.x; i < total; i += (int64_t)P * kThreads) {
        const int64_t w = i % W;
        int64_t r = i / W;
        const int64_t h = r % H;
        r /= H;
        const int64_t c = r % C, n = r / C;
        const int64_t task = ((n * C + c) * a.tiles_h + h / a.tile_h) * a.tiles_w + w / a.tile_w;
        if (task < a.task_b || task >= a.task_e || (task - a.task_b) % a.task_s) continue;
        if (op == EW_ROPE && (w & 1)) continue;  // pairs are handled by their even element
        const int64_t oo = tref_off(a.out, n, c, h, w), o0 = tref_off(a.in0, n, c, h, w), o1 = tref_off(a.in1, n, c, h, w);
        if (integer) {
            switch (idt) {
                case DT_I32: {
                    auto *o = reinterpret_cast<int32_t *>(a.out.ptr);
                    o[oo] = int_math<int32_t>(op, rd0 ? reinterpret_cast<const int32_t *>(a.in0.ptr)[o0] : 0,
                                              bin ? reinterpret_cast<const int32_t *>(a.in1.ptr)[o1] : 0, (int32_t)a.scalar);
                    break;
                }
                case DT_U32: {
                    auto *o = reinterpret_cast<uint32_t *>(a.out.ptr);
                    o[oo] = int_math<uint32_t>(op, rd0 ? reinterpret_cast<const uint32_t *>(a.in0.ptr)[o0] : 0u,
                                               bin ? reinterpret_cast<const uint32_t *>(a.in1.ptr)[o1] : 0u, (uint32_t)a.scalar);
                    break;
                }
                case DT_I8: {
                    auto *o = reinterpret_cast<int8_t *>(a.out.ptr);
                    o[oo] = int_math<int8_t>(op, rd0 ? reinterpret_cast<const int8_t *>(a.in0.ptr)[o0] : (int8_t)0,
                                             bin ? reinterpret_cast<const int8_t *>(a.in1.ptr)[o1] : (int8_t)0, (int8_t)a.scalar);
                    break;
                }
                default: {
                    auto *o = reinterpret_cast<uint8_t *>(a.out.ptr);
                    o[oo] = int_math<uint8_t>(op, rd0 ? reinterpret_cast<const uint8_t *>(a.in0.ptr)[o0] : (uint8_t)0,
                                              bin ? reinterpret_cast<const uint8_t *>(a.in1.ptr)[o1] : (uint8_t)0, (uint8_t)a.scalar);
                    break;
                }
            }
            continue;
        }
        if (op == EW_ROPE) {  // complex multiply of the pair (w, w + 1)
            float xr[1], xi[1], yr[1], yi[1];
            load_any<1>(a.in0.ptr, idt, o0, xr);
            load_any<1>(a.in0.ptr, idt, o0 + a.in0.stride[3], xi);
            load_any<1>(a.in1.ptr, idt, o1, yr);
            load_any<1>(a.in1.ptr, idt, o1 + a.in1.stride[3], yi);
            const float re[1] = {xr[0] * yr[0] - xi[0] * yi[0]}, im[1] = {xr[0] * yi[0] + xi[0] * yr[0]};
            store_any<1>(a.out.ptr, odt, oo, re);
            store_any<1>(a.out.ptr, odt, oo + a.out.stride[3], im);
            continue;
        }
        float x[1] = {0.0f}, y[1] = {0.0f}, rr[1];
        if (rd0) load_any<1>(a.in0.ptr, idt, o0, x);
        if (bin) load_any<1>(a.in1.ptr, idt, o1, y);
        ewise_math<1, false>(op, a.scalar, x, y, rr);
        store_any<1>(a.out.ptr, odt, oo, rr);
    }
}

template <typename T>
__device__ __noinline__ void ewise_light(const EwiseArgs &a, int p, int P) {
    constexpr int VS = 16 / sizeof(T);
    if (a.vec > 1) ewise_light_walk<T, VS>(a, p, P);
    else ewise_light_walk<T, 1>(a, p, P);
}

__device__ __noinline__ void run_ewise(const EwiseArgs &a, int p, int P, unsigned long long iter_no) {
    if (a.task_s > 0) return ewise_masked(a, p, P);
    const int idt = (a.op == EW_SCALAR_ASSIGN) ? a.out.dtype : a.in0.dtype;
    if (idt == a.out.dtype && a.op != EW_COPY && a.op != EW_CAST && idt >= DT_I32) {
        switch (idt) {
            case DT_I32: ewise_int<int32_t>(a, p, P); return;
            case DT_U32: ewise_int<uint32_t>(a, p, P); return;
            case DT_I8: ewise_int<int8_t>(a, p, P); return;
            default: ewise_int<uint8_t>(a, p, P); return;
        }
    }
    const bool light = a.n_units <= (int64_t)4 * P * kThreads && idt == a.out.dtype && a.op != EW_COPY && a.op != EW_CAST &&
                       a.iter_slots <= 1;
    if (light) {
        switch (idt) {
            case DT_F32: ewise_light<float>(a, p, P); return;
            case DT_F16: ewise_light<__half>(a, p, P); return;
            case DT_BF16: ewise_light<__nv_bfloat16>(a, p, P); return;
            default: break;
        }
    }
    ewise_heavy(a, p, P, iter_no);
}

}  // namespace arkb
