// Reductions and fused row operators.
//
// reduce along the last axis  : one warp per row, 128-bit loads, fp32
//                               accumulation, shuffle tree (replaces WwiseReduce,
//                               ark/include/kernels/reduce.h:341-444);
// reduce along another axis   : each thread owns a vector of consecutive
//                               outputs along W and walks the axis (replaces
//                               EwiseReduce, reduce.h:196-338);
// rmsnorm / layernorm / softmax: single-pass row kernels standing in for the
//                               op chains the reference composes in Python
//                               (python/ark/ops.py:491-513,
//                               examples/llama/model.py:92-99).
#include <type_traits>

#include "dev_common.cuh"
#include "dev_gemm.cuh"  // mbarrier and bulk-copy helpers
#include "dev_funcs.h"

namespace arkb {

template <typename T, int V>
__device__ void reduce_last_axis(const ReduceArgs &a, int p, int P) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int WPC = kThreads / 32;
    const int64_t W = a.in.shape[3];
    const int64_t H = a.in.shape[2], C = a.in.shape[1];
    const int64_t rows = (int64_t)a.in.shape[0] * C * H;
    const T *in = reinterpret_cast<const T *>(a.in.ptr);
    T *out = reinterpret_cast<T *>(a.out.ptr);
    const int op = a.op;
    const int64_t nv = W / V;
    if constexpr (V * sizeof(T) == 16) {
        // A warp walks its rows in steps of U 16-byte vectors per lane. Two register buffers alternate: the loads
        // of step t+1 are issued before step t is consumed, across row boundaries too, so the row-end shuffle
        // reduction never leaves the memory pipe empty.
        constexpr int U = 8;
        const int steps = (int)((nv + 32 * U - 1) / (32 * U));
        const int64_t row_step = (int64_t)P * WPC;
        struct Cursor {
            int64_t row;
            int j;
        };
        auto valid = [&](const Cursor &c) { return c.row < rows; };
        auto advance = [&](Cursor &c) {
            if (++c.j == steps) {
                c.j = 0;
                c.row += row_step;
            }
        };
        auto row_ptr = [&](int64_t row, int64_t &n, int64_t &c, int64_t &h) -> const T * {
            h = row % H;
            const int64_t r = row / H;
            c = r % C;
            n = r / C;
            return in + tref_off(a.in, n, c, h, 0);
        };
        auto issue = [&](uint4 (&buf)[U], const Cursor &cu) {
            int64_t n, c, h;
            const T *src = row_ptr(cu.row, n, c, h);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t v = lane + 32 * ((int64_t)cu.j * U + u);
                if (v < nv) buf[u] = ldg16_stream(src + v * V);
            }
        };
        float acc = (op == RD_MAX) ? -3.402823466e+38f : 0.0f;
        auto consume = [&](uint4 (&buf)[U], const Cursor &cu) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t v = lane + 32 * ((int64_t)cu.j * U + u);
                if (v < nv) {
                    const T *e = reinterpret_cast<const T *>(&buf[u]);
#pragma unroll
                    for (int i = 0; i < V; ++i) acc = (op == RD_MAX) ? fmaxf(acc, to_f32(e[i])) : acc + to_f32(e[i]);
                }
            }
            if (cu.j == steps - 1) {  // the row is complete
                int64_t n, c, h;
                const T *src = row_ptr(cu.row, n, c, h);
                for (int64_t w = nv * V + lane; w < W; w += 32) {
                    const float x = to_f32(src[w]);
                    acc = (op == RD_MAX) ? fmaxf(acc, x) : acc + x;
                }
                acc = (op == RD_MAX) ? warp_max(acc) : warp_sum(acc);
                if (op == RD_MEAN) acc /= (float)W;
                if (lane == 0) out[tref_off(a.out, n, c, h, 0)] = from_f32<T>(acc);
                acc = (op == RD_MAX) ? -3.402823466e+38f : 0.0f;
            }
        };
        if (steps == 0) {  // rows shorter than one vector: scalar path below handles them
        } else {
            Cursor ld{(int64_t)p * WPC + warp, 0}, cp = ld;
            uint4 qa[U], qb[U];
            if (valid(ld)) {
                issue(qa, ld);
                advance(ld);
            }
            while (valid(cp)) {
                if (valid(ld)) {
                    issue(qb, ld);
                    advance(ld);
                }
                consume(qa, cp);
                advance(cp);
                if (!valid(cp)) break;
                if (valid(ld)) {
                    issue(qa, ld);
                    advance(ld);
                }
                consume(qb, cp);
                advance(cp);
            }
            return;
        }
    }
    for (int64_t row = (int64_t)p * WPC + warp; row < rows; row += (int64_t)P * WPC) {
        int64_t h = row % H, r = row / H;
        int64_t c = r % C, n = r / C;
        const T *src = in + tref_off(a.in, n, c, h, 0);
        float acc = (op == RD_MAX) ? -3.402823466e+38f : 0.0f;
        for (int64_t v0 = lane; v0 < nv; v0 += 32) {
            float x[V];
            load_vec<T, V>(src + v0 * V, x);
#pragma unroll
            for (int i = 0; i < V; ++i) acc = (op == RD_MAX) ? fmaxf(acc, x[i]) : acc + x[i];
        }
        for (int64_t w = nv * V + lane; w < W; w += 32) {
            float x = to_f32(src[w]);
            acc = (op == RD_MAX) ? fmaxf(acc, x) : acc + x;
        }
        acc = (op == RD_MAX) ? warp_max(acc) : warp_sum(acc);
        if (op == RD_MEAN) acc /= (float)W;
        if (lane == 0) out[tref_off(a.out, n, c, h, 0)] = from_f32<T>(acc);
    }
}

template <typename T, int V>
__device__ void reduce_other_axis(const ReduceArgs &a, int p, int P, float *red) {
    const int ax = a.axis;
    int32_t osh[4] = {a.in.shape[0], a.in.shape[1], a.in.shape[2], a.in.shape[3]};
    const int64_t len = osh[ax];
    osh[ax] = 1;
    const int64_t WV = (osh[3] + V - 1) / V;
    const int64_t units = (int64_t)osh[0] * osh[1] * osh[2] * WV;
    const T *in = reinterpret_cast<const T *>(a.in.ptr);
    T *out = reinterpret_cast<T *>(a.out.ptr);
    const int64_t astr = a.in.stride[ax];
    const int op = a.op;
    // With fewer output vectors than threads, S threads of a CTA share one output vector: each walks 1/S of the
    // reduced axis and the partial results are added through shared memory (segment order: deterministic).
    int S = 1;
    while (S < 16 && units * S * 2 <= (int64_t)P * kThreads && len / (S * 2) >= 16) S *= 2;
    const int UPB = kThreads / S;  // output vectors per CTA pass
    const int ul = threadIdx.x % UPB, seg = threadIdx.x / UPB;
    const int64_t k_lo = len * seg / S, k_hi = len * (seg + 1) / S;
    for (int64_t ub = (int64_t)p * UPB; ub < units; ub += (int64_t)P * UPB) {
        const int64_t u = ub + ul;
        const bool live = u < units;
        int64_t wv = u % WV, r = u / WV;
        int64_t h = r % osh[2];
        r /= osh[2];
        int64_t c = r % osh[1], n = r / osh[1];
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = (op == RD_MAX) ? -3.402823466e+38f : 0.0f;
        if (live) {
            const T *src = in + tref_off(a.in, n, c, h, wv * V);
            constexpr int U = 8;  // independent loads in flight along the reduced axis
            int64_t k = k_lo;
            for (; k + U <= k_hi; k += U) {
                float x[U][V];
#pragma unroll
                for (int j = 0; j < U; ++j) load_vec<T, V>(src + (k + j) * astr, x[j]);
#pragma unroll
                for (int j = 0; j < U; ++j) {
#pragma unroll
                    for (int i = 0; i < V; ++i) acc[i] = (op == RD_MAX) ? fmaxf(acc[i], x[j][i]) : acc[i] + x[j][i];
                }
            }
            for (; k < k_hi; ++k) {
                float x[V];
                load_vec<T, V>(src + k * astr, x);
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = (op == RD_MAX) ? fmaxf(acc[i], x[i]) : acc[i] + x[i];
            }
        }
        if (S > 1) {
            __syncthreads();  // the previous pass no longer reads `red`
            if (seg > 0) {
#pragma unroll
                for (int i = 0; i < V; ++i) red[((size_t)seg * UPB + ul) * V + i] = acc[i];
            }
            __syncthreads();
            if (seg == 0) {
                for (int sg = 1; sg < S; ++sg) {
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        const float x = red[((size_t)sg * UPB + ul) * V + i];
                        acc[i] = (op == RD_MAX) ? fmaxf(acc[i], x) : acc[i] + x;
                    }
                }
            }
        }
        if (live && seg == 0) {
            if (op == RD_MEAN) {
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] /= (float)len;
            }
            store_vec<T, V>(out + tref_off(a.out, n, c, h, wv * V), acc);
        }
    }
}

// A subset of the outputs (a plan's partial task range): one warp per output element, the lanes stride along the
// reduced axis, a shuffle tree adds the partial results (fixed order: deterministic).
template <typename T>
__device__ void reduce_tasks(const ReduceArgs &a, int p, int P) {
    constexpr int WPC = kThreads / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t osh[4] = {a.in.shape[0], a.in.shape[1], a.in.shape[2], a.in.shape[3]};
    const int64_t len = osh[a.axis];
    osh[a.axis] = 1;
    const int64_t astr = a.in.stride[a.axis];
    const T *in = reinterpret_cast<const T *>(a.in.ptr);
    T *out = reinterpret_cast<T *>(a.out.ptr);
    const int64_t n_tasks = a.task_e > a.task_b ? (a.task_e - a.task_b + a.task_s - 1) / a.task_s : 0;
    for (int64_t k = (int64_t)p * WPC + warp; k < n_tasks; k += (int64_t)P * WPC) {
        int64_t r = a.task_b + k * a.task_s;
        const int64_t w = r % osh[3];
        r /= osh[3];
        const int64_t h = r % osh[2];
        r /= osh[2];
        const int64_t c = r % osh[1], n = r / osh[1];
        if (n >= osh[0]) continue;
        const T *src = in + tref_off(a.in, n, c, h, w);
        float acc = (a.op == RD_MAX) ? -3.402823466e+38f : 0.0f;
        for (int64_t i = lane; i < len; i += 32) {
            const float v = to_f32(src[i * astr]);
            acc = (a.op == RD_MAX) ? fmaxf(acc, v) : acc + v;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, acc, o);
            acc = (a.op == RD_MAX) ? fmaxf(acc, other) : acc + other;
        }
        if (lane == 0) out[tref_off(a.out, n, c, h, w)] = from_f32<T>(a.op == RD_MEAN ? acc / (float)len : acc);
    }
}

template <typename T>
__device__ __forceinline__ void reduce_typed(const ReduceArgs &a, int p, int P, float *red) {
    constexpr int V = 16 / sizeof(T);
    if (a.partial) return reduce_tasks<T>(a, p, P);
    if (a.axis == 3) {
        if (a.vec > 1) reduce_last_axis<T, V>(a, p, P);
        else reduce_last_axis<T, 1>(a, p, P);
    } else {
        if (a.vec > 1) reduce_other_axis<T, V>(a, p, P, red);
        else reduce_other_axis<T, 1>(a, p, P, red);
    }
}

__device__ __noinline__ void run_reduce(const ReduceArgs &a, int p, int P, char *smem) {
    float *red = reinterpret_cast<float *>(smem);  // kThreads x 8 floats at most
    switch (a.in.dtype) {
        case DT_F32: reduce_typed<float>(a, p, P, red); break;
        case DT_F16: reduce_typed<__half>(a, p, P, red); break;
        case DT_BF16: reduce_typed<__nv_bfloat16>(a, p, P, red); break;
        default: break;
    }
}

// ---- fused row operators --------------------------------------------------------
// One warp per row. Pass 1 accumulates the row statistics in fp32, pass 2
// re-reads the row (it is still in L2) and writes the result: HBM sees one
// read and one write per element.
// The scale row of a norm: in the rows' own type, or fp32 when the model keeps it so.
template <typename T, int V>
__device__ __forceinline__ void load_row_weight(const RowOpArgs &a, int64_t e, float (&g)[V]) {
    if (a.weight_f32) load_vec_cached<float, V>(reinterpret_cast<const float *>(a.weight) + e, g);
    else load_vec_cached<T, V>(reinterpret_cast<const T *>(a.weight) + e, g);
}

template <typename T>
__device__ __noinline__ void rowop_typed(const RowOpArgs &a, int p, int P) {
    constexpr int V = 16 / sizeof(T);
    constexpr int WPC = kThreads / 32;
    constexpr int U = 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t cols = a.cols;
    const int64_t nv = cols / V;  // host guarantees cols % V == 0 and 16-byte aligned rows
    const T *wgt = reinterpret_cast<const T *>(a.weight);
    const int op = a.op;
    const T *mask = reinterpret_cast<const T *>(a.mask);
    const float scale = (op == RO_SOFTMAX && !mask) ? a.scale : 1.0f;
    for (int64_t row = (int64_t)p * WPC + warp; row < a.rows; row += (int64_t)P * WPC) {
        const T *src = reinterpret_cast<const T *>(a.in) + row * a.in_ld;
        T *dst = reinterpret_cast<T *>(a.out) + row * a.out_ld;
        if (mask) {
            // masked softmax: the logits x * scale + mask are formed first, rounded to the storage type, in the output row
            const T *mk = mask + (row % a.mask_rows) * a.mask_ld;
            for (int64_t v = lane; v < nv; v += 32) {
                float f[V], g[V];
                load_vec<T, V>(src + v * V, f);
                load_vec_cached<T, V>(mk + v * V, g);
#pragma unroll
                for (int i = 0; i < V; ++i) f[i] = f[i] * a.scale + g[i];
                store_vec<T, V>(dst + v * V, f);
            }
            __syncwarp();
            src = dst;
        }
        if (a.residual) {
            // x := x + residual, rounded to the storage type and kept (res_out) for the next block
            const T *res = reinterpret_cast<const T *>(a.residual) + row * a.in_ld;
            T *rout = reinterpret_cast<T *>(a.res_out) + row * a.in_ld;
            for (int64_t v = lane; v < nv; v += 32) {
                float f[V], g[V];
                load_vec<T, V>(src + v * V, f);
                load_vec<T, V>(res + v * V, g);
#pragma unroll
                for (int i = 0; i < V; ++i) f[i] += g[i];
                store_vec<T, V>(rout + v * V, f);
            }
            __syncwarp();
            src = rout;
        }
        float s1 = 0.0f, s2 = 0.0f, mx = -3.402823466e+38f;
        for (int64_t v0 = lane; v0 < nv; v0 += 32 * U) {
            float x[U][V];
#pragma unroll
            for (int j = 0; j < U; ++j)
                if (v0 + j * 32 < nv) load_vec<T, V>(src + (v0 + j * 32) * V, x[j]);
#pragma unroll
            for (int j = 0; j < U; ++j)
                if (v0 + j * 32 < nv) {
#pragma unroll
                    for (int i = 0; i < V; ++i) {
                        const float e = x[j][i] * scale;
                        s1 += e;
                        s2 += e * e;
                        mx = fmaxf(mx, e);
                    }
                }
        }
        float mul = 1.0f, sub = 0.0f;
        if (op == RO_RMSNORM) {
            s2 = warp_sum(s2);
            mul = 1.0f / sqrtf(s2 / (float)cols + a.eps);
        } else if (op == RO_LAYERNORM) {
            s1 = warp_sum(s1);
            const float mean = s1 / (float)cols;
            float var = 0.0f;
            for (int64_t v = lane; v < nv; v += 32) {
                float f[V];
                load_vec<T, V>(src + v * V, f);
#pragma unroll
                for (int i = 0; i < V; ++i) var += (f[i] - mean) * (f[i] - mean);
            }
            var = warp_sum(var);
            mul = 1.0f / sqrtf(var / (float)cols + a.eps);
            sub = mean;
        } else {
            mx = warp_max(mx);
            float se = 0.0f;
            for (int64_t v = lane; v < nv; v += 32) {
                float f[V];
                load_vec<T, V>(src + v * V, f);
#pragma unroll
                for (int i = 0; i < V; ++i) se += expf(f[i] * scale - mx);
            }
            se = warp_sum(se);
            mul = 1.0f / se;
        }
        for (int64_t v = lane; v < nv; v += 32) {
            float f[V];
            load_vec<T, V>(src + v * V, f);
            if (op == RO_SOFTMAX) {
#pragma unroll
                for (int i = 0; i < V; ++i) f[i] = expf(f[i] * scale - mx) * mul;
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) f[i] = (f[i] - sub) * mul;
                if (wgt) {
                    float g[V];
                    load_row_weight<T, V>(a, (int64_t)v * V, g);
#pragma unroll
                    for (int i = 0; i < V; ++i) f[i] *= g[i];
                }
            }
            store_vec<T, V>(dst + v * V, f);
        }
    }
}

// Single-read variant: G warps share a row and keep it packed in registers
// (at most 8 16-byte vectors per lane); cross-warp sums go through a few floats
// of shared memory and a named barrier per warp group. HBM sees exactly one
// read and one write per element.
template <typename T>
__device__ __noinline__ void rowop_regs(const RowOpArgs &a, int p, int P, const int G) {
    constexpr int V = 16 / sizeof(T);
    constexpr int MAXV = 8;
    constexpr int WPC = kThreads / 32;
    __shared__ float red[4][WPC];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = warp / G, wig = warp % G, groups = WPC / G;
    const int li = wig * 32 + lane, lstride = 32 * G;
    const int64_t cols = a.cols, nv = cols / V;
    const int op = a.op;
    const T *mask = reinterpret_cast<const T *>(a.mask);
    const float scale = (op == RO_SOFTMAX && !mask) ? a.scale : 1.0f;
    const float pre_scale = a.scale;
    const int64_t mask_ld = a.mask_ld, mask_rows = a.mask_rows;
    const T *wgt = reinterpret_cast<const T *>(a.weight);
    const int64_t in_ld = a.in_ld, out_ld = a.out_ld, rows = a.rows;
    const float eps = a.eps, inv_cols = 1.0f / (float)cols;
    const T *in = reinterpret_cast<const T *>(a.in);
    const T *resid = reinterpret_cast<const T *>(a.residual);
    T *res_out = reinterpret_cast<T *>(a.res_out);
    T *out = reinterpret_cast<T *>(a.out);
    auto group_sum = [&](float v, int slot, bool is_max) -> float {
        v = is_max ? warp_max(v) : warp_sum(v);
        if (G == 1) return v;
        if (lane == 0) red[slot][warp] = v;
        named_barrier(1 + group, G * 32);
        float r = red[slot][group * G];
        for (int i = 1; i < G; ++i) r = is_max ? fmaxf(r, red[slot][group * G + i]) : r + red[slot][group * G + i];
        return r;
    };
    unsigned it = 0;
    for (int64_t row = (int64_t)p * groups + group; row < rows; row += (int64_t)P * groups, ++it) {
        const T *src = in + row * in_ld;
        uint4 rx[MAXV];
#pragma unroll
        for (int j = 0; j < MAXV; ++j)
            if (li + j * lstride < nv) rx[j] = ldg16_stream(src + (int64_t)(li + j * lstride) * V);
        if (resid) {
            const T *rs = resid + row * in_ld;
            T *ro = res_out + row * in_ld;
#pragma unroll
            for (int j = 0; j < MAXV; ++j)
                if (li + j * lstride < nv) {
                    const uint4 g4 = ldg16_stream(rs + (int64_t)(li + j * lstride) * V);
                    T *e = reinterpret_cast<T *>(&rx[j]);
                    const T *ge = reinterpret_cast<const T *>(&g4);
#pragma unroll
                    for (int i = 0; i < V; ++i) e[i] = from_f32<T>(to_f32(e[i]) + to_f32(ge[i]));
                    *reinterpret_cast<uint4 *>(ro + (int64_t)(li + j * lstride) * V) = rx[j];
                }
        }
        if (mask) {
            // masked softmax: logits x * scale + mask, rounded to the storage type, replace the row in registers
            const T *mk = mask + (row % mask_rows) * mask_ld;
#pragma unroll
            for (int j = 0; j < MAXV; ++j)
                if (li + j * lstride < nv) {
                    const uint4 g4 = *reinterpret_cast<const uint4 *>(mk + (int64_t)(li + j * lstride) * V);
                    T *e = reinterpret_cast<T *>(&rx[j]);
                    const T *ge = reinterpret_cast<const T *>(&g4);
#pragma unroll
                    for (int i = 0; i < V; ++i) e[i] = from_f32<T>(to_f32(e[i]) * pre_scale + to_f32(ge[i]));
                }
        }
        float s1 = 0.0f, s2 = 0.0f, mx = -3.402823466e+38f;
#pragma unroll
        for (int j = 0; j < MAXV; ++j)
            if (li + j * lstride < nv) {
                const T *e = reinterpret_cast<const T *>(&rx[j]);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float x = to_f32(e[i]) * scale;
                    s1 += x;
                    s2 += x * x;
                    mx = fmaxf(mx, x);
                }
            }
        const int slot = (it & 1) * 2;
        float mul = 1.0f, sub = 0.0f;
        if (op == RO_RMSNORM) {
            s2 = group_sum(s2, slot, false);
            mul = 1.0f / sqrtf(s2 * inv_cols + eps);
        } else if (op == RO_LAYERNORM) {
            const float mean = group_sum(s1, slot, false) * inv_cols;
            float var = 0.0f;
#pragma unroll
            for (int j = 0; j < MAXV; ++j)
                if (li + j * lstride < nv) {
                    const T *e = reinterpret_cast<const T *>(&rx[j]);
#pragma unroll
                    for (int i = 0; i < V; ++i) var += (to_f32(e[i]) - mean) * (to_f32(e[i]) - mean);
                }
            var = group_sum(var, slot + 1, false);
            mul = 1.0f / sqrtf(var * inv_cols + eps);
            sub = mean;
        } else {
            mx = group_sum(mx, slot, true);
            float se = 0.0f;
#pragma unroll
            for (int j = 0; j < MAXV; ++j)
                if (li + j * lstride < nv) {
                    const T *e = reinterpret_cast<const T *>(&rx[j]);
#pragma unroll
                    for (int i = 0; i < V; ++i) se += (sizeof(T) == 2 ? __expf(to_f32(e[i]) * scale - mx) : expf(to_f32(e[i]) * scale - mx));
                }
            se = group_sum(se, slot + 1, false);
            mul = 1.0f / se;
        }
        T *dst = out + row * out_ld;
#pragma unroll
        for (int j = 0; j < MAXV; ++j)
            if (li + j * lstride < nv) {
                const int64_t v = li + j * lstride;
                const T *e = reinterpret_cast<const T *>(&rx[j]);
                float f[V];
                if (op == RO_SOFTMAX) {
#pragma unroll
                    for (int i = 0; i < V; ++i) f[i] = (sizeof(T) == 2 ? __expf(to_f32(e[i]) * scale - mx) : expf(to_f32(e[i]) * scale - mx)) * mul;
                } else {
#pragma unroll
                    for (int i = 0; i < V; ++i) f[i] = (to_f32(e[i]) - sub) * mul;
                    if (wgt) {
                        float g[V];
                        load_row_weight<T, V>(a, (int64_t)v * V, g);
#pragma unroll
                        for (int i = 0; i < V; ++i) f[i] *= g[i];
                    }
                }
                store_vec<T, V>(dst + v * V, f);
            }
    }
}

// Streaming variant: every active warp owns one or more row buffers in shared memory. Lane 0
// fetches whole rows with bulk asynchronous copies (completion on an mbarrier), the warp
// computes the statistics and the result in place and lane 0 hands the buffer to a bulk
// store, then refills it. With all 16 warps streaming, an SM keeps ~100 KB of loads
// outstanding — what the HBM bandwidth-delay product asks for — without spending
// registers on it. (More warps beat deeper per-warp buffering here: measured.)
constexpr int kRowStageMaxBufs = 4;
struct RowStageBars {
    unsigned long long bar[(kThreads / 32) * kRowStageMaxBufs];
};

__device__ __forceinline__ void bulk_load_row(void *smem_dst, const void *gsrc, uint32_t bytes, void *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store_row(void *gdst, const void *smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <typename T>
__device__ __noinline__ void rowop_staged(const RowOpArgs &a, int p, int P, char *smem, CtaCtl *ctl, DeviceState *st, int stage_idx,
                             unsigned long long wait_limit) {
    constexpr int V = 16 / sizeof(T);
    __shared__ RowStageBars bars;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int W = a.staged_warps, NB = a.staged_bufs;
    const bool active = warp < W;
    const int64_t cols = a.cols, nv = cols / V;
    const uint32_t row_bytes = (uint32_t)(cols * sizeof(T));
    const uint32_t buf_bytes = (row_bytes + 127) & ~127u;
    char *mybuf = smem + (size_t)warp * NB * buf_bytes;
    unsigned long long *mybar = &bars.bar[warp * kRowStageMaxBufs];
    const int op = a.op;
    const T *mask = reinterpret_cast<const T *>(a.mask);
    const float scale = (op == RO_SOFTMAX && !mask) ? a.scale : 1.0f;
    const float pre_scale = a.scale;
    const float inv_cols = 1.0f / (float)cols, eps = a.eps;
    const T *wgt = reinterpret_cast<const T *>(a.weight);
    const T *in = reinterpret_cast<const T *>(a.in);
    T *out = reinterpret_cast<T *>(a.out);
    const int64_t in_ld = a.in_ld, out_ld = a.out_ld;
    const int64_t first = (int64_t)p * W + warp, step = (int64_t)P * W;
    const int64_t mine = first < a.rows ? (a.rows - first + step - 1) / step : 0;
    // the weight row, once per CTA, behind the row buffers: read from L2 by every warp for every row it cost one L2
    // round trip per 16-byte vector (the loads cannot move above the stores of the iteration before)
    char *wsm = smem + (size_t)W * NB * buf_bytes;
    const bool wsm_on = a.weight_smem != 0;
    if (active && lane == 0) {
        for (int b = 0; b < NB; ++b) mbar_init(&mybar[b], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int64_t i = 0; i < mine && i < NB; ++i) {
            mbar_expect_tx(&mybar[i], row_bytes);
            bulk_load_row(mybuf + i * buf_bytes, in + (first + i * step) * in_ld, row_bytes, &mybar[i]);
        }
    }
    if (wsm_on) {
        const int64_t n16 = cols * (a.weight_f32 ? 4 : (int64_t)sizeof(T)) / 16;
        const uint4 *src = reinterpret_cast<const uint4 *>(a.weight);
        for (int64_t v = threadIdx.x; v < n16; v += kThreads) reinterpret_cast<uint4 *>(wsm)[v] = __ldg(src + v);
        __syncthreads();
    }
    if (!active) return;
    __syncwarp();
    for (int64_t i = 0; i < mine; ++i) {
        const int b = (int)(i % NB);
        bool ok = mbar_wait(&mybar[b], (uint32_t)((i / NB) & 1), wait_limit);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (lane == 0) {
                ctl->abort = 1;
                report(st, ST_MBAR_TIMEOUT, stage_idx);
            }
            return;
        }
        T *row = reinterpret_cast<T *>(mybuf + b * buf_bytes);
        if (mask) {
            // masked softmax: logits x * scale + mask, rounded to the storage type, replace the row in shared memory
            const T *mk = mask + ((first + i * step) % a.mask_rows) * a.mask_ld;
            for (int64_t v = lane; v < nv; v += 32) {
                uint4 q = *reinterpret_cast<const uint4 *>(row + v * V);
                const uint4 g4 = *reinterpret_cast<const uint4 *>(mk + v * V);
                T *e = reinterpret_cast<T *>(&q);
                const T *ge = reinterpret_cast<const T *>(&g4);
#pragma unroll
                for (int k = 0; k < V; ++k) e[k] = from_f32<T>(to_f32(e[k]) * pre_scale + to_f32(ge[k]));
                *reinterpret_cast<uint4 *>(row + v * V) = q;
            }
            __syncwarp();
        }
        if (a.residual) {
            // x := x + residual, rounded to the storage type, kept (res_out) for the next block and normalised below
            const T *rr = reinterpret_cast<const T *>(a.residual) + (first + i * step) * in_ld;
            T *ro = reinterpret_cast<T *>(a.res_out) + (first + i * step) * in_ld;
            for (int64_t v0 = lane; v0 < nv; v0 += 128) {  // four residual loads in flight per lane before the stores
                uint4 g4[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (v0 + 32 * u < nv) g4[u] = ldg16_stream(rr + (v0 + 32 * u) * V);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t v = v0 + 32 * u;
                    if (v < nv) {
                        uint4 q = *reinterpret_cast<const uint4 *>(row + v * V);
                        T *e = reinterpret_cast<T *>(&q);
                        const T *ge = reinterpret_cast<const T *>(&g4[u]);
#pragma unroll
                        for (int k = 0; k < V; ++k) e[k] = from_f32<T>(to_f32(e[k]) + to_f32(ge[k]));
                        *reinterpret_cast<uint4 *>(row + v * V) = q;
                        *reinterpret_cast<uint4 *>(ro + v * V) = q;
                    }
                }
            }
            __syncwarp();
        }
        float s1 = 0.0f, s2 = 0.0f, mx = -3.402823466e+38f;
        for (int64_t v = lane; v < nv; v += 32) {
            const uint4 q = *reinterpret_cast<const uint4 *>(row + v * V);
            const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const float x = to_f32(e[k]) * scale;
                s1 += x;
                s2 += x * x;
                mx = fmaxf(mx, x);
            }
        }
        float mul = 1.0f, sub = 0.0f;
        if (op == RO_RMSNORM) {
            mul = 1.0f / sqrtf(warp_sum(s2) * inv_cols + eps);
        } else if (op == RO_LAYERNORM) {
            const float mean = warp_sum(s1) * inv_cols;
            float var = 0.0f;
            for (int64_t v = lane; v < nv; v += 32) {
                const uint4 q = *reinterpret_cast<const uint4 *>(row + v * V);
                const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
                for (int k = 0; k < V; ++k) var += (to_f32(e[k]) - mean) * (to_f32(e[k]) - mean);
            }
            mul = 1.0f / sqrtf(warp_sum(var) * inv_cols + eps);
            sub = mean;
        } else {
            mx = warp_max(mx);
            float se = 0.0f;
            for (int64_t v = lane; v < nv; v += 32) {
                const uint4 q = *reinterpret_cast<const uint4 *>(row + v * V);
                const T *e = reinterpret_cast<const T *>(&q);
#pragma unroll
                for (int k = 0; k < V; ++k)
                    se += (sizeof(T) == 2 ? __expf(to_f32(e[k]) * scale - mx) : expf(to_f32(e[k]) * scale - mx));
            }
            mul = 1.0f / warp_sum(se);
        }
        for (int64_t v = lane; v < nv; v += 32) {
            const uint4 q = *reinterpret_cast<const uint4 *>(row + v * V);
            const T *e = reinterpret_cast<const T *>(&q);
            float f[V];
            if (op == RO_SOFTMAX) {
#pragma unroll
                for (int k = 0; k < V; ++k)
                    f[k] = (sizeof(T) == 2 ? __expf(to_f32(e[k]) * scale - mx) : expf(to_f32(e[k]) * scale - mx)) * mul;
            } else {
#pragma unroll
                for (int k = 0; k < V; ++k) f[k] = (to_f32(e[k]) - sub) * mul;
                if (wgt) {
                    float g[V];
                    if (!wsm_on) load_row_weight<T, V>(a, (int64_t)v * V, g);
                    else if (a.weight_f32) load_vec_cached<float, V>(reinterpret_cast<const float *>(wsm) + v * V, g);  // plain (generic) loads
                    else load_vec_cached<T, V>(reinterpret_cast<const T *>(wsm) + v * V, g);
#pragma unroll
                    for (int k = 0; k < V; ++k) f[k] *= g[k];
                }
            }
            store_vec<T, V>(row + v * V, f);  // in place, in shared memory
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
            bulk_store_row(out + (first + i * step) * out_ld, row, row_bytes);
            // refill a buffer whose store has finished reading it: with several buffers per warp the one
            // stored an iteration ago (this iteration's store stays in flight), with a single buffer this one
            if (NB == 1) {
                if (i + 1 < mine) {
                    tma_store_wait_read<0>();
                    mbar_expect_tx(&mybar[0], row_bytes);
                    bulk_load_row(mybuf, in + (first + (i + 1) * step) * in_ld, row_bytes, &mybar[0]);
                }
            } else if (i >= 1 && (i - 1) + NB < mine) {
                tma_store_wait_read<1>();
                const int pb = (int)((i - 1) % NB);
                mbar_expect_tx(&mybar[pb], row_bytes);
                bulk_load_row(mybuf + pb * buf_bytes, in + (first + (i - 1 + NB) * step) * in_ld, row_bytes, &mybar[pb]);
            }
        }
        __syncwarp();
    }
    if (lane == 0) {
        tma_store_wait<0>();  // results are in global memory before the stage ends
        // the barriers are re-created by the next row stage: retire them
        for (int b = 0; b < NB; ++b) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&mybar[b])) : "memory");
    }
    __syncwarp();
}

template <typename T>
__device__ __forceinline__ void rowop_dispatch(const RowOpArgs &a, int p, int P, char *smem, CtaCtl *ctl, DeviceState *st,
                                               int stage_idx, unsigned long long wait_limit) {
    const int G = a.warps_per_row;
    if (a.staged_warps > 0) rowop_staged<T>(a, p, P, smem, ctl, st, stage_idx, wait_limit);
    else if (G > 0) rowop_regs<T>(a, p, P, G);
    else rowop_typed<T>(a, p, P);
}

__device__ __noinline__ void run_rowop(const RowOpArgs &a, int p, int P, char *smem, CtaCtl *ctl, DeviceState *st, int stage_idx,
                          unsigned long long wait_limit) {
    switch (a.dtype) {
        case DT_F32: rowop_dispatch<float>(a, p, P, smem, ctl, st, stage_idx, wait_limit); break;
        case DT_F16: rowop_dispatch<__half>(a, p, P, smem, ctl, st, stage_idx, wait_limit); break;
        case DT_BF16: rowop_dispatch<__nv_bfloat16>(a, p, P, smem, ctl, st, stage_idx, wait_limit); break;
        default: break;
    }
}

// ---- transpose / embedding ---------------------------------------------------------
// 4-D permutation (ark/include/kernels/transpose.h). When the innermost dim
// stays innermost the copy is vectorised along it; otherwise a 32x32 shared
// memory tile turns strided reads into coalesced ones.
template <int ES>
__device__ void transpose_es(const TransposeArgs &a, int p, int P, char *smem) {
    typedef typename std::conditional<ES == 4, uint32_t, typename std::conditional<ES == 2, uint16_t, uint8_t>::type>::type E;
    const E *in = reinterpret_cast<const E *>(a.in.ptr);
    E *out = reinterpret_cast<E *>(a.out.ptr);
    const int64_t O0 = a.out.shape[0], O1 = a.out.shape[1], O2 = a.out.shape[2], O3 = a.out.shape[3];
    int64_t is[4];  // input stride seen from each output dim
    for (int i = 0; i < 4; ++i) is[i] = a.in.stride[a.perm[i]];
    if (a.perm[3] == 3 && !a.partial) {
        constexpr int V = 16 / ES;
        const bool vec = (O3 % V == 0) && a.out.contiguous == 2;  // host: 2 = rows 16-byte aligned on both sides
        if (vec) {
            const int64_t WV = O3 / V, units = O0 * O1 * O2 * WV;
            for (int64_t u = (int64_t)p * kThreads + threadIdx.x; u < units; u += (int64_t)P * kThreads) {
                int64_t wv = u % WV, r = u / WV;
                int64_t i2 = r % O2;
                r /= O2;
                int64_t i1 = r % O1, i0 = r / O1;
                const uint4 v = *reinterpret_cast<const uint4 *>(in + i0 * is[0] + i1 * is[1] + i2 * is[2] + wv * V);
                *reinterpret_cast<uint4 *>(out + tref_off(a.out, i0, i1, i2, wv * V)) = v;
            }
            return;
        }
    }
    // generic: one element per thread, writes coalesced
    const int64_t total = O0 * O1 * O2 * O3;
    for (int64_t i = (int64_t)p * kThreads + threadIdx.x; i < total; i += (int64_t)P * kThreads) {
        int64_t i3 = i % O3, r = i / O3;
        int64_t i2 = r % O2;
        r /= O2;
        int64_t i1 = r % O1, i0 = r / O1;
        if (a.partial) {
            const int64_t th = (O2 + a.tile_h - 1) / a.tile_h, tw = (O3 + a.tile_w - 1) / a.tile_w;
            const int64_t task = ((i0 * O1 + i1) * th + i2 / a.tile_h) * tw + i3 / a.tile_w;
            if (task < a.task_b || task >= a.task_e || (task - a.task_b) % a.task_s) continue;
        }
        out[tref_off(a.out, i0, i1, i2, i3)] = in[i0 * is[0] + i1 * is[1] + i2 * is[2] + i3 * is[3]];
    }
}

__device__ __noinline__ void run_transpose(const TransposeArgs &a, int p, int P, char *smem) {
    const int dt = a.in.dtype;
    if (dt == DT_F32 || dt == DT_I32 || dt == DT_U32) transpose_es<4>(a, p, P, smem);
    else if (dt == DT_F16 || dt == DT_BF16) transpose_es<2>(a, p, P, smem);
    else transpose_es<1>(a, p, P, smem);
}

// Row gather (ark/include/kernels/embedding.h; host op ark/ops/ops_embedding.cpp:37-70):
// one warp per index, negative indices wrap.
__device__ __noinline__ void run_embed(const EmbedArgs &a, int p, int P) {
    constexpr int WPC = kThreads / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row_bytes = a.emb_dim * a.esize;
    for (int64_t k = (int64_t)p * WPC + warp; k < a.n_idx; k += (int64_t)P * WPC) {
        const int64_t i = a.task_b + k * a.task_s;
        int64_t r = a.idx[i];
        if (r < 0) r += a.num_emb;
        const char *src = reinterpret_cast<const char *>(a.weight) + r * a.w_ld * a.esize;
        char *dst = reinterpret_cast<char *>(a.out) + i * a.out_ld * a.esize;
        if (((row_bytes | (a.w_ld * a.esize) | (a.out_ld * a.esize)) & 15) == 0 &&
            ((reinterpret_cast<uintptr_t>(a.weight) | reinterpret_cast<uintptr_t>(a.out)) & 15) == 0) {
            for (int64_t b = lane * 16; b < row_bytes; b += 32 * 16)
                *reinterpret_cast<uint4 *>(dst + b) = *reinterpret_cast<const uint4 *>(src + b);
        } else {
            for (int64_t b = lane; b < row_bytes; b += 32) dst[b] = src[b];
        }
    }
}

}  // namespace arkb
