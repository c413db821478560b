// Weight-streaming matmul for one or two activation rows: y[M, N] = x[M, K] . W.
// The reference runs these shapes through the same tiled GEMM as everything
// else (ark/include/kernels/matmul.h:36-115); at one or two rows that work is
// a read of W at HBM speed and nothing else, so this stage is built around the
// read: every lane keeps four to eight 16-byte loads of W in flight (64 KiB and more per SM),
// the activations sit in shared memory as fp32, products are accumulated in
// fp32 on the CUDA cores and rounded once. The tensor cores are left out on
// purpose: with W in the 128-row operand of tcgen05.mma an SM consumes at most
// 32 bytes of W per clock and the accumulate-commit-reload chain of a ring slot
// sits on the critical path; measured, that form stays below 65% of HBM peak.
//
// Two layouts of W:
//   [N, K] (K contiguous): a warp owns whole rows of W inside the CTA's
//       k-range; lanes stride the row in 16-byte vectors; one shuffle
//       reduction per row and activation row.
//   [K, N] (N contiguous): a warp owns 256 output columns and a k-range; a lane
//       owns 8 columns and adds up the rows of the range.
// When K is split into ranges (splits > 1) the fp32 partials go to
// ws[range][m][n] and the split-K sum stage that follows adds them in range
// order, applies the activation and rounds (deterministic).
#include "dev_comm.cuh"
#include "dev_common.cuh"
#include "dev_funcs.h"

namespace arkb {

namespace {


// Sum over the CTA of one float per thread (all threads call it; `scratch` holds one float per warp).
__device__ __forceinline__ float cta_sum(float v, float *scratch) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = 0.0f;
    for (int i = 0; i < nw; ++i) r += scratch[i];
    return r;
}

// Where a folded one-shot all_reduce wants the result: slot [rank] of every rank's staging buffer (dense [M, N]).
struct PushTo {
    char *slot[kMaxPeers];  // this rank's slot on every rank, null when nothing is pushed
    int nranks;
    // The activations are the sum of a one-shot all_reduce that has not been added up yet (src_ord of the stage):
    // slot q of this rank's staging area holds rank q's dense [M, K] partial. Null otherwise.
    const char *src;
    uint64_t src_slot_bytes;
    int src_ranks;
};
__device__ __forceinline__ PushTo push_targets(const GemvArgs &a, const LaunchParams &P, unsigned long long iter_no) {
    PushTo t;
    t.nranks = 0;
    t.src = nullptr; t.src_slot_bytes = 0; t.src_ranks = 0;
    if (a.src_ord > 0) {
        const uint64_t par = (iter_no * (unsigned long long)a.push_per_iter + (unsigned long long)(a.src_ord - 1)) & 1;
        t.src = P.comm[P.rank] + kCommDataOff + par * a.push_stage_bytes;
        t.src_slot_bytes = a.push_stage_bytes / kMaxPeers;
        t.src_ranks = P.nranks;
    }
    if (a.push_ord > 0) {
        const uint64_t par = (iter_no * (unsigned long long)a.push_per_iter + (unsigned long long)(a.push_ord - 1)) & 1;
        const uint64_t base = kCommDataOff + par * a.push_stage_bytes + (uint64_t)P.rank * (a.push_stage_bytes / kMaxPeers);
        t.nranks = P.nranks;
        for (int q = 0; q < kMaxPeers; ++q) t.slot[q] = q < P.nranks ? P.comm[q] + base : nullptr;
    }
    return t;
}

// Eight activations as the producer left them: read from x, or — when the one-shot all_reduce that produces x was
// folded into this stage — added up over the ranks' slots in rank order and rounded where the all_reduce would
// have stored the sum.
template <typename T>
__device__ __forceinline__ void load_raw8(const GemvArgs &a, const PushTo &c, int m, int k, float (&f)[8]) {
    if (c.src) {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = 0.0f;
        for (int q = 0; q < c.src_ranks; ++q) {
            float g[8];
            unpack8<T>(*reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(c.src + q * c.src_slot_bytes) + (int64_t)m * a.K + k), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] += g[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = to_f32(from_f32<T>(f[i]));
        return;
    }
    unpack8<T>(*reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.x) + (int64_t)m * a.ldx + k), f);
}

// The activations as this stage consumes them: the raw x, or the operator folded in before it
// (GP_MUL: x * other; GP_RMSNORM: (x [+ residual]) * rstd * weight), rounded to the storage type like
// the separate operator would have stored them. `rstd` is per activation row (GP_RMSNORM only).
template <typename T>
__device__ __forceinline__ void load_x8(const GemvArgs &a, const PushTo &c, int m, int k, float rstd, float (&f)[8]) {
    if (a.pro == GP_ATTN_MERGE) {
        // the attention's chunks of head k / 128 of sequence m, merged with the usual max / sum rescaling and rounded
        // like the merge stage would have stored them
        const int G = a.mg_group, h = k >> 7, d = k & 127, kvh = h / G, g = h % G;
        const size_t stride = (size_t)G * 130;
        const float *w = reinterpret_cast<const float *>(a.pro_a) + ((size_t)(m * a.mg_kv_heads + kvh) * a.mg_chunks) * stride;
        float mx = -3.402823466e+38f;
        for (int c = 0; c < a.mg_chunks; ++c) mx = fmaxf(mx, w[c * stride + G * 128 + 2 * g]);
        float l = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = 0.0f;
        for (int c = 0; c < a.mg_chunks; ++c) {
            const float e = __expf(w[c * stride + G * 128 + 2 * g] - mx);
            l += w[c * stride + G * 128 + 2 * g + 1] * e;
            const float2 *o = reinterpret_cast<const float2 *>(w + c * stride + g * 128 + d);  // records are 8-byte aligned
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 v = o[i];
                f[2 * i] += v.x * e;
                f[2 * i + 1] += v.y * e;
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = to_f32(from_f32<T>(f[i] / l));
        return;
    }
    load_raw8<T>(a, c, m, k, f);
    if (a.pro == GP_MUL) {
        float g[8];
        unpack8<T>(*reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.pro_a) + (int64_t)m * a.ldx + k), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = to_f32(from_f32<T>(f[i] * g[i]));
    } else if (a.pro == GP_RMSNORM) {
        if (a.pro_b) {
            float g[8];
            unpack8<T>(*reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.pro_b) + (int64_t)m * a.ldx + k), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = to_f32(from_f32<T>(f[i] + g[i]));
        }
        if (a.pro_a) {
            float g[8];
            unpack8<T>(*reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.pro_a) + k), g);
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = to_f32(from_f32<T>(f[i] * rstd * g[i]));
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = to_f32(from_f32<T>(f[i] * rstd));
        }
    }
}

// 1 / rms of every activation row over the WHOLE of K (GP_RMSNORM), into rstd[0..M). With a residual, CTA 0
// also stores x + residual (the value the norm is taken of) for the operators that follow.
template <typename T>
__device__ __forceinline__ void row_rstd(const GemvArgs &a, const PushTo &c, int p, float *rstd, float *scratch) {
    const T *r = reinterpret_cast<const T *>(a.pro_b);
    T *ro = reinterpret_cast<T *>(a.pro_out);
    for (int m = 0; m < a.M; ++m) {
        float ss = 0.0f;
        for (int k = threadIdx.x * 8; k < a.K; k += blockDim.x * 8) {
            float f[8];
            load_raw8<T>(a, c, m, k, f);
            if (r) {
                float g[8];
                unpack8<T>(*reinterpret_cast<const uint4 *>(r + (int64_t)m * a.ldx + k), g);
                union { uint4 q; T e[8]; } o;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    o.e[i] = from_f32<T>(f[i] + g[i]);
                    f[i] = to_f32(o.e[i]);
                }
                if (ro && p == 0) *reinterpret_cast<uint4 *>(ro + (int64_t)m * a.ldx + k) = o.q;
            } else if (ro && p == 0) {  // a folded all_reduce without a residual: its sum is kept
                union { uint4 q; T e[8]; } o;
#pragma unroll
                for (int i = 0; i < 8; ++i) o.e[i] = from_f32<T>(f[i]);
                *reinterpret_cast<uint4 *>(ro + (int64_t)m * a.ldx + k) = o.q;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
        }
        ss = cta_sum(ss, scratch);
        if (threadIdx.x == 0) rstd[m] = 1.0f / sqrtf(ss / (float)a.K + a.pro_eps);
    }
    __syncthreads();
}

// Copies the activations [0..M)[k0 .. k0+kr) into shared memory as fp32. The 8 values of vector v of row m are
// kept as two float4 in separate planes, xs[(m * 2 + h) * nv + v], so that lanes reading consecutive vectors
// touch consecutive 16-byte words (no bank conflicts).
template <typename T>
__device__ __forceinline__ void stage_x(const GemvArgs &a, const PushTo &c, float4 *xs, int nv, int k0, const float *rstd) {
    for (int i = threadIdx.x; i < a.M * nv; i += blockDim.x) {
        const int m = i / nv, v = i % nv;
        float f[8];
        load_x8<T>(a, c, m, k0 + v * 8, a.pro == GP_RMSNORM ? rstd[m] : 1.0f, f);
        xs[((size_t)m * 2 + 0) * nv + v] = make_float4(f[0], f[1], f[2], f[3]);
        xs[((size_t)m * 2 + 1) * nv + v] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

template <typename T>
__device__ __forceinline__ void emit(const GemvArgs &a, const PushTo &push, int split, int m, int n, float v) {
    if (a.splits > 1) {
        a.ws[((int64_t)split * a.M + m) * a.N + n] = v;
    } else if (n >= a.N) {  // a row of the second matrix
        reinterpret_cast<T *>(a.out_b)[(int64_t)m * a.ldo + (n - a.N)] = from_f32<T>(apply_act_fast(a.act_b, v));
    } else {
        v = apply_act_fast(a.act, v);
        if (a.residual) v = to_f32(from_f32<T>(v)) + to_f32(reinterpret_cast<const T *>(a.residual)[(int64_t)m * a.ldo + n]);
        const T r = from_f32<T>(v);
        reinterpret_cast<T *>(a.out)[(int64_t)m * a.ldo + n] = r;
        for (int q = 0; q < push.nranks; ++q) reinterpret_cast<T *>(push.slot[q])[(int64_t)m * a.N + n] = r;
    }
}

// ---- W stored [N, K] ---------------------------------------------------------------
// A warp walks RW rows of W together; per step a lane loads VC 16-byte vectors of each row, 32
// vectors apart (every load instruction covers 512 contiguous bytes; RW * VC = 8 loads per step).
// The activations of a step are read from shared memory once for all RW rows: many rows per warp
// when the matrix has rows to spare, few rows and more vectors per row when it has not. Two register buffers
// alternate: the loads of step t+1 are issued before step t is consumed, across row groups too.
template <typename T, int M, int RW, int VC>
__device__ __noinline__ void gemv_nk(const GemvArgs &a, int p, int P, float4 *xs, const PushTo &push) {
    const int cps = a.ctas_per_split;
    const int split = p / cps, q = p % cps;
    if (split >= a.splits) return;
    const int k0 = split * a.kper;
    const int kr = min(a.K, k0 + a.kper) - k0;
    const int nv = kr / 8;
    float *rstd = reinterpret_cast<float *>(xs + (size_t)a.M * 2 * nv);  // [M], then one float per warp of scratch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int n_rows = a.w_b ? 2 * a.N : a.N;  // with a second matrix the row space is both matrices' rows
    const int row_lo = (int)((int64_t)q * n_rows / cps), row_hi = (int)((int64_t)(q + 1) * n_rows / cps);
    const T *w_b = reinterpret_cast<const T *>(a.w_b) + k0;
    const int n_first = a.N;
    const int steps = (nv + 32 * VC - 1) / (32 * VC);  // per row group
    const T *w = reinterpret_cast<const T *>(a.w) + k0;
    const int64_t ldw = a.ldw;
    const int rows_m = a.M;

    struct Cursor {
        int r0, j;
    };
    auto valid = [&](const Cursor &c) { return c.r0 < row_hi; };
    auto advance = [&](Cursor &c) {
        if (++c.j == steps) {
            c.j = 0;
            c.r0 += nwarps * RW;
        }
    };
    auto issue = [&](uint4 (&buf)[RW][VC], const Cursor &c) {
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int v = 0; v < VC; ++v) {
                const int vi = lane + 32 * (c.j * VC + v);
                const int row = c.r0 + r;
                if (row < row_hi && vi < nv)
                    buf[r][v] = ldg16_stream((row < n_first ? w + (int64_t)row * ldw : w_b + (int64_t)(row - n_first) * ldw) + vi * 8);
                else buf[r][v] = make_uint4(0, 0, 0, 0);
            }
    };
    float acc[RW][M];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = 0.0f;
    auto consume = [&](uint4 (&buf)[RW][VC], const Cursor &c) {
#pragma unroll
        for (int v = 0; v < VC; ++v) {
            const int vi = lane + 32 * (c.j * VC + v);
            if (vi < nv) {
                float f[RW][8];
#pragma unroll
                for (int r = 0; r < RW; ++r) unpack8<T>(buf[r][v], f[r]);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    if (m < rows_m) {
                        const float4 x0 = xs[((size_t)m * 2 + 0) * nv + vi], x1 = xs[((size_t)m * 2 + 1) * nv + vi];
#pragma unroll
                        for (int r = 0; r < RW; ++r)
                            acc[r][m] += f[r][0] * x0.x + f[r][1] * x0.y + f[r][2] * x0.z + f[r][3] * x0.w + f[r][4] * x1.x +
                                         f[r][5] * x1.y + f[r][6] * x1.z + f[r][7] * x1.w;
                    }
                }
            }
        }
        if (c.j == steps - 1) {  // the rows of this group are complete
#pragma unroll
            for (int r = 0; r < RW; ++r)
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    const float sum = warp_sum(acc[r][m]);
                    if (lane == 0 && m < rows_m && c.r0 + r < row_hi) emit<T>(a, push, split, m, c.r0 + r, sum);
                    acc[r][m] = 0.0f;
                }
        }
    };
    Cursor ld{row_lo + warp * RW, 0}, cp = ld;
    uint4 qa[RW][VC], qb[RW][VC];
    // the weights do not depend on the activations: the first loads are in flight while x is normalised and staged
    if (valid(ld)) {
        issue(qa, ld);
        advance(ld);
    }
    if (a.pro == GP_RMSNORM) row_rstd<T>(a, push, p, rstd, rstd + 8);
    stage_x<T>(a, push, xs, nv, k0, rstd);
    __syncthreads();
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
}

// ---- W stored [K, N] ---------------------------------------------------------------
// Item = (block of 256 columns, k-range), one warp per item: a lane owns 8 columns, walks the rows
// of the range U at a time (two register buffers alternating as above) and writes its sums itself,
// so warps never wait for one another. All of x sits in shared memory as 16-bit values.
template <typename T, int M, int U>
__device__ __noinline__ void gemv_kn(const GemvArgs &a, int p, int P, T *xs, const PushTo &push) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwarps = blockDim.x >> 5;
    const int rows_m = a.M;
    const int64_t ldw = a.ldw;
    const int K = a.K;
    {
        float *rstd = reinterpret_cast<float *>(xs + (size_t)rows_m * K);  // [M], then one float per warp of scratch (K is a multiple of 8)
        if (a.pro == GP_RMSNORM) row_rstd<T>(a, push, p, rstd, rstd + 8);
        const int nvk = K / 8;
        for (int i = threadIdx.x; i < rows_m * nvk; i += blockDim.x) {
            const int m = i / nvk, v = i % nvk;
            float f[8];
            load_x8<T>(a, push, m, v * 8, a.pro == GP_RMSNORM ? rstd[m] : 1.0f, f);
            union { uint4 q; T e[8]; } o;
#pragma unroll
            for (int e = 0; e < 8; ++e) o.e[e] = from_f32<T>(f[e]);
            *reinterpret_cast<uint4 *>(xs + (size_t)m * K + v * 8) = o.q;
        }
    }
    __syncthreads();
    const int items = a.nblocks * a.splits;
    const T *w = reinterpret_cast<const T *>(a.w);
    for (int it = p * nwarps + warp; it < items; it += P * nwarps) {
        const int split = it / a.nblocks, nb = it % a.nblocks;
        const int k0 = split * a.kper;
        const int kr = min(K, k0 + a.kper) - k0;
        const int col = nb * 256 + lane * 8;
        if (col >= a.N) continue;  // N is a multiple of 8
        float acc[M][8];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[m][j] = 0.0f;
        const T *wc = w + (int64_t)k0 * ldw + col;
        const T *xk = xs + k0;
        auto issue = [&](uint4 (&buf)[U], int kb) {
#pragma unroll
            for (int u = 0; u < U; ++u) buf[u] = kb + u < kr ? ldg16_stream(wc + (int64_t)(kb + u) * ldw) : make_uint4(0, 0, 0, 0);
        };
        auto consume = [&](uint4 (&buf)[U], int kb) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int k = kb + u;
                if (k < kr) {
                    float f[8];
                    unpack8<T>(buf[u], f);
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        if (m < rows_m) {
                            const float xv = to_f32(xk[(size_t)m * K + k]);
#pragma unroll
                            for (int j = 0; j < 8; ++j) acc[m][j] += xv * f[j];
                        }
                    }
                }
            }
        };
        uint4 qa[U], qb[U];
        int kb = 0;
        issue(qa, kb);
        while (kb < kr) {
            if (kb + U < kr) issue(qb, kb + U);
            consume(qa, kb);
            kb += U;
            if (kb >= kr) break;
            if (kb + U < kr) issue(qa, kb + U);
            consume(qb, kb);
            kb += U;
        }
#pragma unroll
        for (int m = 0; m < M; ++m) {
            if (m < rows_m) {
#pragma unroll
                for (int j = 0; j < 8; ++j) emit<T>(a, push, split, m, col + j, acc[m][j]);
            }
        }
    }
}

template <typename T>
__device__ void gemv_typed(const GemvArgs &a, int p, int P, char *smem, const PushTo &push) {
    if (a.w_is_nk && a.light) {
        // Half the loads in flight per lane (4 x 16 bytes in each of the two buffers): enough for matrices that are
        // small or already in L2, in a function that needs a third of the registers, and a function that needs
        // few registers has little to save and restore when the loop kernel calls it (~1 us less per stage).
        float4 *xs = reinterpret_cast<float4 *>(smem);
        if (a.M == 1) {
            switch (a.rows_together) {
                case 4: gemv_nk<T, 1, 4, 1>(a, p, P, xs, push); break;
                case 2: gemv_nk<T, 1, 2, 2>(a, p, P, xs, push); break;
                default: gemv_nk<T, 1, 1, 4>(a, p, P, xs, push); break;
            }
        } else {
            if (a.rows_together == 2) gemv_nk<T, 2, 2, 1>(a, p, P, xs, push);
            else gemv_nk<T, 2, 1, 2>(a, p, P, xs, push);
        }
        return;
    }
    if (a.w_is_nk) {
        float4 *xs = reinterpret_cast<float4 *>(smem);
        if (a.M == 1) {
            switch (a.rows_together) {
                case 8: gemv_nk<T, 1, 8, 1>(a, p, P, xs, push); break;
                case 4: gemv_nk<T, 1, 4, 2>(a, p, P, xs, push); break;
                case 2: gemv_nk<T, 1, 2, 4>(a, p, P, xs, push); break;
                default: gemv_nk<T, 1, 1, 8>(a, p, P, xs, push); break;
            }
        } else {
            switch (a.rows_together) {
                case 4: gemv_nk<T, 2, 4, 1>(a, p, P, xs, push); break;
                case 2: gemv_nk<T, 2, 2, 2>(a, p, P, xs, push); break;
                default: gemv_nk<T, 2, 1, 4>(a, p, P, xs, push); break;
            }
        }
    } else {
        T *xs = reinterpret_cast<T *>(smem);
        if (a.M == 1) gemv_kn<T, 1, 8>(a, p, P, xs, push);
        else gemv_kn<T, 2, 4>(a, p, P, xs, push);
    }
}

}  // namespace

__device__ __noinline__ void run_gemv(const GemvArgs &a, int p, int P, char *smem, const LaunchParams &LP, unsigned long long iter_no) {
    const PushTo push = push_targets(a, LP, iter_no);
    if (a.dtype == DT_BF16) gemv_typed<__nv_bfloat16>(a, p, P, smem, push);
    else gemv_typed<__half>(a, p, P, smem, push);
}

}  // namespace arkb
