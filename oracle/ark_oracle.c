/*
 * CPU oracle for the ARK op set — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the host baselines that the reference's op unit
 * tests compare the GPU results with (ark/ops/ops_*_test.cpp), plus CPU
 * restatements of the two checks for which the reference has no CPU code
 * (matmul: the reference test calls cuBLAS; all_reduce: closed-form sums).
 * Only the tests, the smoke check and the benchmark's cpu_baseline leg may
 * call into this library; the engine itself never does.
 *
 * Parity pin: every function here is checked bit-for-bit against the
 * reference's own baseline templates compiled from the reference sources
 * (oracle/ref_shim.cpp -> oracle/_ref/libark_ref.so) and against the golden
 * vectors generated from that library (tests/golden/).
 *
 * Conventions (same as the reference baselines):
 *   - tensors are dense row-major, up to 4-D, shape left-padded with 1s to
 *     [N,C,H,W] (ark/api/dims.cpp:59-69);
 *   - floating-point work is done in fp32 (or double where the reference's
 *     expression promotes to double) and rounded ONCE to the storage type
 *     with round-to-nearest-even, unless a comment says otherwise.
 *
 * dtype codes: 0 = fp32, 1 = fp16, 2 = bf16, 3 = int32, 4 = uint32,
 *              5 = int8, 6 = uint8/byte.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_I32 = 3, ORC_U32 = 4, ORC_I8 = 5, ORC_U8 = 6 };

/* ---- storage conversions ------------------------------------------------ */

/* fp32 -> fp16, round to nearest even (ark/half.h:65-140 does the same in
 * software; _Float16 conversion in GCC is IEEE RNE). */
static inline uint16_t f2h(float f) {
    _Float16 h = (_Float16)f;
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}
static inline float h2f(uint16_t u) {
    _Float16 h;
    memcpy(&h, &u, 2);
    return (float)h;
}
/* fp32 -> bf16, round to nearest even, NaN kept quiet (ark/bfloat16.h). */
static inline uint16_t f2b(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7f800000u) == 0x7f800000u && (x & 0x007fffffu)) return 0x7fff;
    x += 0x7fffu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}
static inline float b2f(uint16_t u) {
    uint32_t x = ((uint32_t)u) << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

static inline size_t dsize(int dt) {
    switch (dt) {
        case ORC_F32: case ORC_I32: case ORC_U32: return 4;
        case ORC_F16: case ORC_BF16: return 2;
        default: return 1;
    }
}
static inline float ldf(const void *p, int dt, size_t i) {
    switch (dt) {
        case ORC_F32: return ((const float *)p)[i];
        case ORC_F16: return h2f(((const uint16_t *)p)[i]);
        case ORC_BF16: return b2f(((const uint16_t *)p)[i]);
        case ORC_I32: return (float)((const int32_t *)p)[i];
        case ORC_U32: return (float)((const uint32_t *)p)[i];
        case ORC_I8: return (float)((const int8_t *)p)[i];
        default: return (float)((const uint8_t *)p)[i];
    }
}
static inline void stf(void *p, int dt, size_t i, float v) {
    switch (dt) {
        case ORC_F32: ((float *)p)[i] = v; break;
        case ORC_F16: ((uint16_t *)p)[i] = f2h(v); break;
        case ORC_BF16: ((uint16_t *)p)[i] = f2b(v); break;
        case ORC_I32: ((int32_t *)p)[i] = (int32_t)v; break;
        case ORC_U32: ((uint32_t *)p)[i] = (uint32_t)v; break;
        case ORC_I8: ((int8_t *)p)[i] = (int8_t)v; break;
        default: ((uint8_t *)p)[i] = (uint8_t)v; break;
    }
}
/* round a float through the storage type (models half_t/bfloat16_t
 * arithmetic, where every operator returns the storage type). */
static inline float rnd(int dt, float v) {
    if (dt == ORC_F16) return h2f(f2h(v));
    if (dt == ORC_BF16) return b2f(f2b(v));
    return v;
}

/* ---- unary math: ark/ops/ops_math_test.cpp:10-94, ops_copy_test.cpp ------ */

enum { ORC_GELU = 0, ORC_EXP = 1, ORC_RELU = 2, ORC_RSQRT = 3, ORC_SIGMOID = 4, ORC_SQRT = 5, ORC_COPY = 6 };

/* ops_math_test.cpp:10-12: the expression is evaluated in double (0.5,
 * M_PI, pow) on a float argument and returned as float. */
static float gelu_ref(float x) {
    return (float)(0.5 * x * (1 + tanh(sqrt(2 / M_PI) * (x + 0.044715 * pow(x, 3)))));
}

ORC_API void orc_unary(int op, int dt, void *out, const void *in, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float x = ldf(in, dt, i), y;
        switch (op) {
            case ORC_GELU: y = gelu_ref(x); break;                 /* :14-25 */
            case ORC_EXP: y = expf(x); break;                      /* :27-38 */
            case ORC_RELU: y = x > 0 ? x : 0; break;               /* :40-53 */
            case ORC_RSQRT: y = 1.0f / sqrtf(x); break;            /* :55-66 */
            case ORC_SIGMOID: y = 1 / (1 + expf(-x)); break;       /* :68-81 */
            case ORC_SQRT: y = sqrtf(x); break;                    /* :83-94 */
            default: y = x; break;                                 /* copy */
        }
        stf(out, dt, i, y);
    }
}

/* ---- binary with NumPy broadcast: ark/ops/ops_arithmetic_test.cpp:7-128 -- */

enum { ORC_ADD = 0, ORC_SUB = 1, ORC_MUL = 2, ORC_DIV = 3 };

ORC_API void orc_binary(int op, int dt, void *out, const int64_t *osh, const void *a,
                        const int64_t *ash, const void *b, const int64_t *bsh) {
    for (int64_t n = 0; n < osh[0]; ++n)
        for (int64_t c = 0; c < osh[1]; ++c)
            for (int64_t h = 0; h < osh[2]; ++h)
                for (int64_t w = 0; w < osh[3]; ++w) {
                    size_t io = w + osh[3] * (h + osh[2] * (c + osh[1] * n));
                    size_t ia = (w % ash[3]) + ash[3] * ((h % ash[2]) + ash[2] * ((c % ash[1]) + ash[1] * (n % ash[0])));
                    size_t ib = (w % bsh[3]) + bsh[3] * ((h % bsh[2]) + bsh[2] * ((c % bsh[1]) + bsh[1] * (n % bsh[0])));
                    float x = ldf(a, dt, ia), y = ldf(b, dt, ib), r;
                    switch (op) {
                        case ORC_ADD: r = x + y; break;
                        case ORC_SUB: r = x - y; break;
                        case ORC_MUL: r = x * y; break;
                        default: r = x / y; break;
                    }
                    stf(out, dt, io, r);
                }
}

/* ---- scalar ops: ark/ops/ops_scalar_test.cpp:11-62 ---------------------- */
/* The reference rounds the scalar to the storage type first: T(FACTOR). */
ORC_API void orc_scalar(int op, int dt, void *out, const void *in, size_t n, float val) {
    float s = rnd(dt, val);
    for (size_t i = 0; i < n; ++i) {
        float x = ldf(in, dt, i), r;
        switch (op) {
            case ORC_ADD: r = x + s; break;
            case ORC_SUB: r = x - s; break;
            case ORC_MUL: r = x * s; break;
            default: r = x / s; break;
        }
        stf(out, dt, i, r);
    }
}
/* scalar_assign (ops_scalar_test.cpp: test_scalar_assign_*): fill. */
ORC_API void orc_fill(int dt, void *out, size_t n, float val) {
    for (size_t i = 0; i < n; ++i) stf(out, dt, i, val);
}

/* ---- cast: ark/ops/ops_cast_test.cpp:6-45 ------------------------------- */
ORC_API void orc_cast(int from, int to, void *out, const void *in, size_t n) {
    if (from == to) {
        memcpy(out, in, n * dsize(to));
        return;
    }
    int from_int = from >= ORC_I32, to_int = to >= ORC_I32;
    for (size_t i = 0; i < n; ++i) {
        if (from_int && to_int) {
            int64_t v;
            switch (from) {
                case ORC_I32: v = ((const int32_t *)in)[i]; break;
                case ORC_U32: v = ((const uint32_t *)in)[i]; break;
                case ORC_I8: v = ((const int8_t *)in)[i]; break;
                default: v = ((const uint8_t *)in)[i]; break;
            }
            switch (to) {
                case ORC_I32: ((int32_t *)out)[i] = (int32_t)v; break;
                case ORC_U32: ((uint32_t *)out)[i] = (uint32_t)v; break;
                case ORC_I8: ((int8_t *)out)[i] = (int8_t)v; break;
                default: ((uint8_t *)out)[i] = (uint8_t)v; break;
            }
        } else {
            stf(out, to, i, ldf(in, from, i));
        }
    }
}

/* ---- reductions: ark/ops/ops_reduce_test.cpp:10-230 ---------------------- */
enum { ORC_RSUM = 0, ORC_RMAX = 1, ORC_RMEAN = 2 };

/* fp32 accumulation in index order along the axis, one rounding. */
ORC_API void orc_reduce(int kind, int dt, int axis, void *out, const void *in, const int64_t *ish) {
    int64_t st[4] = {ish[1] * ish[2] * ish[3], ish[2] * ish[3], ish[3], 1};
    int64_t osh[4] = {ish[0], ish[1], ish[2], ish[3]};
    osh[axis] = 1;
    int64_t ost[4] = {osh[1] * osh[2] * osh[3], osh[2] * osh[3], osh[3], 1};
    int64_t len = ish[axis];
    for (int64_t n = 0; n < osh[0]; ++n)
        for (int64_t c = 0; c < osh[1]; ++c)
            for (int64_t h = 0; h < osh[2]; ++h)
                for (int64_t w = 0; w < osh[3]; ++w) {
                    size_t base = n * st[0] + c * st[1] + h * st[2] + w * st[3];
                    float acc = (kind == ORC_RMAX) ? -3.402823466e+38f : 0.0f; /* numeric_limits<float>::lowest() */
                    for (int64_t r = 0; r < len; ++r) {
                        float v = ldf(in, dt, base + r * st[axis]);
                        if (kind == ORC_RMAX) acc = acc > v ? acc : v;
                        else acc += v;
                    }
                    if (kind == ORC_RMEAN) acc /= (float)len;
                    stf(out, dt, n * ost[0] + c * ost[1] + h * ost[2] + w * ost[3], acc);
                }
}

/* ---- rope: ark/ops/ops_rope_test.cpp:8-34 ------------------------------- */
/* Storage-type arithmetic: each product and the sum/difference round to T. */
ORC_API void orc_rope(int dt, void *out, const void *in, const void *other, size_t n) {
    for (size_t i = 0; i + 1 < n; i += 2) {
        float a0 = ldf(in, dt, i), a1 = ldf(in, dt, i + 1);
        float b0 = ldf(other, dt, i), b1 = ldf(other, dt, i + 1);
        stf(out, dt, i, rnd(dt, a0 * b0) - rnd(dt, a1 * b1));
        stf(out, dt, i + 1, rnd(dt, a0 * b1) + rnd(dt, a1 * b0));
    }
}

/* ---- transpose: ark/ops/ops_transpose_test.cpp (all 24 permutations) ----- */
/* out dim i = in dim perm[i]; esize = bytes per element. */
ORC_API void orc_transpose(size_t esize, void *out, const void *in, const int64_t *ish, const int *perm) {
    int64_t osh[4];
    for (int i = 0; i < 4; ++i) osh[i] = ish[perm[i]];
    int64_t ist[4] = {ish[1] * ish[2] * ish[3], ish[2] * ish[3], ish[3], 1};
    int64_t idx[4];
    for (idx[0] = 0; idx[0] < osh[0]; ++idx[0])
        for (idx[1] = 0; idx[1] < osh[1]; ++idx[1])
            for (idx[2] = 0; idx[2] < osh[2]; ++idx[2])
                for (idx[3] = 0; idx[3] < osh[3]; ++idx[3]) {
                    size_t io = idx[3] + osh[3] * (idx[2] + osh[2] * (idx[1] + osh[1] * idx[0]));
                    size_t ii = 0;
                    for (int i = 0; i < 4; ++i) ii += idx[i] * ist[perm[i]];
                    memcpy((char *)out + io * esize, (const char *)in + ii * esize, esize);
                }
}

/* ---- embedding: ark/ops/ops_embedding_test.cpp:10-40 --------------------- */
/* Negative indices wrap by the number of rows. */
ORC_API void orc_embedding(size_t esize, void *out, const int32_t *idx, const void *weight, size_t n_idx,
                           int64_t num_emb, int64_t emb_dim) {
    for (size_t i = 0; i < n_idx; ++i) {
        int64_t r = idx[i];
        if (r < 0) r += num_emb;
        memcpy((char *)out + i * emb_dim * esize, (const char *)weight + r * emb_dim * esize, emb_dim * esize);
    }
}

/* ---- matmul: restatement of blas_matmul semantics ------------------------ */
/* ark/ops/ops_matmul_test.cpp:124-174: C[m,n] = A·B per batch, row-major
 * storage; A is [m,k] (or [k,m] when trans_a), B is [k,n] (or [n,k] when
 * trans_b); leading dimensions lda/ldb/ldc in elements; batch strides in
 * elements (0 = broadcast). The reference's own check runs cuBLAS; this
 * restatement accumulates in fp32 in k order and rounds once, which is the
 * contract the engine's kernels are held to. act: 0 none, 1 relu, 2 gelu
 * (applied on the fp32 accumulator before the rounding, used for the fused
 * epilogue checks). Rows are split over OpenMP threads. */
ORC_API void orc_matmul(int dt, void *C, const void *A, const void *B, int64_t batch, int64_t m, int64_t n,
                        int64_t k, int trans_a, int trans_b, int64_t lda, int64_t ldb, int64_t ldc,
                        int64_t sa, int64_t sb, int64_t sc, int act) {
    for (int64_t bi = 0; bi < batch; ++bi) {
        /* widen the operands once so the inner loop is pure fp32 */
        float *Af = (float *)malloc(sizeof(float) * m * k);
        float *Bf = (float *)malloc(sizeof(float) * k * n);
#pragma omp parallel for
        for (int64_t i = 0; i < m; ++i)
            for (int64_t p = 0; p < k; ++p)
                Af[i * k + p] = ldf(A, dt, bi * sa + (trans_a ? p * lda + i : i * lda + p));
#pragma omp parallel for
        for (int64_t p = 0; p < k; ++p)
            for (int64_t j = 0; j < n; ++j)
                Bf[p * n + j] = ldf(B, dt, bi * sb + (trans_b ? j * ldb + p : p * ldb + j));
#pragma omp parallel for schedule(dynamic, 1)
        for (int64_t i = 0; i < m; ++i) {
            float *acc = (float *)calloc(n, sizeof(float));
            for (int64_t p = 0; p < k; ++p) {
                float a = Af[i * k + p];
                const float *brow = Bf + p * n;
                for (int64_t j = 0; j < n; ++j) acc[j] += a * brow[j];
            }
            for (int64_t j = 0; j < n; ++j) {
                float v = acc[j];
                if (act == 1) v = v > 0 ? v : 0;
                else if (act == 2) v = gelu_ref(v);
                stf(C, dt, bi * sc + i * ldc + j, v);
            }
            free(acc);
        }
        free(Af);
        free(Bf);
    }
}

/* ---- all_reduce: exact fp32 sum of the rank inputs, one rounding --------- */
/* Reference pins: ark/ops/ops_all_reduce_test.cpp:9-24 (rank r holds r+1,
 * every element of the result equals the closed-form sum, exact equality). */
ORC_API void orc_all_reduce(int dt, void *out, const void *const *ins, int nranks, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float acc = 0;
        for (int r = 0; r < nranks; ++r) acc += ldf(ins[r], dt, i);
        stf(out, dt, i, acc);
    }
}

/* ---- fused rows (compositions kept in fp32, one rounding at the end) ----- */
/* RMSNorm as composed by examples/llama/model.py:92-99:
 *   x32 = cast(x); mean = reduce_mean(x32*x32, -1); y = x32 * rsqrt(mean + eps) * w; cast back.
 * (The reference example drops eps; it is an explicit argument here.) */
ORC_API void orc_rmsnorm(int dt, void *out, const void *in, const void *weight, int64_t rows, int64_t cols,
                         float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        float ss = 0;
        for (int64_t j = 0; j < cols; ++j) {
            float v = ldf(in, dt, r * cols + j);
            ss += v * v;
        }
        float inv = 1.0f / sqrtf(ss / (float)cols + eps);
        for (int64_t j = 0; j < cols; ++j) {
            float v = ldf(in, dt, r * cols + j) * inv;
            if (weight) v *= ldf(weight, dt, j);
            stf(out, dt, r * cols + j, v);
        }
    }
}
/* softmax over the last axis: python/ark/ops.py:491-500
 *   (x - max) -> exp -> / sum, here with fp32 intermediates. */
ORC_API void orc_softmax(int dt, void *out, const void *in, int64_t rows, int64_t cols) {
    for (int64_t r = 0; r < rows; ++r) {
        float mx = -3.402823466e+38f, s = 0;
        for (int64_t j = 0; j < cols; ++j) {
            float v = ldf(in, dt, r * cols + j);
            mx = mx > v ? mx : v;
        }
        for (int64_t j = 0; j < cols; ++j) s += expf(ldf(in, dt, r * cols + j) - mx);
        for (int64_t j = 0; j < cols; ++j) stf(out, dt, r * cols + j, expf(ldf(in, dt, r * cols + j) - mx) / s);
    }
}
/* layernorm over the last axis: python/ark/ops.py:503-513
 *   mean -> x-mean -> mean of squares -> rsqrt(var + eps) -> scale. */
ORC_API void orc_layernorm(int dt, void *out, const void *in, int64_t rows, int64_t cols, float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        float mean = 0, var = 0;
        for (int64_t j = 0; j < cols; ++j) mean += ldf(in, dt, r * cols + j);
        mean /= (float)cols;
        for (int64_t j = 0; j < cols; ++j) {
            float d = ldf(in, dt, r * cols + j) - mean;
            var += d * d;
        }
        float inv = 1.0f / sqrtf(var / (float)cols + eps);
        for (int64_t j = 0; j < cols; ++j) stf(out, dt, r * cols + j, (ldf(in, dt, r * cols + j) - mean) * inv);
    }
}
