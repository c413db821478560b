// Attention of one new token per sequence against a K/V cache (the decode
// step): out[b, h] = softmax(scale * q[b, h] . K[b, h / G]^T) . V[b, h / G]
// with G = Hq / Hkv query heads sharing a K/V head and a head size of 128.
// The reference builds this from two Matmuls, a scale and a softmax
// (examples/llama/model.py:336-444), i.e. several tasks with barriers between
// them; at one query row per head those tasks are nothing but a read of the
// cache, so this stage does the whole thing around that read:
//   phase 0  a CTA takes one (sequence, K/V head, chunk of the cache): scores of
//            the chunk for the G query heads (half a warp per key, fp32), their
//            maximum and exp-sum, and the chunk's un-normalised output; written
//            to scratch as fp32 (output, maximum, sum);
//   phase 1  after a barrier, the chunks of a head are merged with the usual
//            max/sum rescaling and the result is rounded once.
// K and V are read exactly once, 16 bytes per lane, rows contiguous.
#include "dev_common.cuh"
#include "dev_funcs.h"

namespace arkb {

namespace {

constexpr int kHeadDim = 128;     // elements per head (16 lanes x 8)
constexpr int kMaxGroup = 8;      // query heads per K/V head


template <typename T, int G>
__device__ __noinline__ void attn_chunks(const DecodeAttnArgs &a, int p, int P, char *smem) {
    constexpr int D = kHeadDim;
    float *qs = reinterpret_cast<float *>(smem);                 // [G][D], already scaled
    float *ml = qs + G * D;                                      // [G][2]: maximum, exp-sum
    float *sc = ml + 2 * kMaxGroup;                              // [G][chunk_len]
    float *red = sc + (size_t)G * a.chunk_len;                   // [16][G][D]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hw = tid >> 4, l16 = tid & 15;                     // half-warp index 0..31, lane within it
    const int items = a.B * a.Hkv * a.chunks;
    const T *qb = reinterpret_cast<const T *>(a.q);
    const T *kb = reinterpret_cast<const T *>(a.k);
    const T *vb = reinterpret_cast<const T *>(a.v);
    for (int item = p; item < items; item += P) {
        const int c = item % a.chunks, bh = item / a.chunks;
        const int kvh = bh % a.Hkv, b = bh / a.Hkv;
        const int t0 = c * a.chunk_len, len = min(a.chunk_len, a.T - t0);
        __syncthreads();  // the previous item's shared memory is no longer read
        for (int i = tid; i < G * D / 8; i += blockDim.x) {
            const int g = i / (D / 8), v = i % (D / 8);
            const uint4 q4 = *reinterpret_cast<const uint4 *>(qb + (int64_t)b * a.q_stride_b + (int64_t)(kvh * G + g) * a.q_stride_h + v * 8);
            float f[8];
            unpack8<T>(q4, f);
            if (a.rope) {
                // rotary embedding of the new token's query (complex multiply of adjacent pairs with the position's
                // (cos, sin) pairs), rounded like the separate operator would have stored it
                float t[8];
                unpack8<T>(*reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(a.rope) + v * 8), t);
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const float re = f[e] * t[e] - f[e + 1] * t[e + 1], im = f[e] * t[e + 1] + f[e + 1] * t[e];
                    f[e] = to_f32(from_f32<T>(re));
                    f[e + 1] = to_f32(from_f32<T>(im));
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) qs[g * D + v * 8 + e] = f[e] * a.scale;
        }
        __syncthreads();
        // scores: half a warp per key, 4 keys in flight
        const T *kbase = kb + (int64_t)b * a.k_stride_b + (int64_t)kvh * a.k_stride_h + (int64_t)t0 * a.k_ld + l16 * 8;
        float qr[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) qr[g][e] = qs[g * D + l16 * 8 + e];
        for (int jb = 2 * warp; jb < len; jb += 32 * 4) {  // same trip count in both halves of a warp (shuffles below)
            const int j0 = jb + (hw & 1);
            uint4 k4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + 32 * u;
                k4[u] = j < len ? ldg16_stream(kbase + (int64_t)j * a.k_ld) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + 32 * u;
                float f[8];
                unpack8<T>(k4[u], f);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float s = 0.0f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) s += qr[g][e] * f[e];
                    s += __shfl_xor_sync(0xffffffffu, s, 8);
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    if (l16 == 0 && j < len) sc[(size_t)g * a.chunk_len + j] = s;
                }
            }
        }
        __syncthreads();
        // per query head: maximum, exponentials in place, their sum (warp g)
        if (warp < G) {
            float *row = sc + (size_t)warp * a.chunk_len;
            float m = -3.402823466e+38f;
            for (int j = lane; j < len; j += 32) m = fmaxf(m, row[j]);
            m = warp_max(m);
            float l = 0.0f;
            for (int j = lane; j < len; j += 32) {
                const float e = __expf(row[j] - m);
                row[j] = e;
                l += e;
            }
            l = warp_sum(l);
            if (lane == 0) {
                ml[warp * 2] = m;
                ml[warp * 2 + 1] = l;
            }
        }
        __syncthreads();
        // un-normalised output: lanes of a half-warp cover the 128 columns, the 32 half-warps interleave the keys
        const T *vbase = vb + (int64_t)b * a.v_stride_b + (int64_t)kvh * a.v_stride_h + (int64_t)t0 * a.v_ld + l16 * 8;
        float acc[G][8];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
        for (int jb = 2 * warp; jb < len; jb += 32 * 4) {
            const int j0 = jb + (hw & 1);
            uint4 v4[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + 32 * u;
                v4[u] = j < len ? ldg16_stream(vbase + (int64_t)j * a.v_ld) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = j0 + 32 * u;
                if (j < len) {
                    float f[8];
                    unpack8<T>(v4[u], f);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const float pj = sc[(size_t)g * a.chunk_len + j];
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[g][e] += pj * f[e];
                    }
                }
            }
        }
        // the two half-warps of a warp hold the same columns: add them, then the 16 warps through shared memory
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], 16);
        if (lane < 16) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float4 *dst = reinterpret_cast<float4 *>(red + ((size_t)warp * G + g) * D + l16 * 8);
                dst[0] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
                dst[1] = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
            }
        }
        __syncthreads();
        float *w = a.ws + (size_t)item * G * (D + 2);
        const int nwarps = blockDim.x >> 5;
        for (int i = tid; i < G * D; i += blockDim.x) {
            float s = 0.0f;
            for (int wi = 0; wi < nwarps; ++wi) s += red[(size_t)wi * G * D + i];
            w[i] = s;  // [g][d]
        }
        if (tid < 2 * G) w[G * D + tid] = ml[tid];  // [g][maximum, sum]
    }
}

// Merges the chunks of every (sequence, query head): thread per output element.
template <typename T>
__device__ void attn_merge(const DecodeAttnArgs &a, int p, int P) {
    constexpr int D = kHeadDim;
    const int G = a.Hq / a.Hkv;
    const int64_t total = (int64_t)a.B * a.Hq * D;
    T *out = reinterpret_cast<T *>(a.out);
    for (int64_t i = (int64_t)p * blockDim.x + threadIdx.x; i < total; i += (int64_t)P * blockDim.x) {
        const int d = (int)(i % D);
        const int h = (int)((i / D) % a.Hq), b = (int)(i / ((int64_t)D * a.Hq));
        const int kvh = h / G, g = h % G;
        const float *w = a.ws + ((size_t)(b * a.Hkv + kvh) * a.chunks) * G * (D + 2);
        const size_t stride = (size_t)G * (D + 2);
        float m = -3.402823466e+38f;
        for (int c = 0; c < a.chunks; ++c) m = fmaxf(m, w[c * stride + G * D + 2 * g]);
        float l = 0.0f, o = 0.0f;
        for (int c = 0; c < a.chunks; ++c) {
            const float f = __expf(w[c * stride + G * D + 2 * g] - m);
            l += w[c * stride + G * D + 2 * g + 1] * f;
            o += w[c * stride + g * D + d] * f;
        }
        out[(int64_t)b * a.o_stride_b + (int64_t)h * a.o_stride_h + d] = from_f32<T>(o / l);
    }
}

template <typename T>
__device__ void attn_typed(const DecodeAttnArgs &a, int p, int P, char *smem) {
    if (a.phase == 1) return attn_merge<T>(a, p, P);
    switch (a.Hq / a.Hkv) {
        case 1: return attn_chunks<T, 1>(a, p, P, smem);
        case 2: return attn_chunks<T, 2>(a, p, P, smem);
        case 4: return attn_chunks<T, 4>(a, p, P, smem);
        default: return attn_chunks<T, 8>(a, p, P, smem);
    }
}

}  // namespace

__device__ __noinline__ void run_decode_attn(const DecodeAttnArgs &a, int p, int P, char *smem) {
    if (a.dtype == DT_BF16) attn_typed<__nv_bfloat16>(a, p, P, smem);
    else attn_typed<__half>(a, p, P, smem);
}

}  // namespace arkb
