// Causal / full self-attention over many query rows in one stage (prefill): S = Q K^T on the tensor cores into
// TMEM, an online softmax on the CUDA cores straight out of TMEM, P (rounded to the storage type) back through shared
// memory as the A operand of O += P V. The scores never reach global memory.
//
// Stands for the reference's matmul -> scale -> mask add -> softmax -> matmul chain of one attention block
// (examples/llama/model.py:336-444 of the reference; ops at ark/ops/ops_matmul.cc, ops_softmax.cc), whose scores
// tensor [B, H, T, T] costs two HBM round trips per layer.
//
// One unit = 128 query rows of one (batch, head). Per unit the CTA walks the 128-key tiles the rows may attend to
// (causal: up to the diagonal) with four roles:
//   warp 4 lane 0 : TMA producer — Q once per unit, K and V tiles into a two-slot ring;
//   warp 5 lane 0 : MMA issuer   — S(j+1) = Q K(j+1)^T is issued before it waits for P(j), so the tensor cores
//                   work on the next scores while the softmax warps work on the current ones (two S buffers);
//   warps 0..3, 8..11 : softmax — two warps per 32 query rows (TMEM lanes), 64 columns each: running maximum m
//                   (exchanged between the two through shared memory) and sum l, O rescaled in TMEM by
//                   exp2(m_old - m_new) when the maximum moved, P = exp2(s*c - m) rounded and written into the
//                   128-byte-swizzled K-major layout the MMA reads; after the last tile O / l goes to global.
// TMEM columns: S0 [0,128), S1 [128,256), O [256,384). Shared memory: Q 32 KiB, 2 x (K 32 KiB + V 32 KiB), P 32 KiB.
// The barriers live behind the tiles and exist only for the duration of the stage. Every wait is bounded.
#include "dev_gemm.cuh"

namespace arkb {

namespace {

constexpr int kAtTile = 128;                       // query rows per unit, keys per tile, head dimension
constexpr int kAtTileBytes = kAtTile * kAtTile * 2;  // 32 KiB: one 128 x 128 tile of 16-bit values
constexpr int kAtQOff = 0;
constexpr int kAtKvOff = kAtTileBytes;              // slot s: K at +s*64 KiB, V 32 KiB behind it
constexpr int kAtPOff = kAtKvOff + 4 * kAtTileBytes;
constexpr int kAtBarOff = kAtPOff + kAtTileBytes;   // 192 KiB
constexpr int kAtXchOff = kAtBarOff + 256;          // row maxima [2][2][128] and row sums [2][2][128] exchanged between the two warps of a row
constexpr int kAtSoftmaxWarps = 8;
constexpr uint32_t kAtS0 = 0, kAtO = 256;

struct AttnBars {
    unsigned long long q_full, q_empty, kv_full[2], kv_empty[2], s_full[2], s_free[2], p_ready, o_done, o_free;
};
static_assert(sizeof(AttnBars) <= 256 && kAtXchOff + 1024 * (int)sizeof(float) <= kGemmSmemBytes, "attention tiles and barriers fit the kernel's shared memory");

struct AttnRun {
    const PrefillAttnArgs *a;      // stage record (shared-memory copy)
    const PrefillAttnArgs *amaps;  // the record in global memory (tensor maps)
    char *smem;
    AttnBars *bars;
    CtaCtl *ctl;
    DeviceState *st;
    unsigned long long lim;
    int stage_idx, p, P;
    uint32_t tmem_base;
};

struct AttnUnit {
    int b, h, hkv, qt, n_tiles;
};

__device__ __forceinline__ AttnUnit attn_unit(const PrefillAttnArgs &a, int u) {
    // longest units first: with a causal mask the last query tile attends to the most keys
    AttnUnit t;
    const int bh = a.B * a.Hq;
    t.qt = a.q_tiles - 1 - u / bh;
    const int r = u % bh;
    t.b = r / a.Hq;
    t.h = r % a.Hq;
    t.hkv = t.h / (a.Hq / a.Hkv);
    const int all = (a.Tkv + kAtTile - 1) / kAtTile;
    if (a.causal) {
        // row i sees keys [0, i + Tkv - Tq]
        const int last_key = min(a.Tkv - 1, t.qt * kAtTile + kAtTile - 1 + a.Tkv - a.Tq);
        t.n_tiles = last_key < 0 ? 0 : min(all, last_key / kAtTile + 1);
    } else {
        t.n_tiles = all;
    }
    return t;
}

__device__ __forceinline__ bool attn_fail(const AttnRun &R) {
    R.ctl->abort = 1;
    report(R.st, ST_MBAR_TIMEOUT, R.stage_idx);
    return false;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- producer ------------------------------------------------------------------------------
__device__ __noinline__ bool attn_produce(const AttnRun &R) {
    const PrefillAttnArgs &a = *R.a;
    AttnBars *B = R.bars;
    const CUtensorMap *tmQ = &R.amaps->tmQ, *tmK = &R.amaps->tmK, *tmV = &R.amaps->tmV;
    unsigned int uc = 0, kc = 0;  // units and key tiles this CTA has staged
    for (int u = R.p; u < a.n_units; u += R.P) {
        const AttnUnit t = attn_unit(a, u);
        if (t.n_tiles == 0) continue;
        if (!mbar_wait(&B->q_empty, (uc & 1) ^ 1, R.lim)) return attn_fail(R);
        mbar_expect_tx(&B->q_full, kAtTileBytes);
        char *sQ = R.smem + kAtQOff;
        tma_load_4d(sQ, tmQ, &B->q_full, 0, t.qt * kAtTile, t.h, t.b);
        tma_load_4d(sQ + kGemmABytes, tmQ, &B->q_full, 64, t.qt * kAtTile, t.h, t.b);
        ++uc;
        for (int j = 0; j < t.n_tiles; ++j, ++kc) {
            const int s = kc & 1;
            if (!mbar_wait(&B->kv_empty[s], ((kc >> 1) & 1) ^ 1, R.lim)) return attn_fail(R);
            mbar_expect_tx(&B->kv_full[s], 2 * kAtTileBytes);
            char *sK = R.smem + kAtKvOff + s * 2 * kAtTileBytes, *sV = sK + kAtTileBytes;
            const int key0 = j * kAtTile;
            // K as the K-major B operand of S = Q K^T: two blocks of 64 head-dimension elements x 128 keys
            tma_load_4d(sK, tmK, &B->kv_full[s], 0, key0, t.hkv, t.b);
            tma_load_4d(sK + kGemmABytes, tmK, &B->kv_full[s], 64, key0, t.hkv, t.b);
            // V as the MN-major B operand of O = P V: per block of 64 keys two chunks of 64 head-dimension columns
            for (int kb = 0; kb < 2; ++kb)
                for (int c = 0; c < 2; ++c)
                    tma_load_4d(sV + kb * 16384 + c * 8192, tmV, &B->kv_full[s], c * 64, key0 + kb * 64, t.hkv, t.b);
        }
    }
    // drain: the MMA thread's last commits on kv_empty / q_empty arrive asynchronously; they must have landed before
    // the barriers are given up at the end of the stage
    for (unsigned int i = kc >= 2 ? kc - 2 : 0; i < kc; ++i)
        if (!mbar_wait(&B->kv_empty[i & 1], (i >> 1) & 1, R.lim)) return attn_fail(R);
    if (uc > 0 && !mbar_wait(&B->q_empty, (uc - 1) & 1, R.lim)) return attn_fail(R);
    return true;
}

// ---- MMA issue -----------------------------------------------------------------------------
__device__ __noinline__ bool attn_issue(const AttnRun &R) {
    const PrefillAttnArgs &a = *R.a;
    AttnBars *B = R.bars;
    const int bf16 = a.dtype == DT_BF16;
    const uint32_t idesc_s = umma_idesc(bf16, 0, 0, kAtTile, kAtTile);   // Q, K both K-major
    const uint32_t idesc_o = umma_idesc(bf16, 0, 1, kAtTile, kAtTile);   // P K-major, V MN-major
    const uint32_t sQ = smem_u32(R.smem + kAtQOff), sP = smem_u32(R.smem + kAtPOff);
    const uint32_t tm = R.tmem_base;
    unsigned int uc = 0, sc = 0, kc_s = 0, kc_o = 0, pc = 0;  // units; S tiles issued; key tiles used by S / by PV; P tiles consumed

    auto issue_s = [&]() -> bool {
        const int slot = kc_s & 1, sb = sc & 1;
        if (!mbar_wait(&B->kv_full[slot], (kc_s >> 1) & 1, R.lim)) return false;
        if (!mbar_wait(&B->s_free[sb], ((sc >> 1) & 1) ^ 1, R.lim)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(R.smem + kAtKvOff + slot * 2 * kAtTileBytes);
        const uint32_t d = tm + kAtS0 + sb * kAtTile;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            const uint64_t da = umma_desc(sQ + kb * kGemmABytes, 16, 1024), db = umma_desc(sK + kb * kGemmABytes, 16, 1024);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_f16(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc_s, (kb | kk) ? 1u : 0u);
        }
        umma_commit(&B->s_full[sb]);
        ++kc_s;
        ++sc;
        return true;
    };

    for (int u = R.p; u < a.n_units; u += R.P) {
        const AttnUnit t = attn_unit(a, u);
        if (t.n_tiles == 0) continue;
        if (!mbar_wait(&B->q_full, uc & 1, R.lim)) return attn_fail(R);
        if (!issue_s()) return attn_fail(R);
        for (int j = 0; j < t.n_tiles; ++j, ++kc_o, ++pc) {
            if (j + 1 < t.n_tiles) {
                if (!issue_s()) return attn_fail(R);
            } else {
                umma_commit(&B->q_empty);  // every S of this unit has been issued: Q may be replaced once they are done
            }
            if (!mbar_wait(&B->p_ready, pc & 1, R.lim)) return attn_fail(R);
            if (j == 0 && !mbar_wait(&B->o_free, (uc & 1) ^ 1, R.lim)) return attn_fail(R);
            tc_fence_after();
            const int slot = kc_o & 1;
            const uint32_t sV = smem_u32(R.smem + kAtKvOff + slot * 2 * kAtTileBytes + kAtTileBytes);
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                const uint64_t da = umma_desc(sP + kb * kGemmABytes, 16, 1024), db = umma_desc(sV + kb * 16384, 8192, 1024);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_f16(tm + kAtO, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 128), idesc_o, (j | kb | kk) ? 1u : 0u);
            }
            umma_commit(&B->kv_empty[slot]);
            umma_commit(&B->o_done);
        }
        ++uc;
    }
    return true;
}

// ---- softmax and output -------------------------------------------------------------------------
// Eight warps: warps 0-3 (half 0) and 8-11 (half 1). Warp q + 8*half owns TMEM lanes 32q..32q+31 (the only ones a warp
// with index = q mod 4 can reach) = query rows 32q.. of the tile, and columns 64*half..+63 of S, P and O. The two warps
// of a row exchange their partial row maxima through shared memory; the partial sums stay apart until the end.
template <typename T>
__device__ __noinline__ bool attn_softmax(const AttnRun &R, int warp, int lane) {
    const PrefillAttnArgs &a = *R.a;
    AttnBars *B = R.bars;
    const int quarter = warp & 3, half = warp >> 3;
    const int row = quarter * 32 + lane;
    const int col0 = half * 64;
    const uint32_t lane_addr = R.tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float c = a.scale * 1.4426950408889634f;  // scores are kept in units of log2(e): exp(x) = exp2(x * log2 e)
    char *sP = R.smem + kAtPOff;
    float *xch = reinterpret_cast<float *>(R.smem + kAtXchOff);  // [2 parities][2 halves][128 rows]
    unsigned int sc = 0, oc = 0;  // S tiles consumed; PV commits waited for
    for (int u = R.p; u < a.n_units; u += R.P) {
        const AttnUnit t = attn_unit(a, u);
        const int qi = t.qt * kAtTile + row;
        T *orow = reinterpret_cast<T *>(a.out) + (int64_t)t.b * a.o_stride_b + (int64_t)t.h * a.o_stride_h + (int64_t)qi * a.o_stride_t + col0;
        if (t.n_tiles == 0) {  // no key visible to any row of the tile: zeros
            if (qi < a.Tq)
                for (int i = 0; i < 64; i += 8) *reinterpret_cast<uint4 *>(orow + i) = make_uint4(0, 0, 0, 0);
            continue;
        }
        const int last_key = a.causal ? min(a.Tkv - 1, qi + a.Tkv - a.Tq) : a.Tkv - 1;  // last key this row may see
        float m = -INFINITY, l = 0.0f;
        for (int j = 0; j < t.n_tiles; ++j, ++sc) {
            const int sb = sc & 1;
            bool ok = mbar_wait(&B->s_full[sb], (sc >> 1) & 1, R.lim);
            if (!__all_sync(0xffffffffu, ok)) {
                if (lane == 0) attn_fail(R);
                return false;
            }
            tc_fence_after();
            const uint32_t s_addr = lane_addr + kAtS0 + sb * kAtTile + col0;
            const int key0 = j * kAtTile + col0;  // first key of this warp's columns
            // masking is needed when these columns hold a key some row of this warp may not see
            const bool masked = key0 + 63 > __shfl_sync(0xffffffffu, last_key, 0);
            uint32_t r0[32], r1[32];
            tmem_ld32(s_addr, r0);
            tmem_ld32(s_addr + 32, r1);
            tmem_ld_wait();
            // scaled (and masked) scores stay in r0 / r1 as float bits until the exponentials
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float a0 = __uint_as_float(r0[i]) * c, a1 = __uint_as_float(r1[i]) * c;
                if (masked) {
                    if (key0 + i > last_key) a0 = -INFINITY;
                    if (key0 + 32 + i > last_key) a1 = -INFINITY;
                }
                r0[i] = __float_as_uint(a0);
                r1[i] = __float_as_uint(a1);
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])));
            const float mx_own = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            float *x = xch + (sc & 1) * 256;
            x[half * 128 + row] = mx_own;
            named_barrier(1 + quarter, 64);
            const float mx = fmaxf(m, fmaxf(mx_own, x[(half ^ 1) * 128 + row]));
            // a row with no visible key so far keeps m = -inf; the exponentials below then see -inf - 0 and give 0
            const float m_use = mx == -INFINITY ? 0.0f : mx;
            const float alpha = ex2(m - m_use);  // m = -inf on the first tile: 0
            // PV of the previous tile must be complete: it reads P and writes O
            if (j > 0) {
                ok = mbar_wait(&B->o_done, oc & 1, R.lim);
                if (!__all_sync(0xffffffffu, ok)) {
                    if (lane == 0) attn_fail(R);
                    return false;
                }
                ++oc;
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    // r0 / r1 still hold the scores: O passes through registers of its own, 32 columns at a time
#pragma unroll 1
                    for (int cc = 0; cc < 2; ++cc) {
                        uint32_t t32[32];
                        tmem_ld32(lane_addr + kAtO + col0 + cc * 32, t32);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) t32[i] = __float_as_uint(__uint_as_float(t32[i]) * alpha);
                        tmem_st32(lane_addr + kAtO + col0 + cc * 32, t32);
                    }
                    tmem_st_wait();
                }
            }
            l *= alpha;
            m = mx;
            // P = exp2(v - m), rounded to the storage type; this warp's 64 keys are k-block `half` of the A operand:
            // row `row`, 16-byte chunks 0..7 of its 128-byte line, 128-byte swizzle
            char *prow = sP + half * kGemmABytes + row * 128;
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int q = 0; q < 8; ++q) {  // eight values = one 16-byte chunk of the line
                union { uint4 v; T e[8]; } o;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t bits = q < 4 ? r0[q * 8 + i] : r1[(q - 4) * 8 + i];
                    o.e[i] = from_f32<T>(ex2(__uint_as_float(bits) - m_use));
                    l4[i & 3] += to_f32(o.e[i]);  // the sum of what the MMA will multiply
                }
                *reinterpret_cast<uint4 *>(prow + ((q ^ (row & 7)) << 4)) = o.v;
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            tc_fence_before();
            fence_async_smem();  // P was written through the generic proxy; the MMA reads it through the async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&B->s_free[sb]);
                mbar_arrive(&B->p_ready);
            }
        }
        // the last PV
        bool ok = mbar_wait(&B->o_done, oc & 1, R.lim);
        if (!__all_sync(0xffffffffu, ok)) {
            if (lane == 0) attn_fail(R);
            return false;
        }
        ++oc;
        tc_fence_after();
        // the row's sum: both halves, added in the same order by both warps
        float *x = xch + 512 + (oc & 1) * 256;
        x[half * 128 + row] = l;
        named_barrier(1 + quarter, 64);
        const float lsum = x[row] + x[128 + row];
        const float inv = lsum > 0.0f ? 1.0f / lsum : 0.0f;
        uint32_t r0[32], r1[32];
        tmem_ld32(lane_addr + kAtO + col0, r0);
        tmem_ld32(lane_addr + kAtO + col0 + 32, r1);
        tmem_ld_wait();
        if (qi < a.Tq) {
            union { uint4 q[4]; T e[32]; } o;
#pragma unroll
            for (int i = 0; i < 32; ++i) o.e[i] = from_f32<T>(__uint_as_float(r0[i]) * inv);
#pragma unroll
            for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4 *>(orow + q * 8) = o.q[q];
#pragma unroll
            for (int i = 0; i < 32; ++i) o.e[i] = from_f32<T>(__uint_as_float(r1[i]) * inv);
#pragma unroll
            for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4 *>(orow + 32 + q * 8) = o.q[q];
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&B->o_free);
    }
    return true;
}

}  // namespace

__device__ __noinline__ void run_prefill_attn(const PrefillAttnArgs &a, const PrefillAttnArgs *amaps, int p, int P, char *smem,
                                              CtaCtl *ctl, DeviceState *st, int stage_idx, unsigned long long lim) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    AttnRun R;
    R.a = &a; R.amaps = amaps; R.smem = smem; R.bars = reinterpret_cast<AttnBars *>(smem + kAtBarOff);
    R.ctl = ctl; R.st = st; R.lim = lim; R.stage_idx = stage_idx; R.p = p; R.P = P; R.tmem_base = ctl->tmem_base;
    AttnBars *B = R.bars;
    if (threadIdx.x == 0) {
        mbar_init(&B->q_full, 1); mbar_init(&B->q_empty, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&B->kv_full[s], 1); mbar_init(&B->kv_empty[s], 1);
            mbar_init(&B->s_full[s], 1); mbar_init(&B->s_free[s], kAtSoftmaxWarps);
        }
        mbar_init(&B->p_ready, kAtSoftmaxWarps); mbar_init(&B->o_done, 1); mbar_init(&B->o_free, kAtSoftmaxWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == kProducerWarp) {
        if (lane == 0) attn_produce(R);
    } else if (warp == kMmaWarp) {
        if (lane == 0) attn_issue(R);
    } else if (warp < kEpiWarps || (warp >= 8 && warp < 12)) {
        if (a.dtype == DT_BF16) attn_softmax<__nv_bfloat16>(R, warp, lane);
        else attn_softmax<__half>(R, warp, lane);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0) {
        // the bytes go back to being plain shared memory for the stages that follow
        unsigned long long *b = reinterpret_cast<unsigned long long *>(B);
        for (int i = 0; i < (int)(sizeof(AttnBars) / 8); ++i)
            asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(b + i)) : "memory");
    }
    __syncthreads();
}

}  // namespace arkb
