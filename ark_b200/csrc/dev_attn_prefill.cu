// Causal / full self-attention over many query rows in one stage (prefill): S = Q K^T on the tensor cores into
// tensor memory, an online softmax on the CUDA cores straight out of it, P (rounded to the storage type) written back
// into the same tensor-memory columns and used from there as the A operand of O += P V. Neither the scores nor the
// probabilities ever reach shared or global memory.
//
// Stands for the reference's matmul -> scale -> mask add -> softmax -> matmul chain of one attention block
// (examples/llama/model.py:336-444 of the reference; ops at ark/ops/ops_matmul.cc, ops_softmax.cc), whose scores
// tensor [B, H, T, T] costs two HBM round trips per layer.
//
// One unit = 128 query rows of one (batch, head). Per unit the CTA walks the 128-key tiles the rows may attend to
// (causal: up to the diagonal). Roles:
//   warp 4 lane 0 : TMA producer of Q (once per unit) and of the K tiles (ring of 3);
//   warp 6 lane 0 : TMA producer of the V tiles (ring of 2);
//   warp 5 lane 0 : MMA issuer. S(j+2) = Q K(j+2)^T is issued right behind P(j) V(j): the tensor cores always have
//                   the scores of the next two tiles done or in flight while the softmax warps work on tile j;
//   warps 0..3, 8..11 : softmax — two warps per 32 query rows (TMEM lanes), 64 columns each. They read S(j), find
//                   the row maximum (the two warps of a row exchange theirs through shared memory), and write
//                   P(j) = exp2(s*c - m) as packed 16-bit pairs over the first 64 columns of S(j). The running
//                   maximum m only moves when the new one exceeds it by more than 8 (a factor 256, harmless in fp32
//                   sums and in fp16 / bf16 P): O then needs rescaling in TMEM only a few times per unit, and only
//                   then does a softmax warp wait for the previous P V to finish. After the last tile O / l goes to
//                   global memory.
// TMEM columns: S/P buffer 0 [0,128), buffer 1 [128,256), O [256,384). Shared memory: Q 32 KiB, 3 x K 32 KiB,
// 2 x V 32 KiB. The barriers live behind the tiles and exist only for the duration of the stage. Every wait is bounded.
#include "dev_gemm.cuh"

namespace arkb {

namespace {

constexpr int kAtTile = 128;                       // query rows per unit, keys per tile, head dimension
constexpr int kAtTileBytes = kAtTile * kAtTile * 2;  // 32 KiB: one 128 x 128 tile of 16-bit values
constexpr int kAtKSlots = 3, kAtVSlots = 2;
constexpr int kAtQOff = 0;
constexpr int kAtKOff = kAtTileBytes;
constexpr int kAtVOff = kAtKOff + kAtKSlots * kAtTileBytes;
constexpr int kAtBarOff = kAtVOff + kAtVSlots * kAtTileBytes;   // 192 KiB
constexpr int kAtXchOff = kAtBarOff + 256;          // row maxima [2][2][128] and row sums [2][2][128] exchanged between the two warps of a row
constexpr int kAtSoftmaxWarps = 8;
constexpr uint32_t kAtS0 = 0, kAtO = 256;
constexpr float kAtLazy = 8.0f;  // the running maximum follows the true one when it lags by more than this (log2 units)

struct AttnBars {
    unsigned long long q_full, q_empty, k_full[kAtKSlots], k_empty[kAtKSlots], v_full[kAtVSlots], v_empty[kAtVSlots];
    // p_ready[i & 1]: P of tile number i is written; o_done[i & 1]: P V number i is complete. Two barriers each, taken
    // in turn: the softmax warps can finish tile i+1 before the MMA thread has seen tile i's arrival, and a parity wait
    // can tell a phase from the next one only.
    unsigned long long s_full[2], p_ready[2], o_done[2], o_free;
};
static_assert(sizeof(AttnBars) <= 256 && kAtXchOff + 1024 * (int)sizeof(float) <= kGemmSmemBytes,
              "attention tiles and barriers fit the kernel's shared memory");

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

// Units are sorted by length (longest first); CTA p takes one unit per round, walking the rounds back and forth, so
// that the CTA with the longest unit of one round gets the shortest of the next.
__device__ __forceinline__ int attn_unit_of(int p, int P, int rnd) {
    return rnd * P + ((rnd & 1) ? P - 1 - p : p);
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld16x(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// D[tmem] (+)= A[tmem] . B[smem]: the A operand (128 rows = lanes, K = 16 elements = 8 columns of packed pairs) is read
// from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p; }"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}

// Two probabilities rounded to the storage type and packed (low half = first key); `sum` gets their fp32 values (the
// rounding errors of the packed values, relative 2^-11 or 2^-8 each and of both signs, average out over a row).
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi, float &sum);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi, float &sum) {
    const __half2 h = __floats2half2_rn(lo, hi);
    sum += lo + hi;
    return *reinterpret_cast<const uint32_t *>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi, float &sum) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    sum += lo + hi;
    return *reinterpret_cast<const uint32_t *>(&h);
}

// ---- producers -----------------------------------------------------------------------------
// Q and the K ring (warp 4), or the V ring (warp 6).
__device__ __noinline__ bool attn_produce(const AttnRun &R, bool is_v) {
    const PrefillAttnArgs &a = *R.a;
    AttnBars *B = R.bars;
    // the record's fields in registers: the barrier and MMA instructions below are asm statements that clobber memory,
    // so fields read through `R` would be re-read from the caller's stack frame after every one of them
    const unsigned long long lim = R.lim;
    char *const smem = R.smem;
    const int cta = R.p, cta_count = R.P;
    const int n_units = a.n_units;
    const CUtensorMap *tmQ = &R.amaps->tmQ, *tmK = &R.amaps->tmK, *tmV = &R.amaps->tmV;
    unsigned int uc = 0, kc = 0;  // units and key tiles this CTA has staged
    const int slots = is_v ? kAtVSlots : kAtKSlots;
    int s = 0;
    uint32_t wrap = 0;  // completed laps of the ring (phase of slot s)
    for (int rnd = 0; rnd * cta_count < n_units; ++rnd) {
        const int u = attn_unit_of(cta, cta_count, rnd);
        if (u >= n_units) continue;
        const AttnUnit t = attn_unit(a, u);
        if (t.n_tiles == 0) continue;
        if (!is_v) {
            if (!mbar_wait(&B->q_empty, (uc & 1) ^ 1, lim)) return attn_fail(R);
            mbar_expect_tx(&B->q_full, kAtTileBytes);
            char *sQ = smem + kAtQOff;
            tma_load_4d(sQ, tmQ, &B->q_full, 0, t.qt * kAtTile, t.h, t.b);
            tma_load_4d(sQ + kGemmABytes, tmQ, &B->q_full, 64, t.qt * kAtTile, t.h, t.b);
        }
        ++uc;
        for (int j = 0; j < t.n_tiles; ++j, ++kc) {
            const int key0 = j * kAtTile;
            if (!is_v) {
                if (!mbar_wait(&B->k_empty[s], (wrap & 1) ^ 1, lim)) return attn_fail(R);
                mbar_expect_tx(&B->k_full[s], kAtTileBytes);
                char *sK = smem + kAtKOff + s * kAtTileBytes;
                // K as the K-major B operand of S = Q K^T: two blocks of 64 head-dimension elements x 128 keys
                tma_load_4d(sK, tmK, &B->k_full[s], 0, key0, t.hkv, t.b);
                tma_load_4d(sK + kGemmABytes, tmK, &B->k_full[s], 64, key0, t.hkv, t.b);
            } else {
                if (!mbar_wait(&B->v_empty[s], (wrap & 1) ^ 1, lim)) return attn_fail(R);
                mbar_expect_tx(&B->v_full[s], kAtTileBytes);
                char *sV = smem + kAtVOff + s * kAtTileBytes;
                // V as the MN-major B operand of O = P V: per block of 64 keys two chunks of 64 head-dimension columns
                for (int kb = 0; kb < 2; ++kb)
                    for (int c = 0; c < 2; ++c)
                        tma_load_4d(sV + kb * 16384 + c * 8192, tmV, &B->v_full[s], c * 64, key0 + kb * 64, t.hkv, t.b);
            }
            if (++s == slots) { s = 0; ++wrap; }
        }
    }
    // drain: the MMA thread's last commits on the empty barriers arrive asynchronously; they must have landed before
    // the barriers are given up at the end of the stage
    for (unsigned int i = kc >= (unsigned)slots ? kc - slots : 0; i < kc; ++i) {
        unsigned long long *bar = is_v ? &B->v_empty[i % slots] : &B->k_empty[i % slots];
        if (!mbar_wait(bar, (i / slots) & 1, lim)) return attn_fail(R);
    }
    if (!is_v && uc > 0 && !mbar_wait(&B->q_empty, (uc - 1) & 1, lim)) return attn_fail(R);
    return true;
}

// ---- MMA issue -----------------------------------------------------------------------------
__device__ __noinline__ bool attn_issue(const AttnRun &R) {
    const PrefillAttnArgs &a = *R.a;
    AttnBars *B = R.bars;
    // the record's fields in registers: the barrier and MMA instructions below are asm statements that clobber memory,
    // so fields read through `R` would be re-read from the caller's stack frame after every one of them
    const unsigned long long lim = R.lim;
    char *const smem = R.smem;
    const int cta = R.p, cta_count = R.P;
    const int n_units = a.n_units;
    const int bf16 = a.dtype == DT_BF16;
    const uint32_t idesc_s = umma_idesc(bf16, 0, 0, kAtTile, kAtTile);   // Q, K both K-major
    const uint32_t idesc_o = umma_idesc(bf16, 0, 1, kAtTile, kAtTile);   // P K-major (tensor memory), V MN-major
    const uint32_t sQ = smem_u32(smem + kAtQOff);
    const uint32_t tm = R.tmem_base;
    unsigned int uc = 0, sc = 0, pc = 0;  // units; S tiles issued; P tiles consumed (= P V issued)
    int ks = 0, vs = 0;                   // ring slots of the next K / V tile
    uint32_t kwrap = 0, vwrap = 0;

    auto issue_s = [&]() -> bool {
        if (!mbar_wait(&B->k_full[ks], kwrap & 1, lim)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + kAtKOff + ks * kAtTileBytes);
        const uint32_t d = tm + kAtS0 + (sc & 1) * kAtTile;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            const uint64_t da = umma_desc(sQ + kb * kGemmABytes, 16, 1024), db = umma_desc(sK + kb * kGemmABytes, 16, 1024);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_f16(d, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc_s, (kb | kk) ? 1u : 0u);
        }
        umma_commit(&B->k_empty[ks]);
        umma_commit(&B->s_full[sc & 1]);
        if (++ks == kAtKSlots) { ks = 0; ++kwrap; }
        ++sc;
        return true;
    };

    for (int rnd = 0; rnd * cta_count < n_units; ++rnd) {
        const int u = attn_unit_of(cta, cta_count, rnd);
        if (u >= n_units) continue;
        const AttnUnit t = attn_unit(a, u);
        if (t.n_tiles == 0) continue;
        if (!mbar_wait(&B->q_full, uc & 1, lim)) return attn_fail(R);
        // both S buffers are free: every P V of the previous unit has been issued, and the pipe runs in issue order
        if (!issue_s()) return attn_fail(R);
        if (t.n_tiles > 1 && !issue_s()) return attn_fail(R);
        if (t.n_tiles <= 2) umma_commit(&B->q_empty);  // the unit's last S is issued: Q may be replaced once it is done
        for (int j = 0; j < t.n_tiles; ++j, ++pc) {
            if (!mbar_wait(&B->p_ready[pc & 1], (pc >> 1) & 1, lim)) return attn_fail(R);
            if (j == 0 && !mbar_wait(&B->o_free, (uc & 1) ^ 1, lim)) return attn_fail(R);
            if (!mbar_wait(&B->v_full[vs], vwrap & 1, lim)) return attn_fail(R);
            tc_fence_after();
            const uint32_t sV = smem_u32(smem + kAtVOff + vs * kAtTileBytes);
            const uint32_t pa = tm + kAtS0 + (pc & 1) * kAtTile;  // P(j) sits where S(j) was
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
                const uint64_t db = umma_desc(sV + kb * 16384, 8192, 1024);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_f16_ts(tm + kAtO, pa + (kb * 4 + kk) * 8, db + (uint64_t)(kk * 128), idesc_o, (j | kb | kk) ? 1u : 0u);
            }
            umma_commit(&B->v_empty[vs]);
            umma_commit(&B->o_done[pc & 1]);
            if (++vs == kAtVSlots) { vs = 0; ++vwrap; }
            // the buffer P(j) occupied takes S(j+2)
            if (j + 2 < t.n_tiles) {
                if (!issue_s()) return attn_fail(R);
                if (j + 3 == t.n_tiles) umma_commit(&B->q_empty);
            }
        }
        ++uc;
    }
    return true;
}

// ---- softmax and output -------------------------------------------------------------------------
// Warp q + 8*half owns TMEM lanes 32q..32q+31 (the only ones a warp with index = q mod 4 can reach) = query rows
// 32q.. of the tile, and columns 64*half..+63 of S and O. Thread = row.
template <typename T, bool MASK>
__device__ __noinline__ bool attn_softmax(const AttnRun &R, int warp, int lane) {
    const PrefillAttnArgs &a = *R.a;
    AttnBars *B = R.bars;
    // the record's fields in registers: the barrier and MMA instructions below are asm statements that clobber memory,
    // so fields read through `R` would be re-read from the caller's stack frame after every one of them
    const unsigned long long lim = R.lim;
    char *const smem = R.smem;
    const int cta = R.p, cta_count = R.P;
    const int n_units = a.n_units;
    const int quarter = warp & 3, half = warp >> 3;
    const int row = quarter * 32 + lane;
    const int col0 = half * 64;
    const uint32_t lane_addr = R.tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float c = a.scale * 1.4426950408889634f;  // scores are kept in units of log2(e): exp(x) = exp2(x * log2 e)
    float *xch = reinterpret_cast<float *>(smem + kAtXchOff);  // [2 parities][2 halves][128 rows], twice
    unsigned int sc = 0;   // S tiles consumed = number of the P V that will use this tile's P
    // P V number i completes phase i / 2 of o_done[i & 1]. A parity wait can tell a phase from the next one only, so
    // every phase of both barriers is observed in turn: tile n always observes P V n-2 (long complete: it costs
    // nothing), which leaves P V n-1 — the one a rescale of O has to wait for — as the only phase that can be open.
    unsigned int oc[2] = {0, 0};  // phases observed per barrier
    auto observe = [&](unsigned int i) -> bool {  // returns once P V number i is complete
        const unsigned int b = i & 1;
        while (oc[b] <= (i >> 1)) {
            const bool ok = mbar_wait(&B->o_done[b], oc[b] & 1, lim);
            if (!__all_sync(0xffffffffu, ok)) {
                if (lane == 0) attn_fail(R);
                return false;
            }
            ++oc[b];
        }
        return true;
    };
    for (int rnd = 0; rnd * cta_count < n_units; ++rnd) {
        const int u = attn_unit_of(cta, cta_count, rnd);
        if (u >= n_units) continue;
        const AttnUnit t = attn_unit(a, u);
        const int qi = t.qt * kAtTile + row;
        T *orow = reinterpret_cast<T *>(a.out) + (int64_t)t.b * a.o_stride_b + (int64_t)t.h * a.o_stride_h + (int64_t)qi * a.o_stride_t + col0;
        if (t.n_tiles == 0) {  // no key visible to any row of the tile: zeros
            if (qi < a.Tq)
                for (int i = 0; i < 64; i += 8) *reinterpret_cast<uint4 *>(orow + i) = make_uint4(0, 0, 0, 0);
            continue;
        }
        const int last_key = a.causal ? min(a.Tkv - 1, qi + a.Tkv - a.Tq) : a.Tkv - 1;  // last key this row may see
        // additive mask: this row's values, in units of the raw score (mask / scale), join the raw scores
        const T *mrow = nullptr;
        float inv_scale = 0.0f;
        if constexpr (MASK) {
            mrow = reinterpret_cast<const T *>(a.mask) + (int64_t)t.b * a.m_stride_b + (int64_t)t.h * a.m_stride_h +
                   (int64_t)min(qi, a.Tq - 1) * a.m_stride_q;
            inv_scale = 1.0f / a.scale;
        }
        float m = -INFINITY, l = 0.0f;
        for (int j = 0; j < t.n_tiles; ++j, ++sc) {
            const int sb = sc & 1;
            bool ok = mbar_wait(&B->s_full[sb], (sc >> 1) & 1, lim);
            if (!__all_sync(0xffffffffu, ok)) {
                if (lane == 0) attn_fail(R);
                return false;
            }
            tc_fence_after();
            const uint32_t buf = lane_addr + kAtS0 + sb * kAtTile;
            const int key0 = j * kAtTile + col0;  // first key of this warp's columns
            // masking is needed when these columns hold a key some row of this warp may not see
            const bool masked = key0 + 63 > __shfl_sync(0xffffffffu, last_key, 0);
            uint32_t r0[32], r1[32];
            tmem_ld32(buf + col0, r0);
            tmem_ld32(buf + col0 + 32, r1);
            tmem_ld_wait();
            // the raw scores stay in r0 / r1 as float bits until the exponentials (the scale is positive: the maximum
            // of the raw scores is the maximum of the scaled ones)
            if constexpr (MASK) {
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {  // 8 keys per 16-byte vector of the mask row
                    const int k0 = key0 + cc * 8;
                    float mv[8];
                    if (k0 + 7 < a.Tkv) {
                        load_vec<T, 8>(mrow + k0, mv);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) mv[i] = k0 + i < a.Tkv ? to_f32(mrow[k0 + i]) : 0.0f;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int idx = cc * 8 + i;
                        if (idx < 32) r0[idx] = __float_as_uint(fmaf(mv[i], inv_scale, __uint_as_float(r0[idx])));
                        else r1[idx - 32] = __float_as_uint(fmaf(mv[i], inv_scale, __uint_as_float(r1[idx - 32])));
                    }
                }
            }
            if (masked) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (key0 + i > last_key) r0[i] = 0xff800000u;       // -inf
                    if (key0 + 32 + i > last_key) r1[i] = 0xff800000u;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(r0[i]), __uint_as_float(r1[i])));
            const float mx_own = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * c;
            float *x = xch + (sc & 1) * 256;
            x[half * 128 + row] = mx_own;
            // both warps of the row have read their S columns behind this barrier: from here on P may overwrite them
            tc_fence_before();
            named_barrier(1 + quarter, 64);
            tc_fence_after();
            const float mx = fmaxf(mx_own, x[(half ^ 1) * 128 + row]);
            // the running maximum moves only when it lags by more than kAtLazy (or was never set)
            float m_new = m;
            if (mx > m + kAtLazy || m == -INFINITY) m_new = fmaxf(m, mx);
            // a row with no visible key so far keeps m = -inf; the exponentials below then see -inf - 0 and give 0
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float alpha = ex2(m - m_use);  // m = -inf: 0; m unchanged: 1
            // O is rescaled between P V (j-1), which must then be complete, and P V (j), which waits for this tile's P
            const bool rescale = j > 0 && __any_sync(0xffffffffu, alpha != 1.0f);
            if (sc >= 2 && !observe(sc - 2)) return false;
            if (rescale) {
                if (!observe(sc - 1)) return false;
                tc_fence_after();
#pragma unroll 1
                for (int cc = 0; cc < 4; ++cc) {  // 16 columns at a time: the scores stay in registers meanwhile
                    uint32_t t16[16];
                    tmem_ld16x(lane_addr + kAtO + col0 + cc * 16, t16);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) t16[i] = __float_as_uint(__uint_as_float(t16[i]) * alpha);
                    tmem_st16(lane_addr + kAtO + col0 + cc * 16, t16);
                }
            }
            l *= alpha;
            m = m_new;
            // P = exp2(v - m), rounded to the storage type, two keys per 32-bit column: this warp's 64 keys are
            // columns 32*half..+31 of the buffer
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    pk[i] = pack2<T>(ex2(fmaf(__uint_as_float(r0[2 * i]), c, -m_use)), ex2(fmaf(__uint_as_float(r0[2 * i + 1]), c, -m_use)), l4[i & 3]);
                tmem_st16(buf + half * 32, pk);
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    pk[i] = pack2<T>(ex2(fmaf(__uint_as_float(r1[2 * i]), c, -m_use)), ex2(fmaf(__uint_as_float(r1[2 * i + 1]), c, -m_use)), l4[i & 3]);
                tmem_st16(buf + half * 32 + 16, pk);
            }
            tmem_st_wait();
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B->p_ready[sc & 1]);
        }
        // the unit's last P V (sc - 1; observing sc - 2 first keeps both barriers' phases in turn)
        if (sc >= 2 && !observe(sc - 2)) return false;
        if (!observe(sc - 1)) return false;
        tc_fence_after();
        // the row's sum: both halves, added in the same order by both warps
        float *x = xch + 512 + (sc & 1) * 256;
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
        for (int s = 0; s < kAtKSlots; ++s) { mbar_init(&B->k_full[s], 1); mbar_init(&B->k_empty[s], 1); }
        for (int s = 0; s < kAtVSlots; ++s) { mbar_init(&B->v_full[s], 1); mbar_init(&B->v_empty[s], 1); }
        for (int s = 0; s < 2; ++s) mbar_init(&B->s_full[s], 1);
        mbar_init(&B->p_ready[0], kAtSoftmaxWarps); mbar_init(&B->p_ready[1], kAtSoftmaxWarps);
        mbar_init(&B->o_done[0], 1); mbar_init(&B->o_done[1], 1);
        mbar_init(&B->o_free, kAtSoftmaxWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == kProducerWarp || warp == kProducerWarpB) {
        if (lane == 0) attn_produce(R, warp == kProducerWarpB);
    } else if (warp == kMmaWarp) {
        if (lane == 0) attn_issue(R);
    } else if (warp < kEpiWarps || (warp >= 8 && warp < 12)) {
        if (a.mask) {
            if (a.dtype == DT_BF16) attn_softmax<__nv_bfloat16, true>(R, warp, lane);
            else attn_softmax<__half, true>(R, warp, lane);
        } else {
            if (a.dtype == DT_BF16) attn_softmax<__nv_bfloat16, false>(R, warp, lane);
            else attn_softmax<__half, false>(R, warp, lane);
        }
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
