// Tile loops of the tensor-core matmul and the CUDA-core fallback (see dev_gemm.cuh).
#include "dev_gemm.cuh"

namespace arkb {

struct TileCoord {
    int m0, n0, bc, bn;
};

__device__ __forceinline__ TileCoord gemm_unit(const GemmArgs &g, int u) {
    TileCoord t;
    if (!g.plan_tiles) {
        const int per = g.tiles_m * g.tiles_n;
        int b = u / per, r = u % per;
        t.bc = b % g.batch_c;
        t.bn = b / g.batch_c;
        const int gsz = g.raster_group * g.tiles_n;
        const int gi = r / gsz, ri = r % gsz;
        const int first_m = gi * g.raster_group;
        const int gm = min(g.raster_group, g.tiles_m - first_m);
        t.m0 = (first_m + ri % gm) * g.tile_m;
        t.n0 = (ri / gm) * g.tile_n;
    } else {
        const int subs = g.sub_m * g.sub_n;
        const int ord = u / subs, sub = u % subs;
        int id = g.task_b + ord * g.task_s;
        const int tw = id % g.p_tiles_w;
        id /= g.p_tiles_w;
        const int th = id % g.p_tiles_h;
        id /= g.p_tiles_h;
        t.bc = id % g.batch_c;
        t.bn = id / g.batch_c;
        t.m0 = th * g.ptm + (sub / g.sub_n) * g.tile_m;
        t.n0 = tw * g.ptn + (sub % g.sub_n) * g.tile_n;
    }
    return t;
}

// Scalars of a GEMM stage held in registers. The stage descriptor lives in
// global memory; reading its fields inside the pipeline loops would put a
// global load on the critical path of every k-block.
struct GemmLocal {
    void *C;
    const void *bias;
    int64_t ldc, c_stride_c, c_stride_n;
    int M, N, K, tile_n, act, c_vec, c_tma, dtype, out_transposed, splits, batch_c, bias_mul, rope_rows, rope_cols;
    float *ws;
    int64_t splits_stride;  // elements between the partials of consecutive k-ranges
    int a_mn_major, b_mn_major, a_bc, a_bn, b_bc, b_bn;
    int peer_rows;
};

template <typename T>
__device__ __forceinline__ void gemm_store_row(const GemmLocal &g, T *crow, const T *brow, int col, int ncols,
                                               uint32_t (&r)[32], int cnt, int bcol0 = 0) {
    // cnt accumulator values (16 or 32) for columns [col, col+cnt) of one row
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = (i < cnt) ? __uint_as_float(r[i]) : 0.0f;
    const bool full = (col + cnt <= ncols) && g.c_vec;
    if (g.bias_mul == 2) {
        // rotary embedding on the accumulator: brow is the table row of this output row, bcol0 the absolute column of
        // column 0 of `crow` (even; the table row length is a multiple of 8, so an 8-vector never wraps)
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (v * 8 < cnt) {
                float b[8];
                load_vec<T, 8>(brow + (bcol0 + col + v * 8) % g.rope_cols, b);
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const float x0 = f[v * 8 + i], x1 = f[v * 8 + i + 1];
                    f[v * 8 + i] = x0 * b[i] - x1 * b[i + 1];
                    f[v * 8 + i + 1] = x0 * b[i + 1] + x1 * b[i];
                }
            }
        }
        if (full) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                if (v * 8 < cnt) {
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = f[v * 8 + i];
                    store_vec<T, 8>(crow + col + v * 8, o);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < cnt && col + i < ncols) crow[col + i] = from_f32<T>(f[i]);
        }
        return;
    }
    if (full) {
        if (brow && !g.bias_mul) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                if (v * 8 < cnt) {
                    float b[8];
                    load_vec<T, 8>(brow + col + v * 8, b);
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[v * 8 + i] += b[i];
                }
            }
        }
        if (g.act != ACT_NONE) {
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = apply_act_fast(g.act, f[i]);
        }
        if (brow && g.bias_mul) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                if (v * 8 < cnt) {
                    float b[8];
                    load_vec<T, 8>(brow + col + v * 8, b);
#pragma unroll
                    for (int i = 0; i < 8; ++i) f[v * 8 + i] *= b[i];
                }
            }
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (v * 8 < cnt) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = f[v * 8 + i];
                store_vec<T, 8>(crow + col + v * 8, o);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (i < cnt && col + i < ncols) {
                float v = f[i];
                if (brow && !g.bias_mul) v += to_f32(brow[col + i]);
                v = apply_act_fast(g.act, v);
                if (brow && g.bias_mul) v *= to_f32(brow[col + i]);
                crow[col + i] = from_f32<T>(v);
            }
        }
    }
}

// Epilogue through shared memory: each warp converts a 32x32 block of its TMEM
// quarter, writes it into a 64-byte-swizzled staging block (conflict-free
// 16-byte stores) and one lane hands the block to a TMA store. Two staging
// blocks per warp alternate so that the conversion of block i+1 overlaps the
// store of block i. Rows and columns outside the tensor are clipped by TMA.
template <typename T>
__device__ __noinline__ void gemm_epilogue_tile_tma(const GemmLocal &g, const CUtensorMap *tmC, const TileCoord &tc, uint32_t tmem_acc,
                                       int warp, int lane, char *stage, unsigned int &blk, int row_shift = 0) {
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(warp * 32) << 16);
    const int ncols_tile = min(g.tile_n, g.N - tc.n0);
    const int row0 = tc.m0 + warp * 32;
    if (row0 >= g.M) return;  // the whole warp is outside the matrix
    for (int c = 0; c < g.tile_n; c += 32) {
        if (c >= ncols_tile) break;
        uint32_t r[32];
        tmem_ld32(lane_addr + c, r);
        char *buf = stage + (warp * 2 + (blk & 1)) * kEpiBlockBytes;
        // the TMA store issued two blocks ago must have finished reading this buffer
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        tmem_ld_wait();
        union { uint4 q[4]; T e[32]; } o;
#pragma unroll
        for (int i = 0; i < 32; ++i) o.e[i] = from_f32<T>(apply_act_fast(g.act, __uint_as_float(r[i])));
#pragma unroll
        for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4 *>(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = o.q[j];
        fence_async_smem();
        __syncwarp();
        if (lane == 0) tma_store_4d(tmC, buf, tc.n0 + c, row0 - row_shift, tc.bc, tc.bn);
        ++blk;
    }
}

template <typename T>
__device__ __noinline__ void gemm_epilogue_tile(const GemmLocal &g, const TileCoord &tc, uint32_t tmem_acc, int warp, int lane) {
    const int row = tc.m0 + warp * 32 + lane;
    const bool row_ok = row < g.M;
    const int64_t boff = (int64_t)tc.bn * g.c_stride_n + (int64_t)tc.bc * g.c_stride_c + (int64_t)row * g.ldc;
    T *crow = reinterpret_cast<T *>(g.C) + boff;
    const T *brow = g.bias ? reinterpret_cast<const T *>(g.bias) + boff : nullptr;
    if (g.bias_mul == 2) brow = reinterpret_cast<const T *>(g.bias) + (int64_t)(row_ok ? row % g.rope_rows : 0) * g.rope_cols - tc.n0;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(warp * 32) << 16);
    const int ncols_tile = min(g.tile_n, g.N - tc.n0);  // valid columns of this tile
    for (int c = 0; c < g.tile_n; c += 32) {
        if (c >= ncols_tile) break;  // uniform across the warp
        uint32_t r[32];
        const int cnt = (g.tile_n - c >= 32) ? 32 : 16;
        if (cnt == 32) tmem_ld32(lane_addr + c, r);
        else tmem_ld16(lane_addr + c, r);
        tmem_ld_wait();
        if (row_ok) gemm_store_row<T>(g, crow + tc.n0, brow ? brow + tc.n0 : nullptr, c, ncols_tile, r, cnt, tc.n0);
    }
}

// Epilogue of the swapped form (A = weights, B = activations): accumulator row =
// output column n (one per lane), accumulator column = output row m. For a fixed m
// the 32 lanes of a warp write 32 consecutive n: coalesced without staging.
// In this form g.M / g.N hold the swapped problem (M' = columns of C, N' = rows of C).
template <typename T>
__device__ __noinline__ void gemm_epilogue_tile_swapped(const GemmLocal &g, const TileCoord &tc, uint32_t tmem_acc, int warp, int lane) {
    const int n = tc.m0 + warp * 32 + lane;
    const bool n_ok = n < g.M;
    const int64_t boff = (int64_t)tc.bn * g.c_stride_n + (int64_t)tc.bc * g.c_stride_c;
    T *cbase = reinterpret_cast<T *>(g.C) + boff;
    const T *bbase = g.bias ? reinterpret_cast<const T *>(g.bias) + boff : nullptr;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(warp * 32) << 16);
    const int rows = min(g.tile_n, g.N - tc.n0);
    for (int c = 0; c < g.tile_n; c += 32) {
        if (c >= rows) break;
        uint32_t r[32];
        const int cnt = (g.tile_n - c >= 32) ? 32 : 16;
        if (cnt == 32) tmem_ld32(lane_addr + c, r);
        else tmem_ld16(lane_addr + c, r);
        tmem_ld_wait();
        if (n_ok) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int m = tc.n0 + c + i;
                if (i < cnt && m < g.N) {
                    float v = __uint_as_float(r[i]);
                    if (bbase && !g.bias_mul) v += to_f32(bbase[(int64_t)m * g.ldc + n]);
                    v = apply_act_fast(g.act, v);
                    if (bbase && g.bias_mul) v *= to_f32(bbase[(int64_t)m * g.ldc + n]);
                    cbase[(int64_t)m * g.ldc + n] = from_f32<T>(v);
                }
            }
        }
    }
}

// Split-K epilogue of the swapped form: the fp32 partial of k-range `split` goes to
// ws[split][batch][m][n] unrounded; run_splitk_reduce finishes the job.
__device__ __noinline__ void gemm_epilogue_tile_partial(const GemmLocal &g, const TileCoord &tc, int split, uint32_t tmem_acc, int warp,
                                           int lane) {
    const int n = tc.m0 + warp * 32 + lane;   // column of C
    const bool n_ok = n < g.M;                // g.M / g.N hold the swapped problem
    const int64_t ncols = g.M, nrows = g.N;
    const int64_t batch = (int64_t)tc.bn * g.batch_c + tc.bc;
    float *w = g.ws + (int64_t)split * g.splits_stride + batch * nrows * ncols;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(warp * 32) << 16);
    const int rows = min(g.tile_n, (int)nrows - tc.n0);
    for (int c = 0; c < g.tile_n; c += 32) {
        if (c >= rows) break;
        uint32_t r[32];
        const int cnt = (g.tile_n - c >= 32) ? 32 : 16;
        if (cnt == 32) tmem_ld32(lane_addr + c, r);
        else tmem_ld16(lane_addr + c, r);
        tmem_ld_wait();
        if (n_ok) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int m = tc.n0 + c + i;
                if (i < cnt && m < nrows) w[(int64_t)m * ncols + n] = __uint_as_float(r[i]);
            }
        }
    }
}

// Split-K epilogue of the ordinary form: accumulator row = row of C (one per lane), accumulator column = column of C;
// the fp32 partial of k-range `split` goes to ws[split][batch][m][n] unrounded.
__device__ __noinline__ void gemm_epilogue_tile_partial_rows(const GemmLocal &g, const TileCoord &tc, int split, uint32_t tmem_acc,
                                                             int warp, int lane) {
    const int m = tc.m0 + warp * 32 + lane;
    const bool m_ok = m < g.M;
    const int64_t batch = (int64_t)tc.bn * g.batch_c + tc.bc;
    float *w = g.ws + (int64_t)split * g.splits_stride + batch * (int64_t)g.M * g.N + (int64_t)m * g.N + tc.n0;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(warp * 32) << 16);
    const int ncols_tile = min(g.tile_n, g.N - tc.n0);
    for (int c = 0; c < g.tile_n; c += 32) {
        if (c >= ncols_tile) break;
        uint32_t r[32];
        const int cnt = (g.tile_n - c >= 32) ? 32 : 16;
        if (cnt == 32) tmem_ld32(lane_addr + c, r);
        else tmem_ld16(lane_addr + c, r);
        tmem_ld_wait();
        if (m_ok) {
            if (c + cnt <= ncols_tile && (g.N % 4) == 0) {  // rows of the scratch are 16-byte aligned
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    if (i < cnt) *reinterpret_cast<uint4 *>(w + c + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (i < cnt && c + i < ncols_tile) w[c + i] = __uint_as_float(r[i]);
            }
        }
    }
}

// Runs the tiles of one GEMM stage assigned to CTA p of P. All threads of the
// CTA call this; it returns with the pipeline drained.
//
// PAIR == false: the CTA owns 128 x tile_n tiles (tcgen05 cta_group::1).
// PAIR == true : CTAs 2q and 2q+1 form a cluster and own 256 x tile_n tiles
//   (cta_group::2). Each CTA stages its 128 rows of A and its half of the B
//   columns; the leader (even CTA) issues the MMAs, which read both CTAs'
//   shared memory and write both CTAs' TMEM. TMA completions of both CTAs are
//   credited to the leader's `full` barrier; the leader's commits release the
//   `empty` slot and publish `acc_full` in both CTAs; the epilogue warps of
//   both CTAs arrive on the leader's `acc_empty`.
// Everything the warp roles of one matmul stage share. Built by every thread at the start of the stage; the roles
// are separate functions (own register allocation: the threads that issue the copies and the MMAs are the critical
// path of large matmuls, and spills or extra instructions there cost several per cent).
struct GemmRun {
    GemmLocal L;
    const GemmArgs *g;      // the stage record (a copy in shared memory)
    const GemmArgs *gmaps;  // the stage record in global memory: the TMA unit reads tensor maps there
    char *smem;
    GemmPipe *pp;
    CtaCtl *ctl;
    DeviceState *st;
    unsigned long long lim;
    int stage_idx;
    int STAGES, G, blk_b_bytes, stage_bytes;  // a ring slot holds G consecutive k-blocks of both operands: [G blocks of A][G blocks of B]
    int n_units, kblocks, crank, up, UP, n_half, splits, kper;
    int tall, a_slot;  // tall: 256-row tiles as two halves; a_slot: bytes of operand A in a ring slot (B follows)
    uint32_t base_par, tmem_base;
    unsigned int t0;
};

// GROUPED == false compiles the loops for one k-block per ring slot (G is the constant 1).
// Producer: one lane of warp 4 (operand A) and one of warp 6 (operand B). Returns false when a wait ran out.
template <bool PAIR, bool GROUPED>
__device__ __noinline__ bool gemm_produce(const GemmRun &R, int warp) {
    const GemmLocal &L = R.L;
    const GemmArgs &g = *R.g;
    const GemmArgs *gmaps = R.gmaps;
    char *smem = R.smem;
    GemmPipe *pp = R.pp;
    CtaCtl *ctl = R.ctl;
    DeviceState *st = R.st;
    const int stage_idx = R.stage_idx;
    const unsigned long long lim = R.lim;
    const int STAGES = R.STAGES, G = GROUPED ? R.G : 1, blk_b_bytes = R.blk_b_bytes, stage_bytes = R.stage_bytes;
    const int n_units = R.n_units, kblocks = R.kblocks, crank = R.crank, up = R.up, UP = R.UP, n_half = R.n_half;
    const int splits = R.splits, kper = R.kper;
    const uint32_t base_par = R.base_par, tmem_base = R.tmem_base;
    const unsigned int t0 = R.t0;
    const CUtensorMap *tmA = &gmaps->tmA, *tmB = &gmaps->tmB, *tmC = &gmaps->tmC;
    (void)L; (void)g; (void)smem; (void)pp; (void)ctl; (void)st; (void)stage_idx; (void)lim; (void)STAGES; (void)G; (void)blk_b_bytes;
    (void)stage_bytes; (void)n_units; (void)kblocks; (void)crank; (void)up; (void)UP; (void)n_half; (void)splits; (void)kper;
    (void)base_par; (void)tmem_base; (void)t0; (void)tmA; (void)tmB; (void)tmC;

    const bool is_a = warp == kProducerWarp;
    const int mn_major = is_a ? L.a_mn_major : L.b_mn_major;
    const int tall = PAIR ? 0 : R.tall, a_slot = R.a_slot;
    const int span = is_a ? kGemmTileM * (1 + tall) : n_half;  // rows (K-major) or columns (MN-major) staged
    const int chunks = mn_major ? (span + 63) / 64 : 1;       // 64-wide MN chunks
    // a slot always receives G whole k-blocks (those past the end of K arrive as zeros)
    const uint32_t bytes = (uint32_t)G * (mn_major ? (uint32_t)chunks * 64 * kGemmBK * 2 : (uint32_t)span * kGemmBK * 2);
    const CUtensorMap *tm = is_a ? tmA : tmB;
    const int has_c = is_a ? L.a_bc : L.b_bc, has_n = is_a ? L.a_bn : L.b_bn;
    int s = 0;
    uint32_t wrap = 0;
    for (int u = up; u < n_units; u += UP) {
        const TileCoord tc = gemm_unit(g, u / splits);
        const int mn0 = is_a ? tc.m0 + crank * kGemmTileM : tc.n0 + crank * n_half;
        const int bc = has_c ? tc.bc : 0, bn = has_n ? tc.bn : 0;
        const int kb_lo = (u % splits) * kper, kb_hi = min(kblocks, kb_lo + kper);
        for (int k = kb_lo; k < kb_hi; k += G, s = (s + 1 == STAGES ? 0 : s + 1), wrap ^= (s == 0)) {
            const uint32_t par = (((base_par >> s) ^ wrap) & 1) ^ 1;
            if (!mbar_wait(&pp->empty[s], par, lim)) {
                ctl->abort = 1;
                report(st, ST_MBAR_TIMEOUT, stage_idx);
                return false;
            }
            char *dst = smem + s * stage_bytes + (is_a ? 0 : a_slot);
            const int chunk_stride = G * 64 * kGemmBK * 2;  // MN-major: G k-blocks of one 64-wide chunk are contiguous
            if constexpr (!PAIR) {
                mbar_expect_tx(&pp->full[s], bytes);
                if (!mn_major) {
                    if (G == 1) {
                        tma_load_4d(dst, tm, &pp->full[s], k * kGemmBK, mn0, bc, bn);
                        if (is_a && tall) tma_load_4d(dst + kGemmABytes, tm, &pp->full[s], k * kGemmBK, mn0 + kGemmTileM, bc, bn);
                    } else {
                        tma_load_5d(dst, tm, &pp->full[s], 0, mn0, k, bc, bn);
                    }
                } else {
                    for (int c = 0; c < chunks; ++c)
                        tma_load_4d(dst + c * chunk_stride, tm, &pp->full[s], mn0 + c * 64, k * kGemmBK, bc, bn);
                }
            } else {
                // both CTAs' copies are credited to the leader's barrier
                const uint32_t full_leader = mapa_u32(smem_u32(&pp->full[s]), 0);
                if (crank == 0) mbar_expect_tx(&pp->full[s], 2 * bytes);
                if (!mn_major) {
                    if (G == 1) tma_load_4d_pair(dst, tm, full_leader, k * kGemmBK, mn0, bc, bn);
                    else tma_load_5d_pair(dst, tm, full_leader, 0, mn0, k, bc, bn);
                } else {
                    for (int c = 0; c < chunks; ++c)
                        tma_load_4d_pair(dst + c * chunk_stride, tm, full_leader, mn0 + c * 64, k * kGemmBK, bc, bn);
                }
            }
        }
    }
    return true;
}

// MMA issue: one lane of warp 5 of the leader CTA.
template <bool PAIR, bool GROUPED, bool TALL>
__device__ __noinline__ bool gemm_issue(const GemmRun &R) {
    const GemmLocal &L = R.L;
    const GemmArgs &g = *R.g;
    const GemmArgs *gmaps = R.gmaps;
    char *smem = R.smem;
    GemmPipe *pp = R.pp;
    CtaCtl *ctl = R.ctl;
    DeviceState *st = R.st;
    const int stage_idx = R.stage_idx;
    const unsigned long long lim = R.lim;
    const int STAGES = R.STAGES, G = GROUPED ? R.G : 1, blk_b_bytes = R.blk_b_bytes, stage_bytes = R.stage_bytes;
    const int n_units = R.n_units, kblocks = R.kblocks, crank = R.crank, up = R.up, UP = R.UP, n_half = R.n_half;
    const int splits = R.splits, kper = R.kper;
    const uint32_t base_par = R.base_par, tmem_base = R.tmem_base;
    const unsigned int t0 = R.t0;
    constexpr int tall = TALL ? 1 : 0;
    const int a_slot = R.a_slot;
    (void)a_slot;
    const CUtensorMap *tmA = &gmaps->tmA, *tmB = &gmaps->tmB, *tmC = &gmaps->tmC;
    (void)L; (void)g; (void)smem; (void)pp; (void)ctl; (void)st; (void)stage_idx; (void)lim; (void)STAGES; (void)G; (void)blk_b_bytes;
    (void)stage_bytes; (void)n_units; (void)kblocks; (void)crank; (void)up; (void)UP; (void)n_half; (void)splits; (void)kper;
    (void)base_par; (void)tmem_base; (void)t0; (void)tmA; (void)tmB; (void)tmC;

    const uint32_t idesc = umma_idesc(L.dtype == DT_BF16, L.a_mn_major, L.b_mn_major, L.tile_n, PAIR ? 256 : 128);
    // per-MMA (K=16) advance of the descriptor start address, in 16-byte units
    const uint32_t a_adv = L.a_mn_major ? (16 * 128) >> 4 : 32 >> 4;
    const uint32_t b_adv = L.b_mn_major ? (16 * 128) >> 4 : 32 >> 4;
    const uint32_t blk_mn_bytes = 64 * kGemmBK * 2;        // one k-block of a 64-wide MN chunk
    const uint32_t chunk_bytes = (uint32_t)G * blk_mn_bytes;  // distance between the chunks of one k-block
    const uint32_t a_blk = L.a_mn_major ? blk_mn_bytes : (uint32_t)kGemmABytes;   // k-block to k-block inside a slot
    const uint32_t b_blk = L.b_mn_major ? blk_mn_bytes : (uint32_t)blk_b_bytes;
    unsigned int t = t0;
    int s = 0;
    uint32_t wrap = 0;
    for (int u = up; u < n_units; u += UP, ++t) {
        const int kb_lo = (u % splits) * kper, kb_hi = min(kblocks, kb_lo + kper);
        const int acc = t & 1;
        if (!mbar_wait(&pp->acc_empty[acc], ((t >> 1) & 1) ^ 1, lim)) {
            ctl->abort = 1;
            report(st, ST_MBAR_TIMEOUT, stage_idx);
            return false;
        }
        if (tall && !mbar_wait(&pp->acc_empty[acc ^ 1], (((t + 1) >> 1) & 1) ^ 1, lim)) {  // the second half: the other buffer
            ctl->abort = 1;
            report(st, ST_MBAR_TIMEOUT, stage_idx);
            return false;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * 256;
        const uint32_t tmem_d2 = tmem_base + (acc ^ 1) * 256;
        for (int k = kb_lo; k < kb_hi; k += G, s = (s + 1 == STAGES ? 0 : s + 1), wrap ^= (s == 0)) {
            if (!mbar_wait(&pp->full[s], ((base_par >> s) ^ wrap) & 1, lim)) {
                ctl->abort = 1;
                report(st, ST_MBAR_TIMEOUT, stage_idx);
                return false;
            }
            tc_fence_after();
            const uint32_t sa0 = smem_u32(smem + s * stage_bytes);
            if (G == 1) {
                const uint32_t sb = sa0 + a_slot;
                const uint64_t da = L.a_mn_major ? umma_desc(sa0, chunk_bytes, 1024) : umma_desc(sa0, 16, 1024);
                const uint64_t db = L.b_mn_major ? umma_desc(sb, chunk_bytes, 1024) : umma_desc(sb, 16, 1024);
#pragma unroll
                for (int kk = 0; kk < kGemmBK / 16; ++kk) {
                    const uint32_t accum = (k > kb_lo || kk > 0) ? 1u : 0u;
                    if constexpr (PAIR) umma_f16_pair(tmem_d, da + (uint64_t)(kk * a_adv), db + (uint64_t)(kk * b_adv), idesc, accum);
                    else umma_f16(tmem_d, da + (uint64_t)(kk * a_adv), db + (uint64_t)(kk * b_adv), idesc, accum);
                }
                if constexpr (TALL) {
                    {  // rows 128..255 of the tile against the same B block (both layouts put them 16 KiB further on)
                        const uint32_t sa2 = sa0 + kGemmABytes;
                        const uint64_t da2 = L.a_mn_major ? umma_desc(sa2, chunk_bytes, 1024) : umma_desc(sa2, 16, 1024);
#pragma unroll
                        for (int kk = 0; kk < kGemmBK / 16; ++kk) {
                            const uint32_t accum = (k > kb_lo || kk > 0) ? 1u : 0u;
                            umma_f16(tmem_d2, da2 + (uint64_t)(kk * a_adv), db + (uint64_t)(kk * b_adv), idesc, accum);
                        }
                    }
                }
            } else {
                const uint32_t sb0 = sa0 + a_slot;
                const int nblk = min(G, kb_hi - k);
                for (int j = 0; j < nblk; ++j) {
                    const uint32_t sa = sa0 + j * a_blk, sb = sb0 + j * b_blk;
                    const uint64_t da = L.a_mn_major ? umma_desc(sa, chunk_bytes, 1024) : umma_desc(sa, 16, 1024);
                    const uint64_t db = L.b_mn_major ? umma_desc(sb, chunk_bytes, 1024) : umma_desc(sb, 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < kGemmBK / 16; ++kk) {
                        const uint32_t accum = (k + j > kb_lo || kk > 0) ? 1u : 0u;
                        if constexpr (PAIR) umma_f16_pair(tmem_d, da + (uint64_t)(kk * a_adv), db + (uint64_t)(kk * b_adv), idesc, accum);
                        else umma_f16(tmem_d, da + (uint64_t)(kk * a_adv), db + (uint64_t)(kk * b_adv), idesc, accum);
                    }
                }
            }
            // free the shared-memory slot once these MMAs have read it
            if constexpr (PAIR) {
                const uint32_t e = smem_u32(&pp->empty[s]);
                umma_commit_pair(mapa_u32(e, 0));
                umma_commit_pair(mapa_u32(e, 1));
            } else {
                umma_commit(&pp->empty[s]);
            }
        }
        if constexpr (PAIR) {  // accumulator complete, in both CTAs
            const uint32_t f = smem_u32(&pp->acc_full[acc]);
            umma_commit_pair(mapa_u32(f, 0));
            umma_commit_pair(mapa_u32(f, 1));
        } else {
            umma_commit(&pp->acc_full[acc]);
            if (tall) {
                umma_commit(&pp->acc_full[acc ^ 1]);
                ++t;  // a tall tile takes two accumulator turns
            }
        }
    }
    return true;
}

// Epilogue: warps 0-3, each on its 32-lane quarter of the accumulator.
template <bool PAIR>
__device__ __noinline__ bool gemm_drain(const GemmRun &R, int warp, int lane) {
    constexpr bool GROUPED = true;
    const GemmLocal &L = R.L;
    const GemmArgs &g = *R.g;
    const GemmArgs *gmaps = R.gmaps;
    char *smem = R.smem;
    GemmPipe *pp = R.pp;
    CtaCtl *ctl = R.ctl;
    DeviceState *st = R.st;
    const int stage_idx = R.stage_idx;
    const unsigned long long lim = R.lim;
    const int STAGES = R.STAGES, G = GROUPED ? R.G : 1, blk_b_bytes = R.blk_b_bytes, stage_bytes = R.stage_bytes;
    const int n_units = R.n_units, kblocks = R.kblocks, crank = R.crank, up = R.up, UP = R.UP, n_half = R.n_half;
    const int splits = R.splits, kper = R.kper;
    const uint32_t base_par = R.base_par, tmem_base = R.tmem_base;
    const unsigned int t0 = R.t0;
    const int tall = PAIR ? 0 : R.tall, a_slot = R.a_slot;
    (void)a_slot;
    const CUtensorMap *tmA = &gmaps->tmA, *tmB = &gmaps->tmB, *tmC = &gmaps->tmC;
    (void)L; (void)g; (void)smem; (void)pp; (void)ctl; (void)st; (void)stage_idx; (void)lim; (void)STAGES; (void)G; (void)blk_b_bytes;
    (void)stage_bytes; (void)n_units; (void)kblocks; (void)crank; (void)up; (void)UP; (void)n_half; (void)splits; (void)kper;
    (void)base_par; (void)tmem_base; (void)t0; (void)tmA; (void)tmB; (void)tmC;
    char *epi_stage = smem + kGemmPipeBytes;
    unsigned int epi_blk = 0;
    unsigned int t = t0;
    for (int u = up, half = 0; u < n_units; ++t) {
        // a tall tile is drained as two tiles of 128 rows, one per accumulator buffer
        TileCoord tc = gemm_unit(g, u / splits);
        tc.m0 += crank * kGemmTileM + half * kGemmTileM;
        const int split = u % splits;
        if (half == tall) { u += UP; half = 0; } else { half = 1; }
        const int acc = t & 1;
        bool ok = mbar_wait(&pp->acc_full[acc], (t >> 1) & 1, lim);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            if (lane == 0) {
                ctl->abort = 1;
                report(st, ST_MBAR_TIMEOUT, stage_idx);
            }
            return false;
        }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + acc * 256;
        if (L.splits > 1) {
            if (L.out_transposed) gemm_epilogue_tile_partial(L, tc, split, tmem_acc, warp, lane);
            else gemm_epilogue_tile_partial_rows(L, tc, split, tmem_acc, warp, lane);
        } else if (L.out_transposed) {
            if (L.dtype == DT_BF16) gemm_epilogue_tile_swapped<__nv_bfloat16>(L, tc, tmem_acc, warp, lane);
            else gemm_epilogue_tile_swapped<__half>(L, tc, tmem_acc, warp, lane);
        } else if (L.c_tma) {
            // fused all_reduce: the tile goes to the rank that sums these rows (tiles never straddle two owners)
            const int owner = L.peer_rows > 0 ? tc.m0 / L.peer_rows : 0;
            const CUtensorMap *tm = L.peer_rows > 0 ? &gmaps->tmPeer[owner] : tmC;
            const int shift = owner * L.peer_rows;
            if (L.dtype == DT_BF16) gemm_epilogue_tile_tma<__nv_bfloat16>(L, tm, tc, tmem_acc, warp, lane, epi_stage, epi_blk, shift);
            else gemm_epilogue_tile_tma<__half>(L, tm, tc, tmem_acc, warp, lane, epi_stage, epi_blk, shift);
        } else {
            if (L.dtype == DT_BF16) gemm_epilogue_tile<__nv_bfloat16>(L, tc, tmem_acc, warp, lane);
            else gemm_epilogue_tile<__half>(L, tc, tmem_acc, warp, lane);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&pp->acc_empty[acc]), 0));
            else mbar_arrive(&pp->acc_empty[acc]);
        }
    }
    // the stage's output must be in global memory before the CTA reaches the next barrier
    if (lane == 0) {
        tma_store_wait<0>();
        if (L.peer_rows > 0) __threadfence_system();  // tiles stored into peer memory: ordered before the peer barrier that follows
    }
    return true;
}

template <bool PAIR, bool GROUPED>
__device__ __noinline__ void run_gemm_t(const GemmArgs &g, const GemmArgs *gmaps, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl,
                           DeviceState *st, int stage_idx, unsigned long long lim) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the record is the same for every thread: one thread builds it in shared memory (per-thread copies would be
    // ~250 bytes of local memory each, written and read back through an L1 that the operand ring leaves little of)
    __shared__ GemmRun Rs;
    __shared__ int my_tiles_s;
    __shared__ unsigned int my_slots_s;
    if (threadIdx.x == 0) {
    GemmRun &R = Rs;
    GemmLocal &L = R.L;
    L.C = g.C; L.bias = g.bias; L.ldc = g.ldc; L.c_stride_c = g.c_stride_c; L.c_stride_n = g.c_stride_n;
    L.M = g.M; L.N = g.N; L.K = g.K; L.tile_n = g.tile_n; L.act = g.act; L.c_vec = g.c_vec; L.c_tma = g.c_tma;
    L.dtype = g.dtype; L.out_transposed = g.out_transposed; L.splits = g.splits; L.ws = g.ws; L.batch_c = g.batch_c;
    L.splits_stride = (int64_t)g.batch_c * g.batch_n * g.M * g.N;
    L.a_mn_major = g.a_mn_major; L.b_mn_major = g.b_mn_major;
    L.a_bc = g.a_bc; L.a_bn = g.a_bn; L.b_bc = g.b_bc; L.b_bn = g.b_bn;
    L.peer_rows = g.peer_rows;
    L.bias_mul = (int)g.bias_mul; L.rope_rows = g.rope_rows; L.rope_cols = g.rope_cols;
    R.g = &g; R.gmaps = gmaps; R.smem = smem; R.pp = pp; R.ctl = ctl; R.st = st; R.lim = lim; R.stage_idx = stage_idx;
    R.STAGES = g.stages;
    R.G = GROUPED ? g.kgroup : 1;
    R.blk_b_bytes = g.stage_b_bytes;
    R.stage_bytes = R.G * (kGemmABytes + R.blk_b_bytes);
    R.n_units = g.n_units;
    R.kblocks = (L.K + kGemmBK - 1) / kGemmBK;
    R.t0 = pp->tile_count;
    // phase bit of every ring slot at the start of this stage; inside the loops the slot index
    // and a wrap bit are stepped by hand (no division on the MMA-issuing thread's critical path)
    R.base_par = 0;
    for (int s = 0; s < R.STAGES; ++s) R.base_par |= (pp->use[s] & 1u) << s;
    R.crank = PAIR ? (p & 1) : 0;          // rank inside the CTA pair
    R.up = PAIR ? (p >> 1) : p;             // which tile walker this CTA belongs to
    R.UP = PAIR ? (P >> 1) : P;
    R.n_half = PAIR ? L.tile_n / 2 : L.tile_n;  // B columns staged by this CTA
    R.tall = (!PAIR && !GROUPED && g.tall) ? 1 : 0;
    R.a_slot = R.G * kGemmABytes * (1 + R.tall);
    R.stage_bytes = R.G * (kGemmABytes * (1 + R.tall) + R.blk_b_bytes);
    // split-K: unit = tile * splits + range; a unit runs k-blocks [kb_lo, kb_hi) of its tile
    R.splits = L.splits > 1 ? L.splits : 1;
    R.kper = g.kper > 0 ? g.kper : (R.kblocks + R.splits - 1) / R.splits;
    int my_tiles = 0;
    unsigned int my_slots = 0;  // ring slots this CTA fills in this stage
    for (int u = R.up; u < R.n_units; u += R.UP) {
        ++my_tiles;
        const int lo = (u % R.splits) * R.kper;
        my_slots += (unsigned int)((min(R.kblocks, lo + R.kper) - lo + R.G - 1) / R.G);
    }
    R.tmem_base = ctl->tmem_base;
    my_tiles_s = my_tiles;
    my_slots_s = my_slots;
    }
    __syncthreads();
    const GemmRun &R = Rs;

    if (warp == kProducerWarp || warp == kProducerWarpB) {
        if (lane == 0) gemm_produce<PAIR, GROUPED>(R, warp);
    } else if (warp == kMmaWarp) {
        if (lane == 0 && R.crank == 0) {
            if constexpr (!PAIR && !GROUPED) {
                if (R.tall) gemm_issue<false, false, true>(R);
                else gemm_issue<false, false, false>(R);
            } else {
                gemm_issue<PAIR, GROUPED, false>(R);
            }
        }
    } else if (warp < kEpiWarps) {
        gemm_drain<PAIR>(R, warp, lane);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int total = my_slots_s;
        for (int s = 0; s < R.STAGES; ++s)
            if (total > (unsigned int)s) pp->use[s] += (total - s + R.STAGES - 1) / R.STAGES;
        pp->tile_count = R.t0 + (unsigned int)my_tiles_s * (unsigned int)(1 + R.tall);
    }
    // the partner may still read this CTA's shared memory / signal its barriers
    if constexpr (PAIR) cluster_sync_all();
    __syncthreads();
}

// Warps without a role in the matmul (7..15) do not enter the stage function: its register save area and the
// GemmRun record are ~0.5 KB of local memory per thread, and with 208 KiB of the SM's memory configured as shared
// there is little L1 left to hold them (an idle pass through the function measured 5.5 us). They only take part in
// the function's three CTA-wide barriers (and the cluster barrier of a pair).
__device__ __forceinline__ bool gemm_warp_has_role() {
    const int warp = threadIdx.x >> 5;
    return warp < kEpiWarps || warp == kProducerWarp || warp == kMmaWarp || warp == kProducerWarpB;
}
__device__ __noinline__ void run_gemm(const GemmArgs &g, const GemmArgs *gmaps, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl,
                         DeviceState *st, int stage_idx, unsigned long long spin_limit) {
    if (!gemm_warp_has_role()) {
        __syncthreads();
        __syncthreads();
        __syncthreads();
        return;
    }
    if (g.kgroup > 1) run_gemm_t<false, true>(g, gmaps, p, P, smem, pp, ctl, st, stage_idx, spin_limit);
    else run_gemm_t<false, false>(g, gmaps, p, P, smem, pp, ctl, st, stage_idx, spin_limit);
}
__device__ __noinline__ void run_gemm_pair(const GemmArgs &g, const GemmArgs *gmaps, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl,
                              DeviceState *st, int stage_idx, unsigned long long spin_limit) {
    if (!gemm_warp_has_role()) {
        __syncthreads();
        __syncthreads();
        cluster_sync_all();
        __syncthreads();
        return;
    }
    if (g.kgroup > 1) run_gemm_t<true, true>(g, gmaps, p, P, smem, pp, ctl, st, stage_idx, spin_limit);
    else run_gemm_t<true, false>(g, gmaps, p, P, smem, pp, ctl, st, stage_idx, spin_limit);
}

// Sums the split-K partials (fixed order: deterministic), adds the optional bias,
// applies the activation and rounds once. Four outputs per thread step.
template <typename T>
__device__ void splitk_reduce_typed(const SplitKReduceArgs &a, int p, int P) {
    const int64_t per = (int64_t)a.M * a.N, total = per * a.batch_c * a.batch_n;
    const int64_t tid = (int64_t)p * kThreads + threadIdx.x, nth = (int64_t)P * kThreads;
    const bool vec = (a.N % 4 == 0);
    const int64_t step = vec ? 4 : 1;
    for (int64_t e0 = tid * step; e0 < total; e0 += nth * step) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < a.splits; ++s) {
            const float *w = a.ws + (int64_t)s * total + e0;
            if (vec) {
                const float4 v = *reinterpret_cast<const float4 *>(w);
                acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
            } else {
                acc[0] += w[0];
            }
        }
        for (int i = 0; i < step; ++i) {
            const int64_t e = e0 + i;
            const int64_t b = e / per, r = e % per;
            const int64_t m = r / a.N, n = r % a.N;
            const int64_t off = (b / a.batch_c) * a.c_stride_n + (b % a.batch_c) * a.c_stride_c + m * a.ldc + n;
            float v = acc[i];
            if (a.bias) v += to_f32(reinterpret_cast<const T *>(a.bias)[off]);
            reinterpret_cast<T *>(a.C)[off] = from_f32<T>(apply_act_fast(a.act, v));
        }
    }
}

__device__ __noinline__ void run_splitk_reduce(const SplitKReduceArgs &a, int p, int P) {
    if (a.dtype == DT_BF16) splitk_reduce_typed<__nv_bfloat16>(a, p, P);
    else splitk_reduce_typed<__half>(a, p, P);
}

// ---- CUDA-core fallback -------------------------------------------------------------
// For operands the TMA path cannot describe (row pitch or base not 16-byte
// aligned) and for fp32. 64x64 tile per CTA pass, fp32 accumulate.
template <typename T>
__device__ void gemm_simt_typed(const GemmSimtArgs &g, int p, int P, char *smem) {
    constexpr int TM = 64, TN = 64, TK = 16;
    float(*sA)[TM + 1] = reinterpret_cast<float(*)[TM + 1]>(smem);                          // [TK][TM+1]
    float(*sB)[TN + 1] = reinterpret_cast<float(*)[TN + 1]>(smem + TK * (TM + 1) * 4);      // [TK][TN+1]
    const int tiles_m = (g.M + TM - 1) / TM, tiles_n = (g.N + TN - 1) / TN;
    const int per = tiles_m * tiles_n;
    const int total = per * g.batch_c * g.batch_n;
    const int tid = threadIdx.x;
    // 512 threads: thread computes a 2x4 block of the 64x64 tile
    const int ty = tid / 16, tx = tid % 16;  // ty 0..31 -> rows ty*2.., tx -> cols tx*4..
    for (int u = p; u < total; u += P) {
        const int b = u / per, r = u % per;
        const int bc = b % g.batch_c, bn = b / g.batch_c;
        const int m0 = (r / tiles_n) * TM, n0 = (r % tiles_n) * TN;
        const T *A = reinterpret_cast<const T *>(g.A) + bn * g.a_stride_n + bc * g.a_stride_c;
        const T *B = reinterpret_cast<const T *>(g.B) + bn * g.b_stride_n + bc * g.b_stride_c;
        T *C = reinterpret_cast<T *>(g.C) + bn * g.c_stride_n + bc * g.c_stride_c;
        float acc[2][4] = {};
        for (int k0 = 0; k0 < g.K; k0 += TK) {
            for (int i = tid; i < TK * TM; i += kThreads) {
                int kk = i / TM, mm = i % TM;
                if (!g.trans_a) { mm = i / TK; kk = i % TK; }
                int m = m0 + mm, k = k0 + kk;
                float v = 0.0f;
                if (m < g.M && k < g.K) v = to_f32(g.trans_a ? A[(int64_t)k * g.lda + m] : A[(int64_t)m * g.lda + k]);
                sA[kk][mm] = v;
            }
            for (int i = tid; i < TK * TN; i += kThreads) {
                int kk = i / TN, nn = i % TN;
                if (g.trans_b) { nn = i / TK; kk = i % TK; }
                int n = n0 + nn, k = k0 + kk;
                float v = 0.0f;
                if (n < g.N && k < g.K) v = to_f32(g.trans_b ? B[(int64_t)n * g.ldb + k] : B[(int64_t)k * g.ldb + n]);
                sB[kk][nn] = v;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < TK; ++kk) {
                float a0 = sA[kk][ty * 2], a1 = sA[kk][ty * 2 + 1];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float bv = sB[kk][tx * 4 + j];
                    acc[0][j] += a0 * bv;
                    acc[1][j] += a1 * bv;
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int m = m0 + ty * 2 + i, n = n0 + tx * 4 + j;
                if (m < g.M && n < g.N) C[(int64_t)m * g.ldc + n] = from_f32<T>(apply_act(g.act, acc[i][j]));
            }
    }
}

__device__ __noinline__ void run_gemm_simt(const GemmSimtArgs &g, int p, int P, char *smem) {
    switch (g.dtype) {
        case DT_F32: gemm_simt_typed<float>(g, p, P, smem); break;
        case DT_F16: gemm_simt_typed<__half>(g, p, P, smem); break;
        case DT_BF16: gemm_simt_typed<__nv_bfloat16>(g, p, P, smem); break;
        default: break;
    }
}

}  // namespace arkb
