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

template <typename T>
__device__ __forceinline__ void gemm_store_row(const GemmArgs &g, T *crow, const T *brow, int col, int ncols,
                                               uint32_t (&r)[32], int cnt) {
    // cnt accumulator values (16 or 32) for columns [col, col+cnt) of one row
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = (i < cnt) ? __uint_as_float(r[i]) : 0.0f;
    const bool full = (col + cnt <= ncols) && g.c_vec;
    if (full) {
        if (brow) {
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
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = apply_act(g.act, f[i]);
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
                if (brow) v += to_f32(brow[col + i]);
                crow[col + i] = from_f32<T>(apply_act(g.act, v));
            }
        }
    }
}

template <typename T>
__device__ void gemm_epilogue_tile(const GemmArgs &g, const TileCoord &tc, uint32_t tmem_acc, int warp, int lane) {
    const int row = tc.m0 + warp * 32 + lane;
    const bool row_ok = row < g.M;
    const int64_t boff = (int64_t)tc.bn * g.c_stride_n + (int64_t)tc.bc * g.c_stride_c + (int64_t)row * g.ldc;
    T *crow = reinterpret_cast<T *>(g.C) + boff;
    const T *brow = g.bias ? reinterpret_cast<const T *>(g.bias) + boff : nullptr;
    const uint32_t lane_addr = tmem_acc + ((uint32_t)(warp * 32) << 16);
    const int ncols_tile = min(g.tile_n, g.N - tc.n0);  // valid columns of this tile
    for (int c = 0; c < g.tile_n; c += 32) {
        if (c >= ncols_tile) break;  // uniform across the warp
        uint32_t r[32];
        const int cnt = (g.tile_n - c >= 32) ? 32 : 16;
        if (cnt == 32) tmem_ld32(lane_addr + c, r);
        else tmem_ld16(lane_addr + c, r);
        tmem_ld_wait();
        if (row_ok) gemm_store_row<T>(g, crow + tc.n0, brow ? brow + tc.n0 : nullptr, c, ncols_tile, r, cnt);
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
template <bool PAIR>
__device__ void run_gemm_t(const GemmArgs &g, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl, DeviceState *st,
                           int stage_idx, unsigned long long lim) {
    using Cfg = GemmCfg<PAIR>;
    constexpr int STAGES = Cfg::kStages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (g.K + kGemmBK - 1) / kGemmBK;
    const unsigned int kb0 = pp->kb_count, t0 = pp->tile_count;
    const int crank = PAIR ? (p & 1) : 0;          // rank inside the CTA pair
    const int up = PAIR ? (p >> 1) : p;             // which tile walker this CTA belongs to
    const int UP = PAIR ? (P >> 1) : P;
    const int n_half = PAIR ? g.tile_n / 2 : g.tile_n;  // B columns staged by this CTA
    int my_tiles = 0;
    for (int u = up; u < g.n_units; u += UP) ++my_tiles;
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == kProducerWarp) {
        if (lane == 0) {
            const int a_chunks = g.a_mn_major ? 2 : 1;                     // 64-wide M chunks
            const int b_chunks = g.b_mn_major ? (n_half + 63) / 64 : 1;    // 64-wide N chunks
            const uint32_t a_bytes = kGemmABytes;
            const uint32_t b_bytes = g.b_mn_major ? (uint32_t)b_chunks * 64 * kGemmBK * 2 : (uint32_t)n_half * kGemmBK * 2;
            unsigned int kb = kb0;
            for (int u = up; u < g.n_units; u += UP) {
                TileCoord tc = gemm_unit(g, u);
                tc.m0 += crank * kGemmTileM;
                tc.n0 += crank * n_half;
                const int a_c = g.a_bc ? tc.bc : 0, a_n = g.a_bn ? tc.bn : 0;
                const int b_c = g.b_bc ? tc.bc : 0, b_n = g.b_bn ? tc.bn : 0;
                for (int k = 0; k < kblocks; ++k, ++kb) {
                    const int s = kb % STAGES;
                    const uint32_t par = ((kb / STAGES) & 1) ^ 1;
                    if (!mbar_wait(&pp->empty[s], par, lim)) {
                        ctl->abort = 1;
                        report(st, ST_MBAR_TIMEOUT, stage_idx);
                        goto done;
                    }
                    char *sa = smem + s * Cfg::kStageBytes;
                    char *sb = sa + kGemmABytes;
                    if constexpr (!PAIR) {
                        mbar_expect_tx(&pp->full[s], a_bytes + b_bytes);
                        if (!g.a_mn_major) {
                            tma_load_4d(sa, &g.tmA, &pp->full[s], k * kGemmBK, tc.m0, a_c, a_n);
                        } else {
                            for (int c = 0; c < a_chunks; ++c)
                                tma_load_4d(sa + c * 64 * kGemmBK * 2, &g.tmA, &pp->full[s], tc.m0 + c * 64, k * kGemmBK, a_c, a_n);
                        }
                        if (!g.b_mn_major) {
                            tma_load_4d(sb, &g.tmB, &pp->full[s], k * kGemmBK, tc.n0, b_c, b_n);
                        } else {
                            for (int c = 0; c < b_chunks; ++c)
                                tma_load_4d(sb + c * 64 * kGemmBK * 2, &g.tmB, &pp->full[s], tc.n0 + c * 64, k * kGemmBK, b_c, b_n);
                        }
                    } else {
                        const uint32_t full_leader = mapa_u32(smem_u32(&pp->full[s]), 0);
                        if (crank == 0) mbar_expect_tx(&pp->full[s], 2 * (a_bytes + b_bytes));
                        if (!g.a_mn_major) {
                            tma_load_4d_pair(sa, &g.tmA, full_leader, k * kGemmBK, tc.m0, a_c, a_n);
                        } else {
                            for (int c = 0; c < a_chunks; ++c)
                                tma_load_4d_pair(sa + c * 64 * kGemmBK * 2, &g.tmA, full_leader, tc.m0 + c * 64, k * kGemmBK, a_c, a_n);
                        }
                        if (!g.b_mn_major) {
                            tma_load_4d_pair(sb, &g.tmB, full_leader, k * kGemmBK, tc.n0, b_c, b_n);
                        } else {
                            for (int c = 0; c < b_chunks; ++c)
                                tma_load_4d_pair(sb + c * 64 * kGemmBK * 2, &g.tmB, full_leader, tc.n0 + c * 64, k * kGemmBK, b_c, b_n);
                        }
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0 && crank == 0) {
            const uint32_t idesc = umma_idesc(g.dtype == DT_BF16, g.a_mn_major, g.b_mn_major, g.tile_n, PAIR ? 256 : 128);
            // per-MMA (K=16) advance of the descriptor start address, in 16-byte units
            const uint32_t a_adv = g.a_mn_major ? (16 * 128) >> 4 : 32 >> 4;
            const uint32_t b_adv = g.b_mn_major ? (16 * 128) >> 4 : 32 >> 4;
            const uint32_t chunk_bytes = 64 * kGemmBK * 2;  // one 64-wide MN chunk
            unsigned int kb = kb0, t = t0;
            for (int i = 0; i < my_tiles; ++i, ++t) {
                const int acc = t & 1;
                if (!mbar_wait(&pp->acc_empty[acc], ((t >> 1) & 1) ^ 1, lim)) {
                    ctl->abort = 1;
                    report(st, ST_MBAR_TIMEOUT, stage_idx);
                    goto done;
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * 256;
                for (int k = 0; k < kblocks; ++k, ++kb) {
                    const int s = kb % STAGES;
                    if (!mbar_wait(&pp->full[s], (kb / STAGES) & 1, lim)) {
                        ctl->abort = 1;
                        report(st, ST_MBAR_TIMEOUT, stage_idx);
                        goto done;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
                    const uint32_t sb = sa + kGemmABytes;
                    const uint64_t da = g.a_mn_major ? umma_desc(sa, chunk_bytes, 1024) : umma_desc(sa, 16, 1024);
                    const uint64_t db = g.b_mn_major ? umma_desc(sb, chunk_bytes, 1024) : umma_desc(sb, 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < kGemmBK / 16; ++kk) {
                        const uint32_t accum = (k > 0 || kk > 0) ? 1u : 0u;
                        if constexpr (PAIR) umma_f16_pair(tmem_d, da + (uint64_t)(kk * a_adv), db + (uint64_t)(kk * b_adv), idesc, accum);
                        else umma_f16(tmem_d, da + (uint64_t)(kk * a_adv), db + (uint64_t)(kk * b_adv), idesc, accum);
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
                }
            }
        }
    } else if (warp < kEpiWarps) {
        unsigned int t = t0;
        for (int u = up; u < g.n_units; u += UP, ++t) {
            TileCoord tc = gemm_unit(g, u);
            tc.m0 += crank * kGemmTileM;
            const int acc = t & 1;
            bool ok = mbar_wait(&pp->acc_full[acc], (t >> 1) & 1, lim);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) {
                    ctl->abort = 1;
                    report(st, ST_MBAR_TIMEOUT, stage_idx);
                }
                goto done;
            }
            tc_fence_after();
            const uint32_t tmem_acc = tmem_base + acc * 256;
            if (g.dtype == DT_BF16) gemm_epilogue_tile<__nv_bfloat16>(g, tc, tmem_acc, warp, lane);
            else gemm_epilogue_tile<__half>(g, tc, tmem_acc, warp, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if constexpr (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&pp->acc_empty[acc]), 0));
                else mbar_arrive(&pp->acc_empty[acc]);
            }
        }
    }
done:
    __syncthreads();
    if (threadIdx.x == 0) {
        pp->kb_count = kb0 + (unsigned int)my_tiles * (unsigned int)kblocks;
        pp->tile_count = t0 + (unsigned int)my_tiles;
    }
    // the partner may still read this CTA's shared memory / signal its barriers
    if constexpr (PAIR) cluster_sync_all();
    __syncthreads();
}

__device__ void run_gemm(const GemmArgs &g, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl, DeviceState *st,
                         int stage_idx, unsigned long long spin_limit) {
    run_gemm_t<false>(g, p, P, smem, pp, ctl, st, stage_idx, spin_limit);
}
__device__ void run_gemm_pair(const GemmArgs &g, int p, int P, char *smem, GemmPipe *pp, CtaCtl *ctl, DeviceState *st,
                              int stage_idx, unsigned long long spin_limit) {
    run_gemm_t<true>(g, p, P, smem, pp, ctl, st, stage_idx, spin_limit);
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

__device__ void run_gemm_simt(const GemmSimtArgs &g, int p, int P, char *smem) {
    switch (g.dtype) {
        case DT_F32: gemm_simt_typed<float>(g, p, P, smem); break;
        case DT_F16: gemm_simt_typed<__half>(g, p, P, smem); break;
        case DT_BF16: gemm_simt_typed<__nv_bfloat16>(g, p, P, smem); break;
        default: break;
    }
}

}  // namespace arkb
