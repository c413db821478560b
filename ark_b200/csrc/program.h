// Device program: what the host lowers a plan into and what the persistent
// loop kernel walks. Shared between host C++ and CUDA device code.
//
// A plan (reference format: docs/plan_file.md) is lowered to a flat list of
// stages. Every CTA of the grid walks the whole list once per iteration and
// executes the stages whose processor range contains it. This is the
// counterpart of the reference's generated `ark_body` (a straight-line list
// of `task_seq<...>` calls and `sync_gpu` barriers, ark/codegen.cpp:119-151,
// ark/include/kernels/kernel_template.in:6-69), held as data instead of
// generated source so that one prebuilt sm_100a kernel runs any plan.
#pragma once
#include <stdint.h>

#include <cuda.h>  // CUtensorMap

namespace arkb {

constexpr int kThreads = 512;       // threads per CTA of the loop kernel
constexpr int kMaxSyncGroups = 64;  // distinct processor ranges that get a barrier
constexpr int kMaxPeers = 8;

enum DType : int32_t { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_I32 = 3, DT_U32 = 4, DT_I8 = 5, DT_U8 = 6 };

enum StageKind : int32_t {
    SK_SYNC = 0,       // barrier over a processor range
    SK_EWISE = 1,      // unary / binary / scalar / cast / copy / rope, NumPy broadcast
    SK_REDUCE = 2,     // sum / mean / max along one axis
    SK_GEMM = 3,       // tcgen05 tiled matmul (+ fused epilogue)
    SK_GEMV = 4,       // skinny matmul (few rows): weight streaming
    SK_TRANSPOSE = 5,  // 4-D permutation
    SK_EMBED = 6,      // row gather
    SK_ROWOP = 7,      // fused row kernels: rmsnorm / layernorm / softmax
    SK_PUT = 8,        // copy a local tensor into a peer's arena (data phase of send)
    SK_WAITFLAG = 9,   // wait until a peer raised a channel flag (recv)
    SK_PEERSYNC = 10,  // barrier across ranks (device_sync)
    SK_ALLREDUCE = 11, // data phase of the in-kernel all_reduce
    SK_GEMM_SIMT = 12, // CUDA-core matmul for shapes the TMA path cannot take
    SK_SIGNAL = 13,    // raise a channel flag on a peer (after the put's data is complete)
    SK_SPLITK_REDUCE = 14,  // sum the fp32 partials of a split-K matmul, add bias, activate, round, store
    SK_DECODE_ATTN = 15,    // one query row per head against a K/V cache: scores, softmax and output in one pass over the cache
    SK_PACKET = 16,         // flag-carrying packets: local data -> a peer's packet buffer, or local packet buffer -> local data
    SK_PACKET_REDUCE = 17,  // own shard + the shards the peers sent (packets or plain) -> local output and every peer's output
    SK_PREFILL_ATTN = 18,   // many query rows per head: S = Q K^T, online softmax and O = P V per 128-row tile, scores stay on chip
};

enum EwiseOp : int32_t {
    EW_COPY = 0, EW_GELU, EW_EXP, EW_RELU, EW_RSQRT, EW_SIGMOID, EW_SQRT, EW_CAST,
    EW_ADD, EW_SUB, EW_MUL, EW_DIV,
    EW_SCALAR_ASSIGN, EW_SCALAR_ADD, EW_SCALAR_MUL,
    EW_ROPE, EW_SILU,
};
enum ReduceOp : int32_t { RD_SUM = 0, RD_MAX = 1, RD_MEAN = 2 };
enum RowOp : int32_t { RO_RMSNORM = 0, RO_LAYERNORM = 1, RO_SOFTMAX = 2 };
enum ActOp : int32_t { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SIGMOID = 3, ACT_SILU = 4 };

// A strided view of up to 4 dims. `stride` is in elements and already 0 for
// broadcast dims; `ptr` already includes the view's offsets.
struct TRef {
    void *ptr;
    int32_t shape[4];
    int64_t stride[4];
    int32_t dtype;
    int32_t contiguous;  // 1 when the view covers a dense row-major block
};

struct EwiseArgs {
    TRef out, in0, in1;
    int32_t op;
    int32_t vec;        // elements per thread access along W (1 or 16/sizeof)
    int32_t flat;       // 1: all operands dense and same shape -> 1-D walk
    float scalar;
    int64_t n_units;    // number of vec units
    // Copy only: a ring of `iter_slots` buffers walked by the iteration number. Iteration i (1-based over the
    // executor's life) reads in0 + ((i - 1) % iter_slots) * in_iter_bytes and writes out + ... * out_iter_bytes,
    // so the host can fill or drain the other slots while the iteration runs. iter_slots <= 1: fixed addresses.
    int32_t iter_slots, pad;
    int64_t in_iter_bytes, out_iter_bytes;
    // A task group that covers only part of the operator's tasks (TaskRange [b, e) step s): task id -> output tile
    // (n, c, tile row, tile column), column fastest, as the reference's UnitOp enumerates them
    // (ark/include/kernels/common/unit_op.h); only elements of those tiles are written. task_s == 0: all of it.
    int32_t task_b, task_e, task_s;
    int32_t tile_h, tile_w, tiles_h, tiles_w, pad2;
};

struct ReduceArgs {
    TRef out, in;       // out has shape 1 along `axis`
    int32_t op;
    int32_t axis;       // 0..3 in 4-D form
    int32_t vec;        // vector width usable on the innermost dim
    int32_t partial;    // 1: only the tasks task_b, task_b + task_s, ... < task_e run (a task = one output element, in the order of the 4-D output)
    int64_t task_b, task_e, task_s;
};

struct RowOpArgs {
    void *out;
    const void *in;
    const void *weight;    // optional (rmsnorm scale), broadcast over rows
    const void *residual;  // optional: in := in + residual before the norm (also written to res_out)
    void *res_out;
    int64_t rows, cols;
    int64_t in_ld, out_ld;
    int32_t op, dtype;
    float eps;
    float scale;           // softmax: logits are multiplied by this first
    int32_t warps_per_row; // 1,2,4,8,16: the row is held in registers by that many warps; 0: two-pass fallback
    int32_t staged_warps;  // > 0: rows are streamed through shared memory with bulk copies by this many warps,
                           // each with `staged_bufs` row buffers (takes precedence over warps_per_row)
    int32_t staged_bufs;
    int32_t mask_rows;     // softmax: logits := logits * scale + mask[row % mask_rows] first (rounded to the storage type)
    const void *mask;      // optional additive mask, mask_rows x cols, row pitch mask_ld
    int64_t mask_ld;
    int32_t weight_f32;    // 1: `weight` holds fp32 values whatever the rows' type (the llama example keeps its norm weights in fp32)
    int32_t weight_smem;   // staged form: the CTA copies the weight row into shared memory (behind the row buffers) once,
                           // instead of every warp fetching it from L2 a vector at a time for every row
};

// Shared memory the loop kernel offers a matmul stage for operand ring slots when its epilogue needs no staging
// area (the swapped and split-K forms); stages with a TMA-store epilogue use the first 192 KiB only.
constexpr int kSwappedRingBytes = 208 * 1024;

struct GemmArgs {
    CUtensorMap tmA;  // dims {inner, rows, C, N}; box {64, 128 or 64, 1, 1}, 128-byte swizzle
    CUtensorMap tmB;  // dims {inner, rows, C, N}; box {64, tile_n or 64, 1, 1}
                      // kgroup > 1, K-major operand: dims {64, rows, K/64, C, N}, box {64, rows, kgroup, 1, 1}
                      // kgroup > 1, MN-major operand: the 4-d map with box {64, 64 * kgroup, 1, 1}
    CUtensorMap tmC;  // output, dims {N, M, C, N}; box {32, 32, 1, 1}, 64-byte swizzle (used when c_tma)
    // Matmul fused with the all_reduce that follows it: the epilogue stores each tile of the partial product
    // straight into the staging slot this rank owns on the rank that will sum those rows (peer memory).
    // tmPeer[r]: dims {N, peer_rows}, rank r's slot for this rank; rows [r * peer_rows, (r+1) * peer_rows) go there.
    CUtensorMap tmPeer[kMaxPeers];
    void *C;
    const void *bias;     // optional tensor combined with the result in the epilogue (same layout as C)
    int32_t bias_mul;     // 0: result = act(acc + bias); 1: result = act(acc) * bias;
                          // 2: rotary embedding: `bias` is a table [rope_rows][rope_cols] of (cos, sin) pairs, row r of the
                          //    result uses table row r % rope_rows, column c pairs with table column c % rope_cols:
                          //    (x0, x1) -> (x0 cos - x1 sin, x0 sin + x1 cos)
    int32_t rope_rows, rope_cols, pad_b;
    int64_t ldc;
    int64_t c_stride_c, c_stride_n;  // batch strides of C in elements
    int32_t M, N, K;
    int32_t batch_c, batch_n;        // output batch dims
    int32_t a_bc, a_bn, b_bc, b_bn;  // 1 when the operand has that batch dim (else broadcast: coordinate 0)
    int32_t a_mn_major, b_mn_major;  // 0: K-major (inner dim = K), 1: MN-major (inner dim = M or N)
    int32_t dtype;                   // DT_F16 / DT_BF16
    int32_t act;
    int32_t tile_n;                  // UMMA N (multiple of 16, <= 256)
    int32_t c_vec;                   // 1: C rows allow 16-byte stores
    int32_t c_tma;                   // 1: the epilogue stages 32x32 blocks in shared memory and stores them with TMA
    int32_t kgroup;                  // k-blocks brought by one ring slot (1, 2 or 4): one bulk tensor copy per operand per slot
    // Unit enumeration. plan_tiles == 0: units are this engine's own tiles
    // (128 x tile_n) over the whole output, rasterised in groups of
    // `raster_group` m-tiles. plan_tiles == 1: units follow the plan's task ids
    // (task id -> (n, c, tile_h, tile_w), w fastest, as the reference's UnitOp
    // does, ark/include/kernels/common/unit_op.h), each plan tile of
    // ptm x ptn being cut into sub_m x sub_n sub-tiles of 128 x tile_n.
    int32_t plan_tiles;
    int32_t tiles_m, tiles_n, raster_group;
    int32_t ptm, ptn, p_tiles_h, p_tiles_w, sub_m, sub_n, task_b, task_s;
    int32_t n_units;
    int32_t tile_m;                  // 128 (one CTA per tile) or 256 (CTA pair per tile)
    int32_t stages, stage_b_bytes;   // ring depth and bytes of the B block of one stage (A block: 16 KiB)
    int32_t out_transposed;          // 1: operands are swapped (A = weights, B = activations); D[n][m] is stored to C[m][n]
    int32_t splits;                  // > 1: K is cut into `splits` ranges; unit = tile * splits + range, fp32 partials go to `ws`
    int32_t kper;                    // k-blocks per range (a multiple of kgroup); 0: ceil(k-blocks / splits)
    int32_t tall;                    // 1 (one CTA per tile only): the CTA owns 256 x tile_n tiles as two 128-row halves that share
                                     // the B block of every ring slot (a third fewer operand bytes per flop at tile_n 256); the
                                     // halves take both accumulator buffers, so the epilogue does not overlap the next tile
    float *ws;                       // split-K partials, layout [splits][batch][rows of C][cols of C]
    int32_t peer_rows;               // > 0: fused all_reduce, rows of C each rank sums (M / ranks)
    int32_t pad3;
};

// Second half of a split-K matmul: C = act(sum_s ws[s] + bias), one rounding.
struct SplitKReduceArgs {
    void *C;
    const void *bias;
    const float *ws;
    int64_t ldc, c_stride_c, c_stride_n;
    int32_t M, N, batch_c, batch_n;
    int32_t splits, dtype, act, pad;
};

struct GemvArgs {
    // y[M, N] = x[M, K] . W with M <= kGemvMaxM on the CUDA cores; W is [N, K] (w_is_nk) or [K, N]
    void *out;        // y, row pitch ldo (written when splits == 1)
    const void *x;    // activations, row pitch ldx
    const void *w;    // weights, row pitch ldw
    float *ws;        // splits > 1: fp32 partials [splits][M][N]
    int64_t ldx, ldw, ldo;
    int32_t M, N, K;
    int32_t w_is_nk;
    int32_t dtype, act;
    int32_t splits;          // k-ranges
    int32_t kper;            // elements of K per range ([N, K]: a multiple of 8)
    int32_t ctas_per_split;  // [N, K]: CTAs that share a k-range and split the rows of W
    int32_t nblocks;         // [K, N]: blocks of 256 output columns
    int32_t rows_together;   // [N, K]: rows of W a warp walks together (8, 4, 2 or 1 for M = 1; 4, 2 or 1 for M = 2)
    // Operators of the same task folded into this stage (each CTA applies the prologue to the activations while
    // it stages them, so the producer needs no stage and no barrier of its own):
    int32_t pro;             // GP_NONE; GP_RMSNORM: x := rmsnorm(x [+ pro_b]) * pro_a; GP_MUL: x := x * pro_a
    const void *pro_a;       // GP_RMSNORM: weight [K] (may be null); GP_MUL: second operand [M, K], row pitch ldx
    const void *pro_b;       // GP_RMSNORM: optional residual [M, K] added first (row pitch ldx)
    void *pro_out;           // GP_RMSNORM with residual: x + residual is also stored here (by CTA 0), row pitch ldx
    float pro_eps;
    int32_t src_ord;         // > 0: x is the sum of the one-shot all_reduce number src_ord - 1, whose partials still lie in this
                             // rank's staging slots (dense [M, K] per rank): the stage adds them up itself
    const void *residual;    // epilogue: y := act(x . W) + residual [M, N] (row pitch ldo); with k-ranges the sum stage adds it
    // The one-shot all_reduce that follows in the same task: the result is also stored into slot [rank] of every rank's
    // staging buffer (the all_reduce's own push stage and its barrier are then left out). push_ord = its ordinal + 1, 0: none.
    int32_t push_ord, push_per_iter;
    uint64_t push_stage_bytes;
    int32_t light;           // [N, K]: the walker with half the loads in flight and a third of the registers (small matrices)
    // GP_ATTN_MERGE: x is the output of a decode attention whose chunks have not been merged yet: x[b, h * 128 + d] is
    // put together from the chunk records (pro_a = the attention's scratch: per (b, kv head, chunk) G x (128 outputs +
    // maximum + sum), fp32) while the activations are staged; M = sequences
    int32_t mg_chunks, mg_group, mg_kv_heads;
    // A second matrix of the same shape over the same activations ([N, K] layout, one k-range): rows N .. 2N-1 of the
    // stage's row space are rows of w_b, their results go to out_b with activation act_b (W1 and W3 of a SwiGLU block:
    // one stage, one staging of x, the CTAs' shares are halves of both)
    int32_t act_b;
    const void *w_b;
    void *out_b;
};
enum GemvPrologue : int32_t { GP_NONE = 0, GP_RMSNORM = 1, GP_MUL = 2, GP_ATTN_MERGE = 3 };
constexpr int kGemvMaxM = 2;

// softmax(scale * q . K^T) . V for one query row per head (decode); phase 0: per cache chunk, phase 1: merge the chunks
struct DecodeAttnArgs {
    void *out;                 // [B, Hq, 1, 128]
    const void *q, *k, *v;     // q [B, Hq, 1, 128]; k, v [B, Hkv, T, 128]
    float *ws;                 // per (b, kv head, chunk): G x (128 outputs + maximum + sum), fp32
    int64_t q_stride_b, q_stride_h, o_stride_b, o_stride_h;          // elements
    int64_t k_stride_b, k_stride_h, k_ld, v_stride_b, v_stride_h, v_ld;
    int32_t B, Hq, Hkv, T;
    int32_t chunks, chunk_len;  // the cache is cut into `chunks` pieces of chunk_len keys (a multiple of 32)
    int32_t dtype, phase;
    float scale;
    int32_t pad;
    const void *rope;          // optional: 128 (cos, sin) values of the token's position; q is rotated while it is loaded
    int64_t pad6;
};

// Self-attention over Tq query rows per head (head dimension 128). The tensors are addressed through tensor maps
// of dims {128, T, H, B}, so both [B, H, T, 128] and [B, T, H, 128] storage work.
struct PrefillAttnArgs {
    alignas(64) CUtensorMap tmQ;  // box {64, 128}: K-major operand blocks
    alignas(64) CUtensorMap tmK;  // box {64, 128}
    alignas(64) CUtensorMap tmV;  // box {64, 64}: MN-major operand chunks
    void *out;
    int64_t o_stride_b, o_stride_h, o_stride_t;  // elements
    int32_t B, Hq, Hkv, Tq, Tkv;
    int32_t causal;   // 1: row i attends to keys [0, i + Tkv - Tq]
    int32_t dtype;
    float scale;      // applied to q.k before the softmax
    int32_t n_units, q_tiles;
    const void *mask; // optional additive mask [B or 1, Hq or 1, Tq, Tkv] of the operands' type, added to scale * q.k
    int64_t m_stride_b, m_stride_h, m_stride_q;  // elements; 0 on a broadcast axis
};

struct GemmSimtArgs {
    void *C;
    const void *A;
    const void *B;
    int64_t lda, ldb, ldc;
    int64_t a_stride_c, a_stride_n, b_stride_c, b_stride_n, c_stride_c, c_stride_n;
    int32_t M, N, K;
    int32_t batch_c, batch_n;
    int32_t trans_a, trans_b;
    int32_t dtype, act;
};

struct TransposeArgs {
    TRef out, in;      // out.shape[i] == in.shape[perm[i]]
    int32_t perm[4];
    // partial != 0: only the tasks task_b, task_b + task_s, ... < task_e run; a task is a tile_h x tile_w tile of the two
    // innermost output dims, numbered (n, c, tile row, tile column) with the column fastest
    int32_t partial, tile_h, tile_w, pad;
    int64_t task_b, task_e, task_s;
};

struct EmbedArgs {
    void *out;
    const int32_t *idx;
    const void *weight;
    int64_t n_idx, num_emb, emb_dim;  // emb_dim in elements
    int64_t w_ld, out_ld;
    int32_t esize, pad;
    int64_t task_b, task_s;  // the rows gathered are task_b, task_b + task_s, ... (n_idx of them); 0, 1: all
};

struct PutArgs {
    void *dst;           // points into the peer's arena mapping
    const void *src;
    int64_t bytes;       // dense copy
    int32_t peer;
    int32_t iter_slots;  // > 1: the source is a ring of buffers walked by the iteration number (see EwiseArgs)
    int64_t src_iter_bytes;
};
struct SignalArgs {
    int32_t peer;        // rank whose comm block gets the flag
    int32_t channel;     // flag index on the receiver: sender_rank * kChannels + channel
};
struct WaitArgs {
    int32_t peer;        // sender rank
    int32_t channel;
};
struct PeerSyncArgs {
    int32_t ord;         // 1-based ordinal of this cross-rank barrier within an iteration
    // 1: the stage is also the grid barrier before and after the exchange: every CTA arrives on the stage's counter,
    // CTA 0 waits for all of them, signals and waits for the peers, and arrives once more, which releases the others
    // (the counter advances by sync_count = CTAs + 1 per barrier)
    int32_t with_grid;
};
// Packets (the reference's SendPacket / RecvPacket, ark/include/kernels/comm.h:376-396): every 8 bytes of payload
// travel as one 16-byte store {d0, flag, d1, flag}, so data and "it has arrived" are the same write and the receiver
// needs neither a signal nor a barrier: it polls the flag words. A packet buffer is twice the size of its payload
// (as the reference sizes them, ark/ops/ops_communication.cpp:183-187). The flag a plan gives is combined with the
// iteration number, so packets of an earlier iteration are never taken for new ones.
struct PacketArgs {
    void *dst;               // get == 0: the peer's packet buffer; get == 1: local data
    const void *src;         // get == 0: local data; get == 1: local packet buffer
    int64_t payload_bytes;   // a multiple of 8
    uint32_t flag;
    int32_t get;
};
// The reduce step of the reference's two all_reduce compositions (read_reduce_and_write, comm.h:398-428):
// out = in + sum of the `npeers` shards the peers put into `scratch` (slot q = q-th peer in rank order), stored
// locally and into every peer's output. packets == 1: scratch slots and peer outputs are packet buffers;
// packets == 0: plain data (a DeviceSync before and after orders it).
struct PacketReduceArgs {
    void *out;
    const void *in;
    const void *scratch;
    void *peer_out[kMaxPeers];
    int64_t nelem;
    int32_t dtype, npeers, packets;
    uint32_t flag;
};

// Data phase of all_reduce over a dense tensor that sits at the same arena
// offset on every rank.
//   algo 0 (one-shot, small): phase 0 pushes the local tensor into slot
//     [rank] of every peer's staging area; phase 1 (after a cross-rank
//     barrier) sums the slots in rank order into the local tensor.
//   algo 1 (two-shot, large): after a cross-rank barrier every rank sums its
//     1/p shard from all ranks' tensors (peer loads, rank order, fp32) and
//     stores the rounded result into every rank's tensor (peer stores).
//   algo 3 (NVLS, large, needs LaunchParams::mc_arena): the same split of the
//     tensor, but the sum of a 16-byte vector over all ranks is one
//     multimem.ld_reduce (the NVSwitch adds the ranks' copies, fp32
//     accumulation) and its broadcast one multimem.st: a rank moves 1/p of the
//     tensor in and 1/p out instead of (p-1)/p each way.
struct AllReduceArgs {
    uint64_t buf_off[kMaxPeers];  // byte offset of the tensor in each rank's arena
    int64_t nelem;
    int32_t dtype;
    int32_t algo, phase;
    int32_t ord, per_iter;    // one-shot: ordinal among the one-shot all_reduces of an iteration, and their count
                              // (consecutive invocations alternate between two staging buffers)
    uint64_t stage_bytes;     // one-shot: bytes of one staging buffer (nranks slots); slots: bytes of one slot
    uint64_t stage_off;       // slots (algo 2): arena offset of this rank's staging slots, filled by the peers' matmul epilogues
    // one-shot: the Add that consumes the sum in the same task, folded into the reduce phase:
    // out := round(sum) + residual, stored to `sum_out` instead of the all_reduce's own tensor
    const void *residual;
    void *sum_out;
    int32_t no_gather;        // slots (algo 2): the sum of this rank's rows stays local (a reduce-scatter); the caller reads
                              // only those rows
    int32_t mc_store;         // two-shot / slots: the result goes out through the multicast address (one store for all ranks)
};

// What a barrier stage does while it waits: L2 prefetch of operands no stage of the plan writes (weights, K/V
// caches) that stages behind the barrier will read. Every CTA of the barrier's range asks for its share.
constexpr int kMaxPrefetch = 6;
struct SyncArgs {
    const void *pf_ptr[kMaxPrefetch];
    uint64_t pf_bytes[kMaxPrefetch];
    int32_t n_pf, pad;
};

struct alignas(128) Stage {
    int32_t kind;
    int32_t proc_b, proc_e, proc_s;  // processor (CTA) range [b, e) step s
    int32_t sync_group;              // SK_SYNC: which barrier counter
    int32_t sync_count;              // SK_SYNC: CTAs taking part
    int32_t sync_ord;                // SK_SYNC: 1-based ordinal of this barrier within an iteration
    int32_t pad0;
    union {
        EwiseArgs ew;
        ReduceArgs rd;
        RowOpArgs ro;
        GemmArgs gm;
        GemvArgs gv;
        DecodeAttnArgs da;
        PrefillAttnArgs pa;
        SplitKReduceArgs sr;
        GemmSimtArgs gs;
        TransposeArgs tp;
        EmbedArgs em;
        PutArgs put;
        WaitArgs wt;
        PeerSyncArgs ps;
        SignalArgs sg;
        AllReduceArgs ar;
        PacketArgs pk;
        PacketReduceArgs pr;
        SyncArgs sy;
    };
};

// Status word written by the device when a bounded wait gives up.
enum StatusCode : int32_t {
    ST_OK = 0,
    ST_BARRIER_TIMEOUT = 1,
    ST_MBAR_TIMEOUT = 2,
    ST_PEER_TIMEOUT = 3,
    ST_IDLE_EXIT = 4,  // loop kernel saw no run request for a long time and returned (not an error)
};

constexpr int kChannels = 64;  // send/recv flag channels per rank pair

struct DeviceState {
    unsigned long long barrier[kMaxSyncGroups];  // monotonic arrive counters (host zeroes them at launch)
    unsigned long long run_seq;                  // run requests published by CTA 0 since launch (zeroed at launch)
    unsigned long long iter_total;               // iterations completed over the executor's life (never reset)
    int32_t status;                              // StatusCode (first failure wins)
    int32_t status_stage;                        // stage index where it happened
    int32_t status_cta;
    int32_t run_iters;                           // iterations requested by the current run (broadcast)
    unsigned long long t_begin, t_end;           // %globaltimer stamps around the last run
    volatile int32_t *host_status;               // host-mapped mirror of `status`
    volatile unsigned long long *host_iters;     // host-mapped mirror of `iter_total`, written before the run flag is cleared
};

// Per-rank communication block, mapped into every peer. It sits at the start
// of each rank's comm allocation; the all_reduce staging area follows it.
struct CommBlock {
    unsigned long long barrier_flag[kMaxPeers];             // [r]: written by rank r
    unsigned long long chan_flag[kMaxPeers * kChannels];    // [src_rank * kChannels + channel]
};
constexpr uint64_t kCommDataOff = 8192;  // staging area offset inside the comm allocation

struct LaunchParams {
    const Stage *stages;
    DeviceState *state;
    volatile int32_t *run_flag;   // host-mapped; >0: run that many iterations; <0: exit
    int32_t n_stages;
    int32_t loop_mode;            // 1: persistent, wait on run_flag; 0: run `iters` once and return
    int32_t iters;
    int32_t rank, nranks;
    int32_t peersyncs_per_iter;
    int32_t pair_mode;            // 1: launched as clusters of 2 CTAs, matmul tiles are 256 rows per CTA pair
    int32_t syncs_per_iter[kMaxSyncGroups];
    char *arena[kMaxPeers];       // arena base of every rank as mapped here (own included)
    char *comm[kMaxPeers];        // comm allocation of every rank as mapped here (own included)
    char *mc_arena;               // NVSwitch multicast address of offset 0 of every rank's arena; null when NVLS is off
    unsigned long long spin_limit;     // nanoseconds a device-side wait may last before it gives up
    unsigned long long idle_limit_ns;  // loop mode: return after this long without a run request
    unsigned long long *stage_times;   // optional [n_stages][grid][2]: when each CTA entered / left each stage of the last iteration (ns)
};

}  // namespace arkb
