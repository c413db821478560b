// Host-side representation of an ARK plan and of the lowered stage program.
#pragma once
#include <cstdint>
#include <functional>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.hpp"
#include "program.h"

namespace arkb {

// Error carrying the status class the C ABI reports (mirrors the reference's
// exception hierarchy, ark/include/ark/error.hpp:13-43).
struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};
enum { E_INTERNAL = 1, E_USAGE = 2, E_MODEL = 3, E_PLAN = 4, E_UNSUPPORTED = 5, E_SYSTEM = 6, E_GPU = 7 };

int dtype_from_name(const std::string &n);  // "FP16" -> DT_F16 ...
size_t dtype_size(int dt);

struct TensorDesc {
    int64_t id = -1;
    int dtype = DT_F32;
    std::vector<int64_t> shape, strides, offsets, padded;
    int64_t buffer_id = -1;
    int buffer_rank = -1;
    std::vector<std::pair<int, int>> send_tags, recv_tags;  // (rank, tag)

    static TensorDesc from_json(const Json &j);
    int64_t nelems() const;
    int64_t stride_bytes() const;  // bytes of the buffer this view needs (ark/api/executor.cpp:135-139)
    std::vector<int64_t> shape4() const;
    std::vector<int64_t> strides4() const;
    std::vector<int64_t> offsets4() const;
    // element strides of the 4-D view and the element offset of its origin
    void elem_strides(int64_t (&es)[4], int64_t &origin) const;
    bool dense() const;
};

struct Range {
    int64_t b = 0, e = 0, s = 1;
    int64_t count() const { return e > b ? (e - b + s - 1) / s : 0; }
    static Range from_json(const Json &j);
    bool overlaps(const Range &o) const;
    bool operator==(const Range &o) const { return b == o.b && e == o.e && s == o.s; }
};

struct OpDesc {
    std::string type, name;
    bool is_virtual = false;
    std::vector<TensorDesc> reads, writes, results;
    Json args, config;
    int64_t arg_int(const std::string &k) const;
    double arg_float(const std::string &k) const;
    bool arg_bool(const std::string &k) const;
    std::vector<int64_t> arg_dims(const std::string &k) const;
    bool has_arg(const std::string &k) const { return args.is_object() && args.contains(k); }
};

struct TaskInfo {
    int64_t id = 0;
    int num_warps = 1, sram_bytes = 0;
    std::vector<OpDesc> ops;
};
struct TaskGroup {
    int64_t task_id = 0;
    Range task_range;
    int64_t granularity = 1;
};
struct ResourceGroup {
    Range proc, warp, sram;
    std::vector<TaskGroup> task_groups;
};
struct ProcessorGroup {
    Range proc;
    std::vector<ResourceGroup> resource_groups;
};

struct Plan {
    int rank = 0, world_size = 1;
    std::string architecture;
    int num_processors = 1, num_warps_per_processor = 1;
    bool arena_reuse = false;  // optional top-level plan field "ArenaReuse": intermediates with disjoint lifetimes share memory
    std::vector<TaskInfo> task_infos;
    std::vector<ProcessorGroup> processor_groups;
    static Plan parse(const std::string &text);
    const TaskInfo &task(int64_t id) const;
};

// ---- buffer layout -------------------------------------------------------------------
struct BufferInfo {
    int64_t id;
    int rank;  // -1 or own rank: local
    size_t bytes = 0;
    size_t offset = 0;  // arena offset on the owning rank
    bool resolved = false;
    std::vector<std::pair<int, int>> send_tags, recv_tags;
};

// One record a rank publishes so peers can resolve their remote buffers:
// kind 0 = send tag, 1 = recv tag, 2 = collective tag, 3 = staging slots of a fused collective.
struct TagRecord {
    int32_t kind, peer, tag, pad;
    uint64_t offset;
};

struct Layout {
    std::map<int64_t, BufferInfo> buffers;
    size_t arena_bytes = 0;
    size_t arena_bytes_no_reuse = 0;  // what the bump allocation of the reference would take (no lifetime reuse)
    int reused_buffers = 0;           // intermediates placed by the lifetime planner
    size_t comm_stage_bytes = 0;  // bytes of ONE one-shot staging buffer (kMaxPeers slots)
    std::vector<TagRecord> published;  // this rank's records
    // collective tag -> arena offset on every rank
    std::map<int, std::vector<uint64_t>> coll_offsets;
    // collective tag -> arena offset, on every rank, of the staging slots of an all_reduce fused into the Matmul before it
    std::map<int, std::vector<uint64_t>> coll_stage_offsets;
};

constexpr size_t kArenaAlign = 256;  // buffer alignment inside the arena

// True when ops[i] of `ti` is a Matmul and ops[i+1] the AllReduce (same task, i.e. planned with Sync=false) that sums
// the Matmul's result in place, in a shape the engine fuses: the Matmul's epilogue stores its tiles into staging
// slots on the rank that sums them. Needs a dense [M, N] fp16/bf16 result with M a multiple of 256 * world size.
bool fused_allreduce(const Plan &plan, const TaskInfo &ti, size_t i);

// Walks the plan, sizes every buffer and bump-allocates the local ones.
// Counterpart of Executor::Impl::init_buffers (ark/api/executor.cpp:300-408),
// with offsets rounded up to kArenaAlign so that TMA and 128-bit accesses
// can be used on every buffer. With Plan::arena_reuse (what the reference leaves
// as "TODO: improve memory planning", api/executor.cpp:374) intermediates whose
// lifetimes do not overlap share arena space: a buffer qualifies when every tensor
// on it is a dense whole-buffer view, it carries no tags and no communication
// operator touches it, some op writes it before any op reads it, and some op reads
// it (inputs, outputs and everything the host may feed or fetch keep their own
// space). Lifetimes are counted in processor groups, the unit the plan orders.
Layout plan_layout(const Plan &plan);
// Resolves remote buffers and collective offsets from the records of all
// ranks (records[r] = what rank r published). Counterpart of the tag/offset
// exchange at ark/api/executor.cpp:410-500.
void resolve_remote(const Plan &plan, Layout &lay, const std::vector<std::vector<TagRecord>> &records);

// ---- lowering ---------------------------------------------------------------------------
struct TmapSpec {
    const void *base;
    int dtype;
    int rank = 4;               // 4, or 5 for the k-block-grouped view {64, rows, K/64, C, N}
    uint64_t dims[5] = {1, 1, 1, 1, 1};
    uint64_t strides_bytes[4] = {0, 0, 0, 0};  // strides of dims 1..rank-1
    uint32_t box[5] = {1, 1, 1, 1, 1};
    int swizzle_bytes = 128;  // 128 or 64
};
// Encodes a 128-byte-swizzled tiled tensor map; throws on failure.
using TmapEncoder = std::function<void(CUtensorMap *out, const TmapSpec &spec)>;

constexpr int kDefaultNumSm = 148;  // SMs of a B200: what plan checks assume on a host with no device to ask

struct LowerEnv {
    int rank = 0, nranks = 1;
    char *arena[kMaxPeers] = {};  // arena base of every rank in this process's address space
    char *comm[kMaxPeers] = {};
    char *mc_arena = nullptr;     // multicast address of the arenas when they are bound to an NVSwitch multicast object
    TmapEncoder encode_tmap;
    int num_sm = kDefaultNumSm;
    bool allow_pair = true;  // let matmul tiles span CTA pairs (tcgen05 cta_group::2) when the plan permits
    char *workspace = nullptr;  // scratch for split-K partials (sized by a first lowering pass: Program::workspace_bytes)
};

// What a stage reads and writes (address ranges in this process's mappings), for the pass that drops barriers no
// data dependency needs. `opaque` stages (communication) are taken to depend on everything.
struct StageAccess {
    std::vector<std::pair<uintptr_t, uintptr_t>> reads, writes;  // [begin, end)
    bool opaque = true;
    // > 0: a flat elementwise walk in which thread t handles the same `aligned_units` units of `aligned_unit_bytes`
    // bytes of every operand: two such stages over the same CTAs touch a common operand thread by thread
    int64_t aligned_units = 0;
    int aligned_unit_bytes = 0;
    // != 0: a tiled matmul whose output tiles (and epilogue operand) are touched tile by tile with this tile -> CTA
    // mapping; `tiled` lists those operands. Two such stages with one signature over the same CTAs hand a common
    // operand from a CTA to itself.
    uint64_t tile_sig = 0;
    std::vector<std::pair<uintptr_t, uintptr_t>> tiled;
    // large operands the stage streams from HBM (weights, caches): candidates for L2 prefetch at an earlier barrier
    struct Streamed {
        const void *ptr;
        size_t bytes;
        int64_t buffer_id;
    };
    std::vector<Streamed> streamed;
};

struct Program {
    std::vector<Stage> stages;
    std::vector<StageAccess> access;  // parallel to `stages`
    std::vector<std::string> notes;  // one line per stage, for dumps and tests
    int grid = 1;
    int n_sync_groups = 0;
    int syncs_per_iter[kMaxSyncGroups] = {};
    int peersyncs_per_iter = 0;
    int oneshots_per_iter = 0;
    int syncs_elided = 0;  // barriers of the straightforward lowering that the dependency pass removed
    size_t smem_bytes = 0;  // dynamic shared memory the stages of this program need (the launch asks for no more: what is
                            // left of the SM's 256 KiB serves as L1, where the stage functions' stack frames then stay)
    size_t prefetch_bytes = 0;  // bytes per iteration that barrier stages ask the L2 to fetch ahead of their readers
    size_t workspace_bytes = 0;  // scratch the program needs beyond the arena (split-K partials)
    bool pair_mode = false;  // launch clusters of 2 CTAs; matmul tiles are 256 x tile_n per pair
    std::string dump() const;
};

Program lower_plan(const Plan &plan, const Layout &lay, const LowerEnv &env);

}  // namespace arkb
