// Host runtime of the engine: arena, peer mapping, program upload, the run
// flag protocol and tensor I/O. Stands behind ark::Executor in place of
// Executor::Impl + GpuManager/GpuKernel/GpuMemory + the MSCCL++ set-up
// (ark/api/executor.cpp:226-886, ark/gpu/*).
#include "executor.hpp"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>

#include "loop_kernel.h"

namespace arkb {

#define CUDA_CHECK(expr)                                                                                 \
    do {                                                                                                 \
        cudaError_t _e = (expr);                                                                         \
        if (_e != cudaSuccess)                                                                           \
            throw Error(E_GPU, std::string(#expr) + " failed: " + cudaGetErrorString(_e));               \
    } while (0)

// ---- tensor map encoding ------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e != cudaSuccess || !p) throw Error(E_GPU, "cuTensorMapEncodeTiled is not available from the driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static void encode_tmap_cuda(CUtensorMap *out, const TmapSpec &sp) {
    cuuint64_t dims[5] = {sp.dims[0], sp.dims[1], sp.dims[2], sp.dims[3], sp.dims[4]};
    cuuint64_t strides[4] = {sp.strides_bytes[0], sp.strides_bytes[1], sp.strides_bytes[2], sp.strides_bytes[3]};
    cuuint32_t box[5] = {sp.box[0], sp.box[1], sp.box[2], sp.box[3], sp.box[4]};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    // strides of size-1 dims still have to be valid (multiple of 16, non-zero)
    for (int i = 0; i < sp.rank - 1; ++i)
        if (strides[i] == 0 || strides[i] % 16) strides[i] = ((strides[i] + 15) / 16 + (strides[i] == 0)) * 16;
    CUtensorMapDataType dt = sp.dtype == DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = get_encode_fn()(out, dt, (cuuint32_t)sp.rank, const_cast<void *>(sp.base), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 sp.swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw Error(E_GPU, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
}

// Checks the same constraints without a driver (used by plan checks on hosts with no GPU).
static void encode_tmap_check(CUtensorMap *out, const TmapSpec &sp) {
    std::memset(out, 0, sizeof(*out));
    if (reinterpret_cast<uintptr_t>(sp.base) % 16) throw Error(E_INTERNAL, "tensor map base not 16-byte aligned");
    for (int i = 0; i < sp.rank - 1; ++i)
        if (sp.dims[i + 1] > 1 && sp.strides_bytes[i] % 16) throw Error(E_INTERNAL, "tensor map stride not a multiple of 16");
    for (int i = 0; i < sp.rank; ++i)
        if (sp.box[i] == 0 || sp.box[i] > 256) throw Error(E_INTERNAL, "tensor map box dimension out of range");
}

// ---- Executor --------------------------------------------------------------------------
static const unsigned long long kDefaultSpinLimit = 10ull * 1000000000;  // device-side waits give up after 10 s
static const unsigned long long kDefaultIdleNs = 20ull * 1000000000;  // loop kernel leaves after 20 s without work

Executor::Executor(int device_id, void *stream, const std::string &name, const std::string &plan_json, bool loop_mode,
                   AllgatherFn ag)
    : device_id_(device_id), name_(name), loop_mode_(loop_mode), allgather_(std::move(ag)) {
    if (device_id < 0) throw Error(E_USAGE, "Invalid device ID " + std::to_string(device_id));
    plan_ = Plan::parse(plan_json);
    int ndev = 0;
    CUDA_CHECK(cudaGetDeviceCount(&ndev));
    if (device_id >= ndev) throw Error(E_USAGE, "device ID " + std::to_string(device_id) + " out of range");
    CUDA_CHECK(cudaSetDevice(device_id));
    cudaDeviceProp prop;
    CUDA_CHECK(cudaGetDeviceProperties(&prop, device_id));
    if (prop.major != 10) throw Error(E_UNSUPPORTED, "this engine runs on sm_100 devices only");
    num_sm_ = prop.multiProcessorCount;
    if (plan_.world_size > 1 && !allgather_) throw Error(E_USAGE, "multi-rank plans need a bootstrap allgather callback");
    if (stream) {
        stream_ = reinterpret_cast<cudaStream_t>(stream);
        own_stream_ = false;
    } else {
        CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
        own_stream_ = true;
    }
    CUDA_CHECK(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
    CUDA_CHECK(cudaEventCreate(&ev_start_));
    CUDA_CHECK(cudaEventCreate(&ev_stop_));
    init_memory();
}

Executor::~Executor() {
    try {
        destroy();
    } catch (...) {
    }
}

void Executor::init_memory() {
    layout_ = plan_layout(plan_);
    const int R = plan_.world_size, me = plan_.rank;
    // arena: zero-filled like the reference (ark/gpu/gpu_memory.cpp:75-77); padded regions rely on it
    arena_bytes_ = (layout_.arena_bytes + 65535) / 65536 * 65536;
    // NVLS on request: the arena becomes a symmetric allocation bound to an NVSwitch multicast object (in-switch
    // reduction and one-store broadcast for the large all_reduce). Every rank takes the same decision: the set-up
    // is collective and fails on all ranks or on none; on failure the plain arena below is used.
    if (R > 1) {
        const char *e = getenv("ARKB_NVLS");
        if (e && atoi(e) != 0) {
            try {
                CUDA_CHECK(cudaFree(nullptr));  // the device's context exists before driver calls are made
                symm_.create(device_id_, me, R, arena_bytes_, allgather_);
                arena_ = symm_.local();
                arena_bytes_ = symm_.bytes();
            } catch (const Error &err) {
                fprintf(stderr, "ark_b200: NVLS not used (%s)\n", err.what());
            }
        }
    }
    if (!symm_.active()) {
        CUDA_CHECK(cudaMalloc(&arena_, arena_bytes_));
        CUDA_CHECK(cudaMemset(arena_, 0, arena_bytes_));
    }
    comm_bytes_ = kCommDataOff + 2 * layout_.comm_stage_bytes + 256;
    CUDA_CHECK(cudaMalloc(&comm_, comm_bytes_));
    CUDA_CHECK(cudaMemset(comm_, 0, comm_bytes_));
    CUDA_CHECK(cudaMalloc(&state_, sizeof(DeviceState)));
    CUDA_CHECK(cudaMemset(state_, 0, sizeof(DeviceState)));
    CUDA_CHECK(cudaHostAlloc(&host_flags_, 4 * sizeof(int32_t), cudaHostAllocMapped));
    host_flags_[0] = 0;  // run flag
    host_flags_[1] = 0;  // status mirror
    host_flags_[2] = host_flags_[3] = 0;  // iterations finished (64 bits)
    int32_t *dflags = nullptr;
    CUDA_CHECK(cudaHostGetDevicePointer(&dflags, host_flags_, 0));
    dev_flags_ = dflags;
    DeviceState init;
    std::memset(&init, 0, sizeof(init));
    init.host_status = dflags + 1;
    init.host_iters = reinterpret_cast<volatile unsigned long long *>(dflags + 2);
    CUDA_CHECK(cudaMemcpy(state_, &init, sizeof(init), cudaMemcpyHostToDevice));
    for (int r = 0; r < kMaxPeers; ++r) peer_arena_[r] = peer_comm_[r] = nullptr;
    peer_arena_[me] = reinterpret_cast<char *>(arena_);
    peer_comm_[me] = reinterpret_cast<char *>(comm_);
    if (R > 1) {
        // exchange tag records, then IPC handles (replaces the bootstrap send/recv of
        // ark/api/executor.cpp:410-500 and registerMemory/connect of :532-623)
        const size_t kMaxRec = 4096;
        if (layout_.published.size() > kMaxRec) throw Error(E_UNSUPPORTED, "too many tagged buffers");
        struct Blob {
            uint64_t n;
            TagRecord rec[kMaxRec];
        };
        std::vector<Blob> all(R);
        Blob *mine = new Blob();
        mine->n = layout_.published.size();
        std::memcpy(mine->rec, layout_.published.data(), mine->n * sizeof(TagRecord));
        int rc = allgather_(mine, all.data(), sizeof(Blob));
        delete mine;
        if (rc != 0) throw Error(E_SYSTEM, "bootstrap allgather failed");
        std::vector<std::vector<TagRecord>> records(R);
        for (int r = 0; r < R; ++r) records[r].assign(all[r].rec, all[r].rec + all[r].n);
        resolve_remote(plan_, layout_, records);
        struct Handles {
            cudaIpcMemHandle_t arena, comm;
            uint64_t arena_bytes;
        };
        Handles h;
        std::memset(&h, 0, sizeof(h));
        if (!symm_.active()) CUDA_CHECK(cudaIpcGetMemHandle(&h.arena, arena_));
        CUDA_CHECK(cudaIpcGetMemHandle(&h.comm, comm_));
        h.arena_bytes = arena_bytes_;
        std::vector<Handles> hs(R);
        if (allgather_(&h, hs.data(), sizeof(Handles)) != 0) throw Error(E_SYSTEM, "bootstrap allgather failed");
        for (int r = 0; r < R; ++r) {
            if (r == me) continue;
            void *pa = nullptr, *pc = nullptr;
            if (symm_.active()) pa = symm_.peer(r);
            else CUDA_CHECK(cudaIpcOpenMemHandle(&pa, hs[r].arena, cudaIpcMemLazyEnablePeerAccess));
            CUDA_CHECK(cudaIpcOpenMemHandle(&pc, hs[r].comm, cudaIpcMemLazyEnablePeerAccess));
            peer_arena_[r] = reinterpret_cast<char *>(pa);
            peer_comm_[r] = reinterpret_cast<char *>(pc);
        }
    } else {
        std::vector<std::vector<TagRecord>> records(1, layout_.published);
        resolve_remote(plan_, layout_, records);
    }
}

void Executor::compile() {
    if (compiled_) return;
    CUDA_CHECK(cudaSetDevice(device_id_));
    LowerEnv env;
    env.rank = plan_.rank;
    env.nranks = plan_.world_size;
    for (int r = 0; r < kMaxPeers; ++r) {
        env.arena[r] = peer_arena_[r];
        env.comm[r] = peer_comm_[r];
    }
    env.encode_tmap = encode_tmap_cuda;
    env.mc_arena = symm_.active() ? symm_.multicast() : nullptr;
    env.num_sm = num_sm_;
    env.allow_pair = getenv("ARKB_NO_PAIR") == nullptr;
    // first pass sizes the scratch (split-K partials) against a stand-in address, second pass uses the real one
    env.workspace = reinterpret_cast<char *>((uintptr_t)1 << 44);
    program_ = lower_plan(plan_, layout_, env);
    if (program_.workspace_bytes > 0) {
        CUDA_CHECK(cudaMalloc(&workspace_, program_.workspace_bytes));
        env.workspace = reinterpret_cast<char *>(workspace_);
        program_ = lower_plan(plan_, layout_, env);
    }
    if (!program_.stages.empty()) {
        CUDA_CHECK(cudaMalloc(&stages_dev_, program_.stages.size() * sizeof(Stage)));
        CUDA_CHECK(cudaMemcpy(stages_dev_, program_.stages.data(), program_.stages.size() * sizeof(Stage),
                              cudaMemcpyHostToDevice));
    }
    CUDA_CHECK(loop_kernel_prepare());
    compiled_ = true;
}

void Executor::fill_params(LaunchParams &P, int iters) const {
    std::memset(&P, 0, sizeof(P));
    P.stages = reinterpret_cast<const Stage *>(stages_dev_);
    P.state = reinterpret_cast<DeviceState *>(state_);
    P.run_flag = dev_flags_;
    P.n_stages = (int32_t)program_.stages.size();
    P.loop_mode = loop_mode_ ? 1 : 0;
    P.iters = iters;
    P.rank = plan_.rank;
    P.nranks = plan_.world_size;
    P.peersyncs_per_iter = program_.peersyncs_per_iter;
    P.pair_mode = program_.pair_mode ? 1 : 0;
    for (int i = 0; i < kMaxSyncGroups; ++i) P.syncs_per_iter[i] = program_.syncs_per_iter[i];
    for (int r = 0; r < kMaxPeers; ++r) {
        P.arena[r] = peer_arena_[r];
        P.comm[r] = peer_comm_[r];
    }
    P.mc_arena = symm_.active() ? symm_.multicast() : nullptr;
    P.spin_limit = spin_limit_ ? spin_limit_ : kDefaultSpinLimit;
    // serialised launches: the kernel serves the request that is already posted and leaves at once
    P.idle_limit_ns = blocking_launch_ ? 0 : (idle_limit_ ? idle_limit_ : kDefaultIdleNs);
    P.stage_times = stage_times_on_ ? stage_times_ : nullptr;
}

void Executor::enable_stage_times(bool on) {
    if (kernel_live_) throw Error(E_USAGE, "stage times are switched before launch");
    if (on && !compiled_) throw Error(E_USAGE, "Need to compile first.");
    if (on && !stage_times_ && !program_.stages.empty()) {
        const size_t bytes = program_.stages.size() * (size_t)program_.grid * 2 * sizeof(unsigned long long);
        CUDA_CHECK(cudaSetDevice(device_id_));
        CUDA_CHECK(cudaMalloc(&stage_times_, bytes));
        CUDA_CHECK(cudaMemset(stage_times_, 0, bytes));
    }
    stage_times_on_ = on && stage_times_;
}

size_t Executor::read_stage_times(unsigned long long *out, size_t capacity, int *n_stages, int *grid) {
    if (n_stages) *n_stages = (int)program_.stages.size();
    if (grid) *grid = program_.grid;
    if (!stage_times_on_ || !out) return 0;
    if (kernel_live_ && pending_) throw Error(E_USAGE, "wait() before reading stage times");
    const size_t words = std::min(capacity, program_.stages.size() * (size_t)program_.grid * 2);
    CUDA_CHECK(cudaMemcpyAsync(out, stage_times_, words * sizeof(unsigned long long), cudaMemcpyDeviceToHost, copy_stream_));
    CUDA_CHECK(cudaStreamSynchronize(copy_stream_));
    return words;
}

void Executor::launch_kernel(int iters) {
    // barrier counters restart at every launch; iter_total and the status persist
    CUDA_CHECK(cudaMemsetAsync(state_, 0, sizeof(unsigned long long) * (kMaxSyncGroups + 1), stream_));  // barrier[] and run_seq
    LaunchParams P;
    fill_params(P, iters);
    CUDA_CHECK(loop_kernel_launch(P, program_.grid, stream_, program_.smem_bytes));
    ++n_launches_;
}

bool Executor::stream_idle() {
    const cudaError_t q = cudaStreamQuery(stream_);
    if (q == cudaSuccess) return true;
    if (q != cudaErrorNotReady) throw Error(E_GPU, std::string("loop kernel failed: ") + cudaGetErrorString(q));
    return false;
}

// Finds out whether kernel launches return before the kernel ends. An empty loop kernel that leaves after 2 ms
// without work is launched: with ordinary launches it is still running when the call returns (it is then told to
// leave through the run flag); with serialised launches (CUDA_LAUNCH_BLOCKING=1, a profiler attached) it has
// already ended, and a resident kernel that waits for the host could never be served by it.
void Executor::probe_blocking_launch() {
    if (probed_) return;
    probed_ = true;
    host_flags_[0] = 0;
    CUDA_CHECK(cudaMemsetAsync(state_, 0, sizeof(unsigned long long) * (kMaxSyncGroups + 1), stream_));
    LaunchParams P;
    fill_params(P, 0);
    P.n_stages = 0;
    P.loop_mode = 1;
    P.idle_limit_ns = 2ull * 1000000;
    P.stage_times = nullptr;
    CUDA_CHECK(loop_kernel_launch(P, program_.grid, stream_, program_.smem_bytes));
    blocking_launch_ = stream_idle();
    if (!blocking_launch_) {
        *reinterpret_cast<volatile int32_t *>(&host_flags_[0]) = -1;
        CUDA_CHECK(cudaStreamSynchronize(stream_));
    }
    host_flags_[0] = 0;
    host_flags_[1] = 0;
    CUDA_CHECK(cudaMemsetAsync(reinterpret_cast<char *>(state_) + offsetof(DeviceState, status), 0, sizeof(int32_t), stream_));
    CUDA_CHECK(cudaStreamSynchronize(stream_));
}

// Starts the resident kernel again after it left (idle exit). A posted run request stays posted: the new kernel
// finds it in the run flag.
void Executor::relaunch_loop_kernel() {
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    host_flags_[1] = 0;
    CUDA_CHECK(cudaMemsetAsync(reinterpret_cast<char *>(state_) + offsetof(DeviceState, status), 0, sizeof(int32_t), stream_));
    launch_kernel(0);
    kernel_live_ = !blocking_launch_;
}

void Executor::launch() {
    if (!compiled_) throw Error(E_USAGE, "Need to compile first before launch.");
    if (launched_) return;  // the reference ignores a second launch with a warning (api/executor_test.cpp:149-155)
    CUDA_CHECK(cudaSetDevice(device_id_));
    elapsed_ms_ = -1;
    if (loop_mode_) probe_blocking_launch();
    CUDA_CHECK(cudaEventRecord(ev_start_, stream_));
    if (loop_mode_) {
        host_flags_[0] = 0;
        if (!blocking_launch_) {
            launch_kernel(0);
            kernel_live_ = true;
        }
    }
    launched_ = true;
    stopped_ = false;
}

void Executor::check_status() {
    const int32_t st = *reinterpret_cast<volatile int32_t *>(&host_flags_[1]);
    if (st != ST_OK && st != ST_IDLE_EXIT) {
        arkb_status_snapshot snap = status();
        iters_expected_ = snap.iterations;  // what did run; later requests count from here
        throw Error(E_GPU, "loop kernel gave up: status " + std::to_string(snap.code) + " at stage " +
                               std::to_string(snap.stage) + " (CTA " + std::to_string(snap.cta) + ")");
    }
}

void Executor::run(int iter) {
    if (!launched_ || stopped_) throw Error(E_USAGE, "Need to launch before run.");
    if (iter <= 0) return;
    CUDA_CHECK(cudaSetDevice(device_id_));
    if (loop_mode_) {
        // the previous request must have been consumed (ark/api/executor.cpp:698-704)
        if (pending_) wait(-1);
        check_status();
        volatile int32_t *flag = host_flags_;
        // The request is posted before anything else: a kernel started from here on finds it, and a resident
        // kernel that leaves (idle exit) at this very moment is noticed by wait(), which starts it again.
        iters_expected_ += (unsigned long long)iter;
        pending_ = true;
        *flag = iter;
        if (blocking_launch_) {
            relaunch_loop_kernel();  // returns when the request is done and the kernel has left again
        } else if (!kernel_live_ || stream_idle()) {
            relaunch_loop_kernel();
        }
    } else {
        iters_expected_ += (unsigned long long)iter;
        pending_ = true;
        launch_kernel(iter);
    }
}

void Executor::wait(int64_t max_spin_count) {
    if (!pending_) return;
    CUDA_CHECK(cudaSetDevice(device_id_));
    if (loop_mode_) {
        volatile int32_t *flag = host_flags_;
        int64_t spins = 0;
        int relaunches = 0;
        const int64_t every = max_spin_count >= 0 ? std::max<int64_t>(max_spin_count, 1) : 0x100000;
        while (*flag > 0) {
            if (++spins < every) continue;
            spins = 0;
            if (!stream_idle()) continue;
            if (*flag <= 0) break;  // finished between the two looks
            // The kernel is gone and the request is still posted. Either a bounded wait gave up (the status says
            // so), or the kernel left for lack of work just before the request arrived: start it again, twice at most.
            kernel_live_ = false;
            const int32_t st = *reinterpret_cast<volatile int32_t *>(&host_flags_[1]);
            if (st != ST_OK && st != ST_IDLE_EXIT) break;
            if (relaunches++ >= 2) {
                *flag = 0;
                pending_ = false;
                iters_expected_ = *reinterpret_cast<volatile unsigned long long *>(&host_flags_[2]);
                throw Error(E_GPU, "run request was not picked up by the loop kernel (relaunched twice)");
            }
            relaunch_loop_kernel();
        }
    } else {
        CUDA_CHECK(cudaStreamSynchronize(stream_));
    }
    pending_ = false;
    if (*reinterpret_cast<volatile int32_t *>(&host_flags_[0]) > 0) host_flags_[0] = 0;  // abort path: withdraw the request
    check_status();
    // never report success for iterations that did not run
    const unsigned long long done = *reinterpret_cast<volatile unsigned long long *>(&host_flags_[2]);
    if (done != iters_expected_) {
        const unsigned long long want = iters_expected_;
        iters_expected_ = done;
        throw Error(E_GPU, "loop kernel finished " + std::to_string(done) + " iterations, " + std::to_string(want) + " were requested");
    }
}

float Executor::stop(int64_t max_spin_count) {
    if (!launched_ || stopped_) return elapsed_ms_ < 0 ? 0.0f : elapsed_ms_;
    CUDA_CHECK(cudaSetDevice(device_id_));
    std::string err;
    try {
        wait(max_spin_count);
    } catch (const Error &e) {
        err = e.what();
    }
    if (loop_mode_ && kernel_live_) {
        *reinterpret_cast<volatile int32_t *>(&host_flags_[0]) = -1;
    }
    CUDA_CHECK(cudaEventRecord(ev_stop_, stream_));
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    kernel_live_ = false;
    host_flags_[0] = 0;
    if (host_flags_[1] == ST_IDLE_EXIT) host_flags_[1] = 0;
    CUDA_CHECK(cudaEventElapsedTime(&elapsed_ms_, ev_start_, ev_stop_));
    stopped_ = true;
    launched_ = false;
    if (!err.empty()) throw Error(E_GPU, err);
    return elapsed_ms_;
}

void Executor::barrier() {
    if (plan_.world_size <= 1) return;
    std::vector<int> all(plan_.world_size);
    int mine = plan_.rank;
    if (allgather_(&mine, all.data(), sizeof(int)) != 0) throw Error(E_SYSTEM, "bootstrap allgather failed");
}

void Executor::destroy() {
    if (destroyed_) return;
    cudaSetDevice(device_id_);
    if (launched_ && !stopped_) {
        try {
            stop(-1);
        } catch (...) {
        }
    }
    for (int r = 0; r < kMaxPeers; ++r) {
        if (r == plan_.rank) continue;
        if (peer_arena_[r] && !symm_.active()) cudaIpcCloseMemHandle(peer_arena_[r]);
        if (peer_comm_[r]) cudaIpcCloseMemHandle(peer_comm_[r]);
        peer_arena_[r] = peer_comm_[r] = nullptr;
    }
    if (stages_dev_) cudaFree(stages_dev_);
    if (workspace_) cudaFree(workspace_);
    workspace_ = nullptr;
    if (stage_times_) cudaFree(stage_times_);
    stage_times_ = nullptr;
    if (symm_.active()) symm_.destroy(allgather_);  // collective: no rank unbinds while another may still use the multicast address
    else if (arena_) cudaFree(arena_);
    if (comm_) cudaFree(comm_);
    if (state_) cudaFree(state_);
    if (host_flags_) cudaFreeHost(host_flags_);
    if (ev_start_) cudaEventDestroy(ev_start_);
    if (ev_stop_) cudaEventDestroy(ev_stop_);
    if (copy_stream_) cudaStreamDestroy(copy_stream_);
    if (own_stream_ && stream_) cudaStreamDestroy(stream_);
    stages_dev_ = arena_ = comm_ = state_ = nullptr;
    host_flags_ = nullptr;
    destroyed_ = true;
}

arkb_status_snapshot Executor::status() {
    arkb_status_snapshot s;
    std::memset(&s, 0, sizeof(s));
    DeviceState ds;
    cudaSetDevice(device_id_);
    CUDA_CHECK(cudaMemcpyAsync(&ds, state_, sizeof(ds), cudaMemcpyDeviceToHost, copy_stream_));
    CUDA_CHECK(cudaStreamSynchronize(copy_stream_));
    s.code = ds.status;
    s.stage = ds.status_stage;
    s.cta = ds.status_cta;
    s.n_stages = (int)program_.stages.size();
    s.n_launches = n_launches_;
    s.iterations = ds.iter_total;
    s.last_run_ns = ds.t_end > ds.t_begin ? ds.t_end - ds.t_begin : 0;
    return s;
}

// ---- tensor I/O ----------------------------------------------------------------------------
char *Executor::tensor_base(const TensorDesc &t) const {
    auto it = layout_.buffers.find(t.buffer_id);
    if (it == layout_.buffers.end()) throw Error(E_USAGE, "tensor's buffer is not part of the plan");
    const BufferInfo &b = it->second;
    if (b.rank != -1 && b.rank != plan_.rank) throw Error(E_USAGE, "tensor lives on another rank");
    int64_t es[4], org;
    t.elem_strides(es, org);
    return reinterpret_cast<char *>(arena_) + b.offset + (size_t)org * dtype_size(t.dtype);
}

uintptr_t Executor::tensor_address(const std::string &tensor_json) const {
    TensorDesc t = TensorDesc::from_json(Json::parse(tensor_json));
    return reinterpret_cast<uintptr_t>(tensor_base(t));
}

void Executor::tensor_io(const std::string &tensor_json, void *data, size_t bytes, void *stream, bool is_d2d, bool write) {
    TensorDesc t = TensorDesc::from_json(Json::parse(tensor_json));
    const size_t es = dtype_size(t.dtype);
    const size_t want = (size_t)t.nelems() * es;
    if (bytes != want)  // same check as the reference (api/executor_test.cpp:171-183)
        throw Error(E_USAGE, "Destination bytes (" + std::to_string(bytes) + ") mismatches the tensor data bytes (" + std::to_string(want) + ").");
    CUDA_CHECK(cudaSetDevice(device_id_));
    cudaStream_t cs = stream ? reinterpret_cast<cudaStream_t>(stream) : copy_stream_;
    char *base = tensor_base(t);
    const cudaMemcpyKind kind = is_d2d ? cudaMemcpyDeviceToDevice : (write ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost);
    if (t.dense()) {
        if (write) CUDA_CHECK(cudaMemcpyAsync(base, data, bytes, kind, cs));
        else CUDA_CHECK(cudaMemcpyAsync(data, base, bytes, kind, cs));
        CUDA_CHECK(cudaStreamSynchronize(cs));
        return;
    }
    // strided view: one 2-D copy per (n, c) slab; rows are `W` elements long, `ld` apart
    auto sh = t.shape4();
    int64_t est[4], org;
    t.elem_strides(est, org);
    const size_t row = (size_t)sh[3] * es;
    char *host = reinterpret_cast<char *>(data);
    for (int64_t n = 0; n < sh[0]; ++n)
        for (int64_t c = 0; c < sh[1]; ++c) {
            char *dev = base + (size_t)(n * est[0] + c * est[1]) * es;
            char *h = host + (size_t)((n * sh[1] + c) * sh[2]) * row;
            if (write) CUDA_CHECK(cudaMemcpy2DAsync(dev, (size_t)est[2] * es, h, row, row, (size_t)sh[2], kind, cs));
            else CUDA_CHECK(cudaMemcpy2DAsync(h, row, dev, (size_t)est[2] * es, row, (size_t)sh[2], kind, cs));
        }
    CUDA_CHECK(cudaStreamSynchronize(cs));
}

// ---- plan check without a GPU ----------------------------------------------------------------
void plan_check(const std::string &plan_json, int *n_stages, size_t *arena_bytes, int *n_processors) {
    Plan plan = Plan::parse(plan_json);
    Layout lay = plan_layout(plan);
    // stand-in addresses: 1 TiB apart, aligned like cudaMalloc
    LowerEnv env;
    env.rank = plan.rank;
    env.nranks = plan.world_size;
    for (int r = 0; r < plan.world_size; ++r) {
        env.arena[r] = reinterpret_cast<char *>((uintptr_t)(r + 1) << 40);
        env.comm[r] = reinterpret_cast<char *>(((uintptr_t)(r + 1) << 40) + ((uintptr_t)1 << 39));
    }
    env.encode_tmap = encode_tmap_check;
    env.num_sm = kDefaultNumSm;  // no device to ask
    env.workspace = reinterpret_cast<char *>((uintptr_t)1 << 44);
    // every rank is assumed to publish the same records as this one (SPMD plans)
    std::vector<std::vector<TagRecord>> records(plan.world_size, lay.published);
    for (auto &kv : lay.buffers) {
        BufferInfo &b = kv.second;
        if (!b.resolved) {  // remote stand-ins: any aligned offset serves for checking
            b.offset = 0;
            b.resolved = true;
        }
    }
    resolve_remote(plan, lay, records);
    Program prog = lower_plan(plan, lay, env);
    if (n_stages) *n_stages = (int)prog.stages.size();
    if (arena_bytes) *arena_bytes = lay.arena_bytes;
    if (n_processors) *n_processors = prog.grid;
}

std::string plan_dump(const std::string &plan_json) {
    Plan plan = Plan::parse(plan_json);
    Layout lay = plan_layout(plan);
    LowerEnv env;
    env.rank = plan.rank;
    env.nranks = plan.world_size;
    for (int r = 0; r < plan.world_size; ++r) {
        env.arena[r] = reinterpret_cast<char *>((uintptr_t)(r + 1) << 40);
        env.comm[r] = reinterpret_cast<char *>(((uintptr_t)(r + 1) << 40) + ((uintptr_t)1 << 39));
    }
    env.encode_tmap = encode_tmap_check;
    env.allow_pair = getenv("ARKB_NO_PAIR") == nullptr;  // the same switches as the executor's lowering
    env.workspace = reinterpret_cast<char *>((uintptr_t)1 << 44);
    std::vector<std::vector<TagRecord>> records(plan.world_size, lay.published);
    for (auto &kv : lay.buffers)
        if (!kv.second.resolved) {
            kv.second.offset = 0;
            kv.second.resolved = true;
        }
    resolve_remote(plan, lay, records);
    std::string text = lower_plan(plan, lay, env).dump();
    text += "arena=" + std::to_string(lay.arena_bytes) + " bytes";
    if (plan.arena_reuse)
        text += " (" + std::to_string(lay.reused_buffers) + " intermediates share space by lifetime; " +
                std::to_string(lay.arena_bytes_no_reuse) + " bytes without reuse)";
    return text + "\n";
}

void device_info(int device_id, DeviceInfo &out) {
    int ndev = 0;
    CUDA_CHECK(cudaGetDeviceCount(&ndev));
    if (device_id < 0 || device_id >= ndev) throw Error(E_USAGE, "Invalid device ID " + std::to_string(device_id));
    cudaDeviceProp p;
    CUDA_CHECK(cudaGetDeviceProperties(&p, device_id));
    out.cc_major = p.major;
    out.cc_minor = p.minor;
    out.num_sm = p.multiProcessorCount;
    out.max_threads_per_block = p.maxThreadsPerBlock;
    out.smem_per_block_optin = (int)p.sharedMemPerBlockOptin;
    out.regs_per_sm = p.regsPerMultiprocessor;
    out.total_mem = p.totalGlobalMem;
    out.arch = "CUDA_" + std::to_string(p.major * 10 + p.minor);
    out.name = p.name;
}

}  // namespace arkb
