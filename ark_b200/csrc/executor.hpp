// Host runtime class behind the C ABI (see include/ark_b200.h).
#pragma once
#include <cuda_runtime.h>

#include <functional>
#include <string>

#include "plan.hpp"
#include "symm_arena.hpp"

namespace arkb {

struct arkb_status_snapshot {
    int code, stage, cta, n_stages, n_launches;
    uint64_t iterations, last_run_ns;
};

struct DeviceInfo {
    int cc_major, cc_minor, num_sm, max_threads_per_block, smem_per_block_optin, regs_per_sm;
    size_t total_mem;
    std::string arch, name;
};

using AllgatherFn = std::function<int(const void *send, void *recv, size_t bytes)>;

class Executor {
   public:
    Executor(int device_id, void *stream, const std::string &name, const std::string &plan_json, bool loop_mode,
             AllgatherFn allgather);
    ~Executor();
    void compile();
    void launch();
    void run(int iter);
    void wait(int64_t max_spin_count);
    float stop(int64_t max_spin_count);
    void barrier();
    void destroy();
    uintptr_t tensor_address(const std::string &tensor_json) const;
    void tensor_io(const std::string &tensor_json, void *data, size_t bytes, void *stream, bool is_d2d, bool write);
    arkb_status_snapshot status();
    void *stream() const { return stream_; }
    const Program &program() const { return program_; }
    void set_spin_limit(unsigned long long v) { spin_limit_ = v; }
    void set_idle_limit(unsigned long long v) { idle_limit_ = v; }
    void enable_stage_times(bool on);
    // copies the [n_stages][grid][2] time stamps of the last iteration; returns the number of words written
    size_t read_stage_times(unsigned long long *out, size_t capacity, int *n_stages, int *grid);
    std::string dump_text;

   private:
    void init_memory();
    void fill_params(LaunchParams &P, int iters) const;
    void launch_kernel(int iters);
    void relaunch_loop_kernel();
    void probe_blocking_launch();
    void check_status();
    bool stream_idle();
    char *tensor_base(const TensorDesc &t) const;

    int device_id_;
    std::string name_;
    bool loop_mode_;
    AllgatherFn allgather_;
    Plan plan_;
    Layout layout_;
    Program program_;
    int num_sm_ = 0;
    cudaStream_t stream_ = nullptr, copy_stream_ = nullptr;
    bool own_stream_ = false;
    cudaEvent_t ev_start_ = nullptr, ev_stop_ = nullptr;
    void *workspace_ = nullptr;  // split-K partials
    unsigned long long *stage_times_ = nullptr;  // per-stage, per-CTA time stamps (diagnostic, off by default)
    bool stage_times_on_ = false;
    void *arena_ = nullptr, *comm_ = nullptr, *state_ = nullptr, *stages_dev_ = nullptr;
    size_t arena_bytes_ = 0, comm_bytes_ = 0;
    int32_t *host_flags_ = nullptr;          // [0] run flag, [1] status mirror, [2..3] 64-bit count of finished iterations (mapped host memory)
    volatile int32_t *dev_flags_ = nullptr;  // device view of host_flags_
    char *peer_arena_[kMaxPeers], *peer_comm_[kMaxPeers];
    SymmArena symm_;  // the arena as a multicast-bound allocation, when NVLS was asked for (ARKB_NVLS=1) and is available
    bool compiled_ = false, launched_ = false, stopped_ = false, destroyed_ = false, pending_ = false;
    bool kernel_live_ = false;
    float elapsed_ms_ = -1;
    int n_launches_ = 0;
    unsigned long long spin_limit_ = 0, idle_limit_ = 0;
    // Kernel launches that only return when the kernel has ended (CUDA_LAUNCH_BLOCKING, a profiler): a resident
    // loop kernel cannot be kept, so every run request gets a launch of its own that leaves when the request is done.
    bool blocking_launch_ = false, probed_ = false;
    unsigned long long iters_expected_ = 0;  // iterations requested over the executor's life
};

void plan_check(const std::string &plan_json, int *n_stages, size_t *arena_bytes, int *n_processors);
std::string plan_dump(const std::string &plan_json);
void device_info(int device_id, DeviceInfo &out);

}  // namespace arkb
