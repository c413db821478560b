/*
 * libark_b200 — C ABI of the B200-native execution engine for ARK plans.
 *
 * This is the boundary a host framework binds to run an ARK plan (the JSON
 * produced by ark::Planner, format: docs/plan_file.md of the reference) on
 * sm_100a. It replaces, behind ark::Executor, what the reference implements
 * with its code generator, nvcc JIT, GPU manager and MSCCL++ channel set-up.
 * Each entry point names the reference interface it stands for.
 *
 * Conventions: every function returns an arkb_status (0 = success); after a
 * non-zero return arkb_last_error() gives the message (thread-local). Status
 * values follow the reference's exception classes (ark/include/ark/error.hpp:29-43)
 * so a C++ binding can re-throw the matching type. Handles are opaque; one
 * executor is used from one thread at a time. No entry point takes or returns
 * a framework type: plain pointers, sizes and NUL-terminated strings only.
 */
#ifndef ARK_B200_H_
#define ARK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum arkb_status {
    ARKB_OK = 0,
    ARKB_INTERNAL_ERROR = 1,      /* ark::InternalError */
    ARKB_INVALID_USAGE = 2,       /* ark::InvalidUsageError */
    ARKB_MODEL_ERROR = 3,         /* ark::ModelError */
    ARKB_PLAN_ERROR = 4,          /* ark::PlanError */
    ARKB_UNSUPPORTED = 5,         /* ark::UnsupportedError */
    ARKB_SYSTEM_ERROR = 6,        /* ark::SystemError */
    ARKB_GPU_ERROR = 7            /* ark::GpuError */
} arkb_status;

typedef struct arkb_executor arkb_executor;

/* Device facts the planner needs. Replaces GpuManager::Info
 * (ark/gpu/gpu_manager.hpp:40-54). */
typedef struct arkb_device_info {
    int cc_major, cc_minor;
    int num_sm;
    int max_threads_per_block;
    int smem_per_block_optin; /* bytes */
    int regs_per_sm;
    size_t total_mem;         /* bytes */
    char arch[16];            /* "CUDA_100" on B200 */
    char name[64];
} arkb_device_info;

/* Snapshot of the device-side status block, filled by arkb_executor_status. */
typedef struct arkb_run_status {
    int code;            /* 0 ok, 1 grid barrier timed out, 2 tensor-core pipeline wait timed out,
                            3 peer flag wait timed out, 4 loop kernel left after a long idle period */
    int stage;           /* index of the lowered stage where it happened */
    int cta;
    int n_stages;        /* stages in the lowered program */
    int n_launches;      /* loop-kernel launches since creation */
    uint64_t iterations; /* iterations completed since creation */
    uint64_t last_run_ns;/* device time of the last run request (globaltimer) */
} arkb_run_status;

/* Bootstrap callback used only at set-up on multi-rank plans: gathers `bytes`
 * bytes from every rank into `recv` (rank-major). Stands in for the MSCCL++
 * TCP bootstrap of the reference (ark/api/executor.cpp:291-298, 410-500); the
 * host supplies it (NCCL / gloo / MPI all work). May be NULL when WorldSize == 1. */
typedef int (*arkb_allgather_fn)(void *ctx, const void *send, void *recv, size_t bytes);

const char *arkb_last_error(void);
/* Version string "major.minor.patch" (ark::version(), ark/api/version.cpp). */
const char *arkb_version(void);

/* GpuManager::get_instance(dev)->info() — ark/gpu/gpu_manager.cpp. Needs a GPU. */
arkb_status arkb_device_info_get(int device_id, arkb_device_info *out);

/* Parses and validates a plan without touching a GPU; writes the number of
 * lowered stages, the arena bytes and the processor count it needs.
 * Counterpart of the checks in Executor::Impl::init + CodeGenerator
 * (ark/api/executor.cpp:226-289, ark/codegen.cpp:79-180). */
arkb_status arkb_plan_check(const char *plan_json, int *n_stages, size_t *arena_bytes, int *n_processors);
/* Same lowering, written out as text (one line per stage) into `buf`; `needed`
 * receives the size the full text takes. Counterpart of inspecting the .cu
 * the reference's CodeGenerator::code() returns (ark/codegen.hpp:15-32). */
arkb_status arkb_plan_dump(const char *plan_json, char *buf, size_t buf_bytes, size_t *needed);

/* ark::Executor::Executor(device_id, stream, name, plan, loop_mode)
 * (ark/include/ark/executor.hpp:25-29, ark/api/executor.cpp:888-899).
 * `stream` is a cudaStream_t or NULL for an executor-owned stream. */
arkb_status arkb_executor_create(int device_id, void *stream, const char *name, const char *plan_json,
                                 int loop_mode, arkb_allgather_fn allgather, void *allgather_ctx,
                                 arkb_executor **out);
/* Executor::compile (executor.hpp:46): lowers the plan to the stage program,
 * allocates and zero-fills the arena, maps peers, uploads the program. */
arkb_status arkb_executor_compile(arkb_executor *e);
/* Executor::launch (executor.hpp:49): starts the loop kernel (loop mode) and records the start event.
 * When kernel launches only return once the kernel has ended (CUDA_LAUNCH_BLOCKING=1, a profiler
 * attached; found out with a 2 ms probe launch) no resident kernel is kept: every run() then launches a
 * kernel that serves that request and leaves. */
arkb_status arkb_executor_launch(arkb_executor *e);
/* Executor::run(iter) (executor.hpp:52). */
arkb_status arkb_executor_run(arkb_executor *e, int iter);
/* Executor::wait(max_spin_count) (executor.hpp:55); a device-side timeout comes back as ARKB_GPU_ERROR,
 * and so does a request whose iterations did not all run: the count of finished iterations the kernel
 * reports is compared with what was asked for, and a request that met no kernel is served by a relaunch. */
arkb_status arkb_executor_wait(arkb_executor *e, int64_t max_spin_count);
/* Executor::stop(max_spin_count) (executor.hpp:61): returns milliseconds between launch and stop. */
arkb_status arkb_executor_stop(arkb_executor *e, int64_t max_spin_count, float *elapsed_msec);
/* Executor::barrier (executor.hpp:64): host-side barrier over all ranks through the bootstrap callback. */
arkb_status arkb_executor_barrier(arkb_executor *e);
/* Executor::destroy (executor.hpp:67). Also frees the handle. */
arkb_status arkb_executor_destroy(arkb_executor *e);

/* Executor::tensor_address / tensor_read / tensor_write (executor.hpp:73-90).
 * The tensor is given as its JSON serialisation (ModelTensor::serialize,
 * ark/model/model_tensor.cpp:95-105): {"Id","DataType","Shape","Strides",
 * "Offsets","PaddedShape","Buffer":{"Id",...}}. `bytes` must equal
 * shape.nelems() * sizeof(dtype); strided tensors are packed/unpacked. */
arkb_status arkb_executor_tensor_address(arkb_executor *e, const char *tensor_json, uintptr_t *addr);
arkb_status arkb_executor_tensor_read(arkb_executor *e, const char *tensor_json, void *data, size_t bytes,
                                      void *stream, int is_d2d);
arkb_status arkb_executor_tensor_write(arkb_executor *e, const char *tensor_json, const void *data, size_t bytes,
                                       void *stream, int is_d2d);

/* Device status block and counters (the reference has no equivalent: its device waits are unbounded). */
arkb_status arkb_executor_status(arkb_executor *e, arkb_run_status *out);
/* Stream the executor launches on (for callers that record their own events). */
arkb_status arkb_executor_stream(arkb_executor *e, void **stream);
/* Human-readable dump of the lowered stage program (one line per stage). The
 * returned pointer stays valid until the next call on the same executor.
 * Counterpart of reading the generated .cu the reference leaves in $ARK_TMP. */
arkb_status arkb_executor_program_dump(arkb_executor *e, const char **text);
/* Upper bound, in nanoseconds, of every device-side wait (grid barrier,
 * tensor-core pipeline, peer flags); 0 restores the default of 10 s. Takes effect at the next
 * launch. Stands in for the MaxSpinCount template argument of the reference's
 * comm::wait (ark/include/kernels/comm.h:197-206), which its ops leave at -1. */
arkb_status arkb_executor_set_wait_limit(arkb_executor *e, uint64_t nanoseconds);
/* How long, in nanoseconds, the resident loop kernel stays on the GPU without a run request before it
 * returns (0 restores the default of 20 s). The next run() starts it again and wait() notices a request
 * that arrived just as the kernel left, so the limit only trades GPU occupancy against relaunch cost.
 * Takes effect at the next launch. The reference's loop kernel has no such limit: it spins on the flag
 * until stop() (ark/include/kernels/kernel_template.in:40-69). */
arkb_status arkb_executor_set_idle_limit(arkb_executor *e, uint64_t nanoseconds);
/* Diagnostic: per-stage, per-CTA time stamps. enable = 1 / 0 switches the recording on / off (after
 * compile, before launch; -1 leaves it as it is). When it is on, every CTA notes the GPU's nanosecond
 * timer on entering and leaving each stage; `out` receives the stamps of the last finished iteration
 * as [n_stages][grid][2] words (at most `capacity`), `written` how many. Call after wait(). Stands in
 * for reading the reference's per-kernel timings out of a profiler; off by default (it adds a CTA-wide
 * barrier after every stage). */
arkb_status arkb_executor_stage_times(arkb_executor *e, int enable, uint64_t *out, size_t capacity, size_t *written,
                                      int *n_stages, int *grid);

/* y[m, n] = x[m, k] . w[n, k]^T for 1 <= m <= 16 (dtype 1 = fp16, 2 = bf16; fp32 accumulation), the
 * split-K form of the engine's skinny Matmul, for callers that cannot allocate device memory at the
 * point of the call (inside a stream capture, in a pre-allocated real-time loop, inside a host whose
 * memory pool they do not own). It has no counterpart in the reference. It allocates nothing: the
 * fp32 partial sums live in a 4 MiB array that is part of the library image (every GPU that loads
 * the library holds it until the process exits). x, w and y are device pointers (x and w 16-byte
 * aligned), k a multiple of 8; `stream` is a cudaStream_t or NULL. A call whose partials
 * (k-ranges * m * n * 4 bytes; the k-range count is chosen by the library, up to 64) exceed 4 MiB
 * returns ARKB_INVALID_USAGE. All calls on a device share the array: it needs no clearing (each call
 * overwrites what it reads), but calls that overlap in time on the GPU race on it — order them on
 * one stream or with events. The first call on each device resolves the array's device address;
 * make that call before any stream capture begins. */
arkb_status arkb_matvec_splitk_static(const void *x, const void *w, void *y, int m, int n, int k, int dtype,
                                      void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ARK_B200_H_ */
