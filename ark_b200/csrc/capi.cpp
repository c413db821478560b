// extern "C" surface of libark_b200 (declared in include/ark_b200.h).
#include <cstring>
#include <string>

#include "ark_b200.h"
#include "executor.hpp"

namespace {
thread_local std::string g_last_error;

template <typename F>
arkb_status guard(F &&f) {
    try {
        f();
        return ARKB_OK;
    } catch (const arkb::Error &e) {
        g_last_error = e.what();
        return (arkb_status)e.code;
    } catch (const std::exception &e) {
        g_last_error = e.what();
        return ARKB_INTERNAL_ERROR;
    } catch (...) {
        g_last_error = "unknown error";
        return ARKB_INTERNAL_ERROR;
    }
}
arkb::Executor *ex(arkb_executor *e) {
    if (!e) throw arkb::Error(arkb::E_USAGE, "null executor handle");
    return reinterpret_cast<arkb::Executor *>(e);
}
}  // namespace

namespace arkb {
void set_last_error(const std::string &msg) { g_last_error = msg; }
}  // namespace arkb

extern "C" {

const char *arkb_last_error(void) { return g_last_error.c_str(); }
const char *arkb_version(void) { return "0.1.0"; }

arkb_status arkb_device_info_get(int device_id, arkb_device_info *out) {
    return guard([&] {
        if (!out) throw arkb::Error(arkb::E_USAGE, "null output");
        arkb::DeviceInfo di;
        arkb::device_info(device_id, di);
        std::memset(out, 0, sizeof(*out));
        out->cc_major = di.cc_major;
        out->cc_minor = di.cc_minor;
        out->num_sm = di.num_sm;
        out->max_threads_per_block = di.max_threads_per_block;
        out->smem_per_block_optin = di.smem_per_block_optin;
        out->regs_per_sm = di.regs_per_sm;
        out->total_mem = di.total_mem;
        std::strncpy(out->arch, di.arch.c_str(), sizeof(out->arch) - 1);
        std::strncpy(out->name, di.name.c_str(), sizeof(out->name) - 1);
    });
}

arkb_status arkb_plan_check(const char *plan_json, int *n_stages, size_t *arena_bytes, int *n_processors) {
    return guard([&] {
        if (!plan_json) throw arkb::Error(arkb::E_USAGE, "null plan");
        arkb::plan_check(plan_json, n_stages, arena_bytes, n_processors);
    });
}

arkb_status arkb_plan_dump(const char *plan_json, char *buf, size_t buf_bytes, size_t *needed) {
    return guard([&] {
        if (!plan_json) throw arkb::Error(arkb::E_USAGE, "null plan");
        std::string s = arkb::plan_dump(plan_json);
        if (needed) *needed = s.size() + 1;
        if (buf && buf_bytes) {
            std::strncpy(buf, s.c_str(), buf_bytes - 1);
            buf[buf_bytes - 1] = 0;
        }
    });
}

arkb_status arkb_executor_create(int device_id, void *stream, const char *name, const char *plan_json, int loop_mode,
                                 arkb_allgather_fn allgather, void *allgather_ctx, arkb_executor **out) {
    return guard([&] {
        if (!out || !plan_json) throw arkb::Error(arkb::E_USAGE, "null argument");
        arkb::AllgatherFn ag;
        if (allgather)
            ag = [allgather, allgather_ctx](const void *s, void *r, size_t b) { return allgather(allgather_ctx, s, r, b); };
        *out = reinterpret_cast<arkb_executor *>(
            new arkb::Executor(device_id, stream, name ? name : "", plan_json, loop_mode != 0, ag));
    });
}
arkb_status arkb_executor_compile(arkb_executor *e) { return guard([&] { ex(e)->compile(); }); }
arkb_status arkb_executor_launch(arkb_executor *e) { return guard([&] { ex(e)->launch(); }); }
arkb_status arkb_executor_run(arkb_executor *e, int iter) { return guard([&] { ex(e)->run(iter); }); }
arkb_status arkb_executor_wait(arkb_executor *e, int64_t max_spin_count) {
    return guard([&] { ex(e)->wait(max_spin_count); });
}
arkb_status arkb_executor_stop(arkb_executor *e, int64_t max_spin_count, float *elapsed_msec) {
    return guard([&] {
        float ms = ex(e)->stop(max_spin_count);
        if (elapsed_msec) *elapsed_msec = ms;
    });
}
arkb_status arkb_executor_barrier(arkb_executor *e) { return guard([&] { ex(e)->barrier(); }); }
arkb_status arkb_executor_destroy(arkb_executor *e) {
    return guard([&] {
        arkb::Executor *x = ex(e);
        x->destroy();
        delete x;
    });
}
arkb_status arkb_executor_tensor_address(arkb_executor *e, const char *tensor_json, uintptr_t *addr) {
    return guard([&] {
        if (!tensor_json || !addr) throw arkb::Error(arkb::E_USAGE, "null argument");
        *addr = ex(e)->tensor_address(tensor_json);
    });
}
arkb_status arkb_executor_tensor_read(arkb_executor *e, const char *tensor_json, void *data, size_t bytes, void *stream,
                                      int is_d2d) {
    return guard([&] {
        if (!tensor_json || !data) throw arkb::Error(arkb::E_USAGE, "null argument");
        ex(e)->tensor_io(tensor_json, data, bytes, stream, is_d2d != 0, false);
    });
}
arkb_status arkb_executor_tensor_write(arkb_executor *e, const char *tensor_json, const void *data, size_t bytes,
                                       void *stream, int is_d2d) {
    return guard([&] {
        if (!tensor_json || !data) throw arkb::Error(arkb::E_USAGE, "null argument");
        ex(e)->tensor_io(tensor_json, const_cast<void *>(data), bytes, stream, is_d2d != 0, true);
    });
}
arkb_status arkb_executor_status(arkb_executor *e, arkb_run_status *out) {
    return guard([&] {
        if (!out) throw arkb::Error(arkb::E_USAGE, "null output");
        arkb::arkb_status_snapshot s = ex(e)->status();
        out->code = s.code;
        out->stage = s.stage;
        out->cta = s.cta;
        out->n_stages = s.n_stages;
        out->n_launches = s.n_launches;
        out->iterations = s.iterations;
        out->last_run_ns = s.last_run_ns;
    });
}
arkb_status arkb_executor_stream(arkb_executor *e, void **stream) {
    return guard([&] {
        if (!stream) throw arkb::Error(arkb::E_USAGE, "null output");
        *stream = ex(e)->stream();
    });
}
arkb_status arkb_executor_program_dump(arkb_executor *e, const char **text) {
    return guard([&] {
        if (!text) throw arkb::Error(arkb::E_USAGE, "null output");
        arkb::Executor *x = ex(e);
        x->dump_text = x->program().dump();
        *text = x->dump_text.c_str();
    });
}
arkb_status arkb_executor_set_wait_limit(arkb_executor *e, uint64_t nanoseconds) {
    return guard([&] { ex(e)->set_spin_limit(nanoseconds); });
}

arkb_status arkb_executor_set_idle_limit(arkb_executor *e, uint64_t nanoseconds) {
    return guard([&] { ex(e)->set_idle_limit(nanoseconds); });
}

arkb_status arkb_executor_stage_times(arkb_executor *e, int enable, uint64_t *out, size_t capacity, size_t *written,
                                      int *n_stages, int *grid) {
    return guard([&] {
        arkb::Executor *x = ex(e);
        if (enable >= 0) x->enable_stage_times(enable != 0);
        const size_t w = x->read_stage_times(reinterpret_cast<unsigned long long *>(out), capacity, n_stages, grid);
        if (written) *written = w;
    });
}

}  // extern "C"
