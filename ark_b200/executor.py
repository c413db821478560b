"""ctypes binding of libark_b200 and the Executor class with the reference's
method set (ark/include/ark/executor.hpp:19-100, python/executor_py.cpp:43-85).

The library is built in-tree by `ark_b200/csrc/build.sh`; there is no CPU
fallback — importing the library fails loudly when it was not built.
"""
import ctypes
import os

import numpy as np

from .error import STATUS_TO_ERROR, BaseError, InvalidUsageError

_HERE = os.path.dirname(os.path.abspath(__file__))
# ARK_B200_LIB overrides the library location (e.g. an instrumented build)
LIB_PATH = os.environ.get("ARK_B200_LIB") or os.path.join(_HERE, "lib", "libark_b200.so")
_lib = None

ALLGATHER_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t)


class DeviceInfo(ctypes.Structure):
    _fields_ = [("cc_major", ctypes.c_int), ("cc_minor", ctypes.c_int), ("num_sm", ctypes.c_int),
                ("max_threads_per_block", ctypes.c_int), ("smem_per_block_optin", ctypes.c_int),
                ("regs_per_sm", ctypes.c_int), ("total_mem", ctypes.c_size_t), ("arch", ctypes.c_char * 16),
                ("name", ctypes.c_char * 64)]


class RunStatus(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int), ("stage", ctypes.c_int), ("cta", ctypes.c_int), ("n_stages", ctypes.c_int),
                ("n_launches", ctypes.c_int), ("iterations", ctypes.c_uint64), ("last_run_ns", ctypes.c_uint64)]


def lib():
    """Loads libark_b200.so (raises when it is missing: build it with
    `python -c "import __graft_entry__ as g; g.build()"` or ark_b200/csrc/build.sh)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build the CUDA library first (ark_b200/csrc/build.sh)")
        L = ctypes.CDLL(LIB_PATH)
        L.arkb_last_error.restype = ctypes.c_char_p
        L.arkb_version.restype = ctypes.c_char_p
        vp, cp, ci = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int
        L.arkb_device_info_get.argtypes = [ci, ctypes.POINTER(DeviceInfo)]
        L.arkb_plan_check.argtypes = [cp, ctypes.POINTER(ci), ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ci)]
        L.arkb_plan_dump.argtypes = [cp, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]
        L.arkb_executor_create.argtypes = [ci, vp, cp, cp, ci, ALLGATHER_FN, vp, ctypes.POINTER(vp)]
        for f in ("compile", "launch", "barrier", "destroy"):
            getattr(L, "arkb_executor_" + f).argtypes = [vp]
        L.arkb_executor_run.argtypes = [vp, ci]
        L.arkb_executor_wait.argtypes = [vp, ctypes.c_int64]
        L.arkb_executor_stop.argtypes = [vp, ctypes.c_int64, ctypes.POINTER(ctypes.c_float)]
        L.arkb_executor_tensor_address.argtypes = [vp, cp, ctypes.POINTER(ctypes.c_size_t)]
        L.arkb_executor_tensor_read.argtypes = [vp, cp, vp, ctypes.c_size_t, vp, ci]
        L.arkb_executor_tensor_write.argtypes = [vp, cp, vp, ctypes.c_size_t, vp, ci]
        L.arkb_executor_status.argtypes = [vp, ctypes.POINTER(RunStatus)]
        L.arkb_executor_stream.argtypes = [vp, ctypes.POINTER(vp)]
        L.arkb_executor_program_dump.argtypes = [vp, ctypes.POINTER(cp)]
        L.arkb_executor_set_wait_limit.argtypes = [vp, ctypes.c_uint64]
        L.arkb_executor_set_idle_limit.argtypes = [vp, ctypes.c_uint64]
        if hasattr(L, "arkb_executor_stage_times"):  # absent from older builds of the library
            L.arkb_executor_stage_times.argtypes = [vp, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t),
                                                    ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        L.arkb_matvec_splitk_static.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp]
        _lib = L
    return _lib


def _check(status):
    if status != 0:
        msg = lib().arkb_last_error().decode("utf-8", "replace")
        raise STATUS_TO_ERROR.get(status, BaseError)(msg)


def version():
    return lib().arkb_version().decode()


def device_info(device_id=0):
    di = DeviceInfo()
    _check(lib().arkb_device_info_get(device_id, ctypes.byref(di)))
    return {"cc": (di.cc_major, di.cc_minor), "num_sm": di.num_sm, "smem_per_block_optin": di.smem_per_block_optin,
            "total_mem": di.total_mem, "arch": di.arch.decode(), "name": di.name.decode()}


def plan_check(plan_str):
    """Validates and lowers a plan without a GPU. Returns (n_stages, arena_bytes, n_processors)."""
    ns, ab, npr = ctypes.c_int(), ctypes.c_size_t(), ctypes.c_int()
    _check(lib().arkb_plan_check(str(plan_str).encode(), ctypes.byref(ns), ctypes.byref(ab), ctypes.byref(npr)))
    return ns.value, ab.value, npr.value


def plan_dump(plan_str):
    need = ctypes.c_size_t()
    _check(lib().arkb_plan_dump(str(plan_str).encode(), None, 0, ctypes.byref(need)))
    buf = ctypes.create_string_buffer(need.value)
    _check(lib().arkb_plan_dump(str(plan_str).encode(), buf, need.value, ctypes.byref(need)))
    return buf.value.decode()


def matvec_splitk_static(x_ptr, w_ptr, y_ptr, m, n, k, dtype, stream=0):
    """y[m,n] = x[m,k] . w[n,k]^T on device pointers without any allocation (scratch is a fixed 4 MiB
    array inside the library). dtype: "fp16" or "bf16". Raises InvalidUsageError when the problem's
    partial sums do not fit the fixed scratch. Calls sharing a device must not overlap on the GPU."""
    code = {"fp16": 1, "bf16": 2}[dtype]
    _check(lib().arkb_matvec_splitk_static(ctypes.c_void_p(x_ptr), ctypes.c_void_p(w_ptr), ctypes.c_void_p(y_ptr), int(m),
                                           int(n), int(k), code, ctypes.c_void_p(stream or None)))


def torch_allgather(group=None):
    """Bootstrap callback over torch.distributed (any backend): gathers raw bytes from all ranks.
    Pass a gloo group when the callback can be invoked (Executor.barrier) while a loop kernel is
    resident: the kernel keeps every SM busy, so an NCCL kernel would wait until it leaves."""
    import torch
    import torch.distributed as dist

    def fn(_ctx, send, recv, nbytes):
        try:
            ws = dist.get_world_size(group)
            backend = dist.get_backend(group)
            dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
            src = np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(send)).copy()
            t = torch.from_numpy(src).to(dev)
            outs = [torch.empty_like(t) for _ in range(ws)]
            dist.all_gather(outs, t, group=group)
            dst = np.ctypeslib.as_array((ctypes.c_uint8 * (nbytes * ws)).from_address(recv))
            for r in range(ws):
                dst[r * nbytes:(r + 1) * nbytes] = outs[r].cpu().numpy()
            return 0
        except Exception as e:  # reported as ARKB_SYSTEM_ERROR by the library
            print(f"ark_b200: bootstrap allgather failed: {e}")
            return 1
    return fn


class Executor:
    """ark::Executor. `stream` is a raw cudaStream_t value (0: executor-owned stream)."""

    def __init__(self, device_id, stream, name, plan, loop_mode=True, allgather=None):
        self._h = ctypes.c_void_p()
        self._destroyed = False
        self._cb = ALLGATHER_FN(allgather) if allgather is not None else ctypes.cast(None, ALLGATHER_FN)
        if device_id is None or device_id < 0:
            raise InvalidUsageError(f"Invalid device ID {device_id}")
        _check(lib().arkb_executor_create(int(device_id), ctypes.c_void_p(stream or None), name.encode(),
                                          str(plan).encode(), int(bool(loop_mode)), self._cb, None,
                                          ctypes.byref(self._h)))
        self.device_id = device_id
        self.loop_mode = loop_mode

    def compile(self):
        _check(lib().arkb_executor_compile(self._h))

    def launch(self):
        _check(lib().arkb_executor_launch(self._h))

    def run(self, iter=1):
        _check(lib().arkb_executor_run(self._h, int(iter)))

    def wait(self, max_spin_count=-1):
        _check(lib().arkb_executor_wait(self._h, int(max_spin_count)))

    def stop(self, max_spin_count=-1):
        ms = ctypes.c_float()
        _check(lib().arkb_executor_stop(self._h, int(max_spin_count), ctypes.byref(ms)))
        return ms.value

    def barrier(self):
        _check(lib().arkb_executor_barrier(self._h))

    def destroy(self):
        if not self._destroyed and self._h:
            self._destroyed = True
            _check(lib().arkb_executor_destroy(self._h))
            self._h = ctypes.c_void_p()

    def destroyed(self):
        return self._destroyed

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def stream(self):
        s = ctypes.c_void_p()
        _check(lib().arkb_executor_stream(self._h, ctypes.byref(s)))
        return s.value or 0

    def status(self):
        st = RunStatus()
        _check(lib().arkb_executor_status(self._h, ctypes.byref(st)))
        return {f[0]: getattr(st, f[0]) for f in RunStatus._fields_}

    def program_dump(self):
        p = ctypes.c_char_p()
        _check(lib().arkb_executor_program_dump(self._h, ctypes.byref(p)))
        return p.value.decode()

    def set_wait_limit(self, nanoseconds):
        """Bound of every device-side wait; a wait that runs out makes wait() raise GpuError."""
        _check(lib().arkb_executor_set_wait_limit(self._h, int(nanoseconds)))

    def set_idle_limit(self, nanoseconds):
        """How long the resident loop kernel stays without a run request before it returns (0: default, 20 s)."""
        _check(lib().arkb_executor_set_idle_limit(self._h, int(nanoseconds)))

    def enable_stage_times(self, on=True):
        """Diagnostic (after compile, before launch): every CTA records when it enters and leaves each stage."""
        _check(lib().arkb_executor_stage_times(self._h, 1 if on else 0, None, 0, None, None, None))

    def stage_times(self):
        """Time stamps of the last finished iteration as an int64 array [n_stages, grid, 2] (GPU nanosecond
        timer; zeros for CTAs outside a stage's processor range). Call after wait()."""
        ns, grid, w = ctypes.c_int(), ctypes.c_int(), ctypes.c_size_t()
        _check(lib().arkb_executor_stage_times(self._h, -1, None, 0, None, ctypes.byref(ns), ctypes.byref(grid)))
        out = np.zeros((ns.value, grid.value, 2), np.uint64)
        _check(lib().arkb_executor_stage_times(self._h, -1, ctypes.c_void_p(out.ctypes.data), out.size, ctypes.byref(w), None, None))
        return out.astype(np.int64)

    @staticmethod
    def _tjson(tensor):
        return (tensor if isinstance(tensor, str) else tensor.json()).encode()

    def tensor_address(self, tensor):
        a = ctypes.c_size_t()
        _check(lib().arkb_executor_tensor_address(self._h, self._tjson(tensor), ctypes.byref(a)))
        return a.value

    def tensor_read(self, tensor, address, nbytes, stream=0, is_d2d=False):
        _check(lib().arkb_executor_tensor_read(self._h, self._tjson(tensor), ctypes.c_void_p(address), nbytes,
                                               ctypes.c_void_p(stream or None), int(is_d2d)))

    def tensor_write(self, tensor, address, nbytes, stream=0, is_d2d=False):
        _check(lib().arkb_executor_tensor_write(self._h, self._tjson(tensor), ctypes.c_void_p(address), nbytes,
                                                ctypes.c_void_p(stream or None), int(is_d2d)))

    # numpy conveniences (python/ark/tensor.py:33-93)
    def tensor_to_numpy(self, tensor, ndarray=None):
        npdt = tensor.dtype.to_numpy()
        if ndarray is None:
            ndarray = np.zeros(tensor.shape, dtype=npdt)
        elif not ndarray.flags["C_CONTIGUOUS"] or ndarray.nbytes != tensor.nbytes():
            raise InvalidUsageError("destination array must be contiguous and of the tensor's size")
        self.tensor_read(tensor, ndarray.ctypes.data, ndarray.nbytes)
        return ndarray

    def tensor_from_numpy(self, tensor, ndarray):
        a = np.ascontiguousarray(ndarray)
        if a.nbytes != tensor.nbytes():
            raise InvalidUsageError(f"array bytes ({a.nbytes}) mismatch the tensor data bytes ({tensor.nbytes()})")
        self.tensor_write(tensor, a.ctypes.data, a.nbytes)
