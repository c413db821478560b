"""Runtime: the launch/run/wait/stop state machine of python/ark/runtime.py:27-200."""
import logging
from enum import Enum

from .executor import Executor, torch_allgather
from .model import Model
from .planner import Plan, Planner


class _RuntimeState:
    runtime = None
    executor = None


class Runtime:
    class State(Enum):
        Init = 0
        LaunchedNotRunning = 1
        Running = 2

    @staticmethod
    def get_runtime():
        if _RuntimeState.runtime is None:
            _RuntimeState.runtime = Runtime()
        return _RuntimeState.runtime

    def __init__(self):
        self.executor = None
        self.state = Runtime.State.Init
        _RuntimeState.runtime = self

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.reset()

    def launched(self):
        return self.state in (Runtime.State.LaunchedNotRunning, Runtime.State.Running)

    def running(self):
        return self.state == Runtime.State.Running

    def launch(self, plan=None, device_id=0, stream=0, loop_mode=True, allgather=None):
        """Plans (unless a plan is given), creates the executor, compiles and launches."""
        if self.launched():
            logging.warning("Runtime is already launched, skip launching")
            return
        plan = Planner(device_id).plan() if plan is None else plan
        if self.state == Runtime.State.Init:
            if _RuntimeState.executor is not None and not _RuntimeState.executor.destroyed():
                logging.warning("Destroying an old executor")
                _RuntimeState.executor.destroy()
            ws = plan.world_size if isinstance(plan, Plan) else Model.get_model().world_size
            if allgather is None and ws > 1:
                allgather = torch_allgather()
            _RuntimeState.executor = Executor(device_id, stream, "ArkRuntime", str(plan), loop_mode, allgather)
            self.executor = _RuntimeState.executor
            self.executor.compile()
        self.executor.launch()
        self.state = Runtime.State.LaunchedNotRunning

    def run(self, iter=1, non_blocking=False):
        if self.state != Runtime.State.LaunchedNotRunning:
            raise RuntimeError("ARK runtime is not launched")
        self.state = Runtime.State.Running
        self.executor.run(iter)
        if not non_blocking:
            self.wait()

    def barrier(self):
        if self.state != Runtime.State.LaunchedNotRunning:
            raise RuntimeError("ARK runtime is not launched")
        self.executor.barrier()

    def wait(self):
        if self.state != Runtime.State.Running:
            logging.warning("ARK runtime is not running, skip waiting")
            return
        self.state = Runtime.State.LaunchedNotRunning
        self.executor.wait()

    def stop(self):
        if not self.launched():
            logging.warning("ARK runtime is never launched, skip stopping")
            return None
        elapsed = self.executor.stop()
        self.state = Runtime.State.LaunchedNotRunning
        return elapsed

    def reset(self):
        if self.launched():
            try:
                self.stop()
            except Exception:
                pass
        if self.executor is not None:
            if not self.executor.destroyed():
                self.executor.destroy()
            self.executor = None
        _RuntimeState.executor = None
        self.state = Runtime.State.Init
