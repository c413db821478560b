"""Planner: model -> plan JSON in the reference's plan-file format
(docs/plan_file.md; ark/api/planner.cpp:127-262). Config precedence is the
reference's: PlannerContext `config` > installed rules > the op's default.
"""
import json

from .error import PlanError
from .model import Model

ARCH = "CUDA_100"
DEFAULT_NUM_SM = 148  # B200


class Plan:
    """A plan as a dict plus (de)serialisation (python/ark/planner.py:110-166)."""

    def __init__(self, plan):
        self.plan = plan if plan is not None else {}

    def __str__(self):
        return json.dumps(self.plan)

    @property
    def rank(self):
        return self.plan["Rank"]

    @property
    def world_size(self):
        return self.plan["WorldSize"]

    @property
    def num_processors(self):
        return self.plan["NumProcessors"]

    @property
    def task_infos(self):
        return self.plan["TaskInfos"]

    @property
    def processor_groups(self):
        return self.plan["ProcessorGroups"]

    @staticmethod
    def from_str(s):
        return Plan(json.loads(s))

    @staticmethod
    def from_file(path):
        with open(path) as f:
            return Plan(json.load(f))


class PlannerContext:
    """Scopes planning hints over the ops created inside it
    (python/ark/planner.py:168-208, ark/api/planner.cpp:41-87): processor_range,
    warp_range, sram_range, sync (False merges the ops into one task) and config."""

    def __init__(self, processor_range=None, warp_range=None, sram_range=None, sync=True, config=None):
        m = Model.get_model()
        self._model = m
        ctx = {}
        if not any("Id" in c for c in m._ctx_stack):
            ctx["Id"] = m._ctx_id
            m._ctx_id += 1
        if processor_range is not None:
            ctx["ProcessorRange"] = [int(x) for x in processor_range]
        if warp_range is not None:
            ctx["WarpRange"] = [int(x) for x in warp_range]
        if sram_range is not None:
            ctx["SramRange"] = [int(x) for x in sram_range]
        if sync is False:
            ctx["Sync"] = False
        if config is not None:
            ctx["Config"] = dict(config)
        self._ctx = ctx

    def __enter__(self):
        self._model._ctx_stack.append(self._ctx)
        return self

    def __exit__(self, *exc):
        self._model._ctx_stack.pop()


def _dims4(v):
    return [1] * (4 - len(v)) + list(v)


def default_config(op, num_sm=DEFAULT_NUM_SM):
    """Default Config of an op for CUDA_100, in the reference's per-op schema
    (docs/plan_file.md "Config Details"). The engine splits elementwise work
    itself, so Tile/NumWarps/SramBytes only document the task shape."""
    t = op.type
    if t == "Matmul":
        a, b = op.reads[0], op.reads[1]
        ta, tb = op.args["TransposeInput"], op.args["TransposeOther"]
        ash, bsh = a.padded_shape, b.padded_shape
        m = 1 if len(ash) == 1 else ash[-2]
        k = ash[-1]
        n = 1 if len(bsh) == 1 else bsh[-1]
        if ta:
            m, k = k, m
        if tb:
            n = bsh[-2]
        tm, tn = (256, 128) if m > n else (128, 256)  # ark/ops/ops_matmul.cpp:191-192
        res4 = _dims4(op.results[0].shape)
        nt = res4[0] * res4[1] * ((m + tm - 1) // tm) * ((n + tn - 1) // tn)
        return {"NumWarps": 8, "SramBytes": 147456, "TileShapeMNK": [tm, tn, 64], "NumTasks": nt}
    if t in ("ReduceSum", "ReduceMax", "ReduceMean"):
        nd = len(op.reads[0].shape)
        last = op.args["Axis"] in (nd - 1, -1)
        return {"NumWarps": 1, "ImplType": "WarpWise" if last else "ElementWise", "SramBytes": 256 if last else 0,
                "NumTasks": op.results[0].nelems()}
    if t in ("Send", "SendDone", "Recv", "DeviceSync"):
        c = {"ChannelType": "Sm", "NumTasks": 1, "NumWarps": 1, "SramBytes": 0}
        if t == "Send":
            c["Signal"] = True
            c["NumTasks"] = num_sm  # the copy is spread over the whole grid
        if t == "Recv":
            c["Wait"] = True
        return c
    if t == "AllReduce":
        return {"NumWarps": 16, "SramBytes": 0, "NumTasks": num_sm, "Algo": "auto"}
    if t in ("SendPacket", "RecvPacket", "RecvReduceSendPacket", "RecvReduceSend"):
        # ark/ops/ops_communication.cpp:226-246, 332-351, 434-453, 541-557 (1-warp tasks over 1 x 128 / 1 x 512 tiles)
        sh = _dims4(op.results[0].shape)
        ty = 512 if t == "SendPacket" else 128
        c = {"NumWarps": 1, "SramBytes": 0, "Tile": [1, ty], "NumTasks": sh[0] * sh[1] * sh[2] * ((sh[3] + ty - 1) // ty)}
        if t != "RecvReduceSend":
            c["PacketType"] = "mscclpp::LL16Packet"
        return c
    if t in ("RMSNorm", "LayerNorm", "Softmax"):
        sh = _dims4(op.reads[0].shape)
        return {"NumWarps": 1, "SramBytes": 0, "NumTasks": sh[0] * sh[1] * sh[2]}
    if t == "PrefillAttention":
        sh = _dims4(op.results[0].shape)
        return {"NumWarps": 16, "SramBytes": 0, "NumTasks": sh[0] * (sh[1] * sh[2] + 127) // 128}
    if t == "DecodeAttention":
        sh = _dims4(op.results[0].shape)
        return {"NumWarps": 16, "SramBytes": 0, "NumTasks": sh[0] * sh[1]}
    if t == "Embedding":
        sh = _dims4(op.results[0].shape)
        return {"NumWarps": 1, "SramBytes": 0, "NumTasks": sh[0] * sh[1] * sh[2]}
    if t == "Transpose":
        sh = _dims4(op.results[0].shape)
        return {"NumWarps": 1, "SramBytes": 0, "Tile": [8, 8],
                "NumTasks": sh[0] * sh[1] * ((sh[2] + 7) // 8) * ((sh[3] + 7) // 8)}
    if t == "Noop":
        return {"NumWarps": 1, "SramBytes": 0, "NumTasks": 0}
    # Broadcast1 / Broadcast2 family (ark/ops/ops_broadcast.cpp:47-68, 120-141)
    sh = _dims4(op.results[0].shape)
    tx, ty = (64, 1) if sh[2] > sh[3] else (1, 64)
    nt = sh[0] * sh[1] * ((sh[2] + tx - 1) // tx) * ((sh[3] + ty - 1) // ty)
    return {"NumWarps": 1, "SramBytes": 0, "Tile": [tx, ty], "NumTasks": nt}


class Planner:
    """ark::Planner (ark/include/ark/planner.hpp:35-51)."""

    def __init__(self, device_id=0, num_sm=None, model=None, reuse_memory=False):
        """`reuse_memory`: the plan asks the executor (top-level field "ArenaReuse") to let intermediates whose
        lifetimes do not overlap share arena space. Off by default, as in the reference, where every tensor keeps
        its memory and can be read back after a run (ark/api/executor.cpp:374-408)."""
        self.reuse_memory = reuse_memory
        self.device_id = device_id
        self.model = model if model is not None else Model.get_model()
        self.num_sm = num_sm
        self._rules = []

    def install_config_rule(self, rule):
        """`rule(op_json: str, arch: str) -> str` returns a Config JSON or ""."""
        def safe(op_str, arch):
            try:
                return rule(op_str, arch)
            except Exception:  # a failing rule is skipped (ark/api/planner.cpp:108-118)
                return ""
        self._rules.append(safe)

    def _num_sm(self):
        if self.num_sm is not None:
            return self.num_sm
        try:
            from .executor import device_info
            return device_info(self.device_id)["num_sm"]
        except Exception:
            return DEFAULT_NUM_SM

    def plan(self, pretty=False):
        num_sm = self._num_sm()
        task_infos, processor_groups = [], []
        max_proc, max_warp = 1, 1
        next_task_id = 0
        prev_ctx_id = -1
        first = True
        for op in self.model.ops:
            if op.virtual:
                continue
            ctx = op.context
            config = None
            if ctx.get("Config"):
                config = dict(default_config(op, num_sm))
                config.update(ctx["Config"])
            elif self._rules:
                op_str = json.dumps(op.serialize())
                for rule in self._rules:
                    s = rule(op_str, ARCH)
                    if s:
                        config = json.loads(s)
                        break
            if not config:
                config = default_config(op, num_sm)
            for f in ("NumWarps", "NumTasks", "SramBytes"):
                if f not in config:
                    raise PlanError(f"Config field not found: {f} in {op.name}")
            num_warps, num_tasks, sram = config["NumWarps"], config["NumTasks"], config["SramBytes"]
            gran = config.get("Granularity", 1)
            cid = ctx.get("Id", -1)
            sync = ctx.get("Sync", True)
            op_json = op.serialize()
            op_json["Config"] = config
            if cid == prev_ctx_id and not sync and task_infos:
                ti = task_infos[-1]
                ti["NumWarps"] = max(ti["NumWarps"], num_warps)
                ti["SramBytes"] = max(ti["SramBytes"], sram)
                ti["Ops"].append(op_json)
                # the task's range covers the op with the most tasks (the reference keeps the first op's count,
                # ark/api/planner.cpp:229-231, which only suits ops with equal task counts)
                tgrp = processor_groups[-1]["ResourceGroups"][0]["TaskGroups"][0]
                tgrp["TaskRange"] = [0, max(tgrp["TaskRange"][1], num_tasks)]
            else:
                tid = next_task_id if first else next_task_id + 1
                next_task_id = tid
                task_infos.append({"Id": tid, "NumWarps": num_warps, "SramBytes": sram, "Ops": [op_json]})
                if "ProcessorRange" in ctx:
                    pr = list(ctx["ProcessorRange"])
                    max_proc = max(max_proc, pr[1])
                else:
                    # the engine splits an op over all CTAs of its range itself, so the
                    # default range is the whole grid (the reference caps it at NumTasks)
                    single = op.type in ("Recv", "SendDone", "DeviceSync", "Noop")
                    n = 1 if single else num_sm
                    pr = [0, n]
                    max_proc = max(max_proc, n)
                wr = list(ctx["WarpRange"]) if "WarpRange" in ctx else [0, num_warps]
                max_warp = max(max_warp, wr[1])
                sr = list(ctx["SramRange"]) if "SramRange" in ctx else [0, sram]
                processor_groups.append({"ProcessorRange": pr, "ResourceGroups": [{
                    "ProcessorRange": pr, "WarpRange": wr, "SramRange": sr,
                    "TaskGroups": [{"TaskId": tid, "TaskRange": [0, num_tasks], "Granularity": gran}]}]})
            prev_ctx_id = cid
            first = False
        plan = {"Rank": self.model.rank, "WorldSize": self.model.world_size, "Architecture": ARCH,
                "NumProcessors": max_proc, "NumWarpsPerProcessor": max_warp, "TaskInfos": task_infos,
                "ProcessorGroups": processor_groups}
        if self.reuse_memory:
            plan["ArenaReuse"] = True
        return Plan(plan)
