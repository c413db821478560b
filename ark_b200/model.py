"""Model graph: tensors, buffers and operators, serialised in the reference's
JSON shapes (ark/model/model_tensor.cpp:95-105, model_buffer.cpp:35-50,
model_op_arg.cpp:13-39). Mirrors ark::Model (ark/include/ark/model.hpp:18-258)
for the operators the engine runs; `ark_b200.ops` is the functional front end.
"""
import json

from . import data_type as dt
from .error import ModelError

INT_MIN = -2147483648


class Buffer:
    def __init__(self, model, rank=-1):
        self.id = model._next_buffer_id()
        self.rank = rank
        self.send_tags = []  # [rank, tag]
        self.recv_tags = []

    def tag_send(self, rank, tag):
        if [rank, tag] not in self.send_tags:
            self.send_tags.append([rank, tag])

    def tag_recv(self, rank, tag):
        if [rank, tag] not in self.recv_tags:
            self.recv_tags.append([rank, tag])

    def serialize(self):
        return {"Id": self.id, "Rank": self.rank, "SendTags": self.send_tags, "RecvTags": self.recv_tags}


class Tensor:
    """A view (shape, strides, offsets, padded_shape) over a buffer. `strides`
    are the allocated extents per dimension, not byte strides."""

    def __init__(self, model, dtype, buffer, shape, strides=None, offsets=None, padded_shape=None, name=""):
        shape = [int(s) for s in shape]
        if len(shape) > 4:
            raise ModelError("tensors have at most 4 dimensions")
        self.model = model
        self.id = model._next_tensor_id()
        self.dtype = dtype
        self.buffer = buffer
        self.shape = shape
        self.padded_shape = [int(s) for s in padded_shape] if padded_shape else list(shape)
        self.strides = [int(s) for s in strides] if strides else list(self.padded_shape)
        self.offsets = [int(s) for s in offsets] if offsets else [0] * len(shape)
        self.name = name
        nd = len(shape)
        if not (len(self.strides) == len(self.offsets) == len(self.padded_shape) == nd):
            raise ModelError("shape, strides, offsets and padded_shape must have the same rank")
        for i in range(nd):
            if self.shape[i] > self.padded_shape[i] or self.offsets[i] + self.padded_shape[i] > self.strides[i]:
                raise ModelError("tensor view does not fit its strides")

    def clone_view(self):
        return Tensor(self.model, self.dtype, self.buffer, self.shape, self.strides, self.offsets, self.padded_shape)

    def nelems(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def nbytes(self):
        return self.nelems() * self.dtype.nbytes

    def is_dense(self):
        return self.strides == self.shape and all(o == 0 for o in self.offsets)

    def serialize(self):
        return {"Id": self.id, "DataType": self.dtype.name, "Shape": self.shape, "Strides": self.strides,
                "Offsets": self.offsets, "PaddedShape": self.padded_shape, "Buffer": self.buffer.serialize()}

    def json(self):
        return json.dumps(self.serialize())

    # ---- data access through the running executor (python/ark/tensor.py:33-93) ----
    def _executor(self):
        from .runtime import Runtime
        rt = Runtime.get_runtime()
        if rt.executor is None:
            raise RuntimeError("the runtime is not launched")
        return rt.executor

    def to_numpy(self, ndarray=None):
        return self._executor().tensor_to_numpy(self, ndarray)

    def from_numpy(self, ndarray):
        self._executor().tensor_from_numpy(self, ndarray)
        return self

    def __repr__(self):
        return f"Tensor(id={self.id}, {self.dtype.name}, shape={self.shape})"


class Op:
    def __init__(self, type_, name, reads, writes, results, args=None, virtual=False):
        self.type = type_
        self.name = name
        self.reads = reads
        self.writes = writes
        self.results = results
        self.args = args or {}
        self.virtual = virtual
        self.context = {}

    @staticmethod
    def _arg(v):
        if isinstance(v, bool):
            return {"BOOL": v}
        if isinstance(v, int):
            return {"INT": v}
        if isinstance(v, float):
            return {"FLOAT": v}
        if isinstance(v, (list, tuple)):
            return {"DIMS": [int(x) for x in v]}
        raise ModelError(f"unsupported argument value {v!r}")

    def serialize(self):
        return {"Type": self.type, "Name": self.name, "IsVirtual": self.virtual,
                "ReadTensors": [t.serialize() for t in self.reads],
                "WriteTensors": [t.serialize() for t in self.writes],
                "ResultTensors": [t.serialize() for t in self.results],
                "Args": {k: self._arg(v) for k, v in self.args.items()}}


class Model:
    """Holds the operator list in creation order. One global instance is used by
    the functional API (python/ark/model.py:13-86)."""
    _model = None
    _rank = 0
    _world_size = 1

    def __init__(self, rank=None, world_size=None):
        self.rank = Model._rank if rank is None else rank
        self.world_size = Model._world_size if world_size is None else world_size
        self.ops = []
        self._tid = 0
        self._bid = 0
        self._tag = INT_MIN
        self._names = {}
        self._ctx_stack = []
        self._ctx_id = 0

    # ---- global instance ----
    @staticmethod
    def get_model():
        if Model._model is None:
            Model._model = Model()
        return Model._model

    @staticmethod
    def reset():
        Model._model = None

    @staticmethod
    def set_rank(rank):
        Model._rank = rank
        if Model._model is not None:
            Model._model.rank = rank

    @staticmethod
    def set_world_size(ws):
        Model._world_size = ws
        if Model._model is not None:
            Model._model.world_size = ws

    def _next_tensor_id(self):
        self._tid += 1
        return self._tid - 1

    def _next_buffer_id(self):
        self._bid += 1
        return self._bid - 1

    def unique_tag(self):
        """Tags count up from INT_MIN (ark/api/model.cpp:27-49)."""
        t = self._tag
        self._tag += 1
        return t

    def _unique_name(self, name):
        n = self._names.get(name, 0)
        self._names[name] = n + 1
        return name if n == 0 else f"{name}_{n}"

    def add_op(self, type_, name, reads, writes, results, args=None, virtual=False):
        op = Op(type_, self._unique_name(name or type_.lower()), reads, writes, results, args, virtual)
        ctx = {}
        for c in self._ctx_stack:  # outer to inner; Id is fixed by the outermost context
            for k, v in c.items():
                if k == "Id" and "Id" in ctx:
                    continue
                if k == "Config" and "Config" in ctx:
                    merged = dict(ctx["Config"])
                    merged.update(v)
                    ctx["Config"] = merged
                else:
                    ctx[k] = v
        op.context = ctx
        self.ops.append(op)
        return op

    def new_tensor(self, shape, dtype, strides=None, offsets=None, padded_shape=None, rank=-1, name=""):
        t = Tensor(self, dtype, Buffer(self, rank), shape, strides, offsets, padded_shape, name)
        self.add_op("Tensor", name or "tensor", [], [], [t], virtual=True)
        return t

    def serialize(self):
        return {"Rank": self.rank, "WorldSize": self.world_size, "Nodes": [o.serialize() for o in self.ops]}
