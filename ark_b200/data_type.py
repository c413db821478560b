"""Data types of tensors (python/ark/data_type.py, ark/api/data_type.cpp:28-36)."""
import numpy as np


class DataType:
    def __init__(self, name, nbytes, np_type):
        self.name = name          # serialised name, e.g. "FP16"
        self.nbytes = nbytes
        self.np_type = np_type    # numpy storage type (bf16 is carried as uint16 bit patterns)

    def element_size(self):
        return self.nbytes

    def to_numpy(self):
        return self.np_type

    def __repr__(self):
        return f"ark.{self.name.lower()}"

    @staticmethod
    def from_name(name):
        for t in ALL_TYPES:
            if t.name == name:
                return t
        raise ValueError(f"unknown data type {name}")

    @staticmethod
    def from_numpy(np_type):
        np_type = np.dtype(np_type)
        for t in ALL_TYPES:
            if t is not bf16 and t is not byte and np.dtype(t.np_type) == np_type:
                return t
        raise ValueError(f"no ARK data type for numpy {np_type}")


fp32 = DataType("FP32", 4, np.float32)
fp16 = DataType("FP16", 2, np.float16)
bf16 = DataType("BF16", 2, np.uint16)
int32 = DataType("INT32", 4, np.int32)
uint32 = DataType("UINT32", 4, np.uint32)
int8 = DataType("INT8", 1, np.int8)
uint8 = DataType("UINT8", 1, np.uint8)
byte = DataType("BYTE", 1, np.uint8)
ALL_TYPES = [fp32, fp16, bf16, int32, uint32, int8, uint8, byte]
