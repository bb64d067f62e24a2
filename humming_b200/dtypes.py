"""Data type descriptors with the reference's names and string forms.

Mirrors ``humming/dtypes.py`` of the reference (``DataType.from_str`` :10-20,
``InergerType`` :45-86, ``FloatingPointType`` :89-155, module constants
:158-183, ``torch_dtype_map`` :186-192).  ``to_cpp_str`` is kept because callers
use it as a specialisation key; ``to_native`` maps a dtype to the integer codes
of the C ABI (``HM_*`` in ``include/humming_b200.h``).
"""
import re

import torch


class DataType(object):
    is_integer_type = False
    is_floating_point_type = False

    @classmethod
    def from_str(cls, s):
        if isinstance(s, DataType):
            return s
        if "float" in s:
            return FloatingPointType.from_str(s)
        if "int" in s:
            return InergerType.from_str(s)
        raise NotImplementedError(s)

    @classmethod
    def from_torch_dtype(cls, torch_dtype):
        name = str(torch_dtype)
        if "float" in name:
            return FloatingPointType.from_torch_dtype(torch_dtype)
        if "int" in name:
            return InergerType.from_torch_dtype(torch_dtype)
        raise NotImplementedError(name)

    def to_str(self, lowercase=True):
        raise NotImplementedError

    def to_native(self):
        raise NotImplementedError

    def __hash__(self):
        return hash(str(self))

    def __eq__(self, other):
        return str(self) == str(other)

    def __repr__(self):
        return self.to_str()


class InergerType(DataType):  # (sic) the reference spells it this way
    is_integer_type = True

    def __init__(self, is_signed, num_bits):
        self.is_signed = bool(is_signed)
        self.num_bits = int(num_bits)

    @classmethod
    def from_str(cls, s):
        if isinstance(s, InergerType):
            return s
        m = re.fullmatch(r"(u*)int(\d+)", s.lower())
        if not m:
            raise ValueError(f"invalid integer dtype: {s}")
        return cls(is_signed=m.group(1) == "", num_bits=int(m.group(2)))

    @classmethod
    def from_torch_dtype(cls, torch_dtype):
        assert isinstance(torch_dtype, torch.dtype)
        return cls.from_str(str(torch_dtype)[6:])

    def to_str(self, lowercase=True):
        s = ("Int" if self.is_signed else "UInt") + str(self.num_bits)
        return s.lower() if lowercase else s

    def to_cpp_str(self):
        return f"IntegerType<{str(self.is_signed).lower()}, {self.num_bits}>"

    def to_native(self):
        return (0x200 if self.is_signed else 0x100) + self.num_bits

    def id(self):
        return int(1e7 + self.num_bits * 1e5 + self.is_signed * 1e4)


IntegerType = InergerType


class FloatingPointType(DataType):
    is_floating_point_type = True

    def __init__(self, num_bits, exponent_bits, mantissa_bits):
        self.num_bits = int(num_bits)
        self.exponent_bits = int(exponent_bits)
        self.mantissa_bits = int(mantissa_bits)
        self.sign_bits = self.num_bits - self.exponent_bits - self.mantissa_bits
        assert self.sign_bits in (0, 1)
        self.is_signed = self.sign_bits != 0

    @classmethod
    def from_str(cls, s):
        if isinstance(s, FloatingPointType):
            return s
        s = s.lower()
        if s in ("float16", "half"):
            return cls(16, 5, 10)
        if s == "bfloat16":
            return cls(16, 8, 7)
        if s == "float32":
            return cls(32, 8, 23)
        m = re.fullmatch(r"float(\d+)_*e(\d+)m(\d+)", s)
        if not m:
            raise ValueError(f"invalid floating point dtype: {s}")
        return cls(int(m.group(1)), int(m.group(2)), int(m.group(3)))

    @classmethod
    def from_torch_dtype(cls, torch_dtype):
        assert isinstance(torch_dtype, torch.dtype)
        name = str(torch_dtype)[6:].replace("fnu", "").replace("fn", "")
        return cls.from_str(name)

    def to_str(self, lowercase=True):
        s = f"Float{self.num_bits}E{self.exponent_bits}M{self.mantissa_bits}"
        s = {"Float16E5M10": "Float16", "Float16E8M7": "BFloat16", "Float32E8M23": "Float32"}.get(s, s)
        return s.lower() if lowercase else s

    def to_cpp_str(self):
        return f"FloatingPointType<{self.num_bits}, {self.exponent_bits}, {self.mantissa_bits}>"

    def to_native(self):
        key = (self.num_bits, self.exponent_bits, self.mantissa_bits)
        codes = {(16, 5, 10): 1, (16, 8, 7): 2, (32, 8, 23): 3, (8, 4, 3): 4, (8, 5, 2): 5, (8, 8, 0): 6, (4, 2, 1): 7}
        if key not in codes:
            raise NotImplementedError(f"{self} has no native code")
        return codes[key]

    def id(self):
        return int(2e7 + self.num_bits * 1e5 + self.is_signed * 1e4 + self.exponent_bits * 1e2 + self.mantissa_bits)


# Module-level constants (reference humming/dtypes.py:158-183): dtypes.uint4,
# dtypes.float8e4m3, dtypes.bfloat16, ...
_INT_NAMES = [f"uint{b}" for b in range(1, 9)] + ["int2", "int3", "int4", "int5", "int6", "int7", "int8", "int32"]
_FLOAT_NAMES = ["float4e2m1", "float6e2m3", "float6e3m2", "float8e4m3", "float8e5m2", "float8e8m0",
                "float16", "bfloat16", "float32"]
for _n in _INT_NAMES + _FLOAT_NAMES:
    globals()[_n] = DataType.from_str(_n)
del _n

torch_dtype_map = {
    globals()["float8e8m0"]: torch.float8_e8m0fnu,
    globals()["float8e4m3"]: torch.float8_e4m3fn,
    globals()["float8e5m2"]: torch.float8_e5m2,
    globals()["float16"]: torch.float16,
    globals()["bfloat16"]: torch.bfloat16,
    # Not in the reference's map: fp32 group scales are accepted natively here.
    globals()["float32"]: torch.float32,
}
