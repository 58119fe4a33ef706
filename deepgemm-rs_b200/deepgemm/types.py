"""Host-side mirror of the reference's public types (deepgemm/src/types.rs, error.rs)."""
import enum
from dataclasses import dataclass
from typing import Optional

import torch


class Dtype(enum.IntEnum):       # types.rs:5-11
    Fp8 = 0
    Fp4 = 1
    Bf16 = 2
    F32 = 3


class Major(enum.IntEnum):       # types.rs:33-37
    K = 0
    Mn = 1


class SfGran(enum.IntEnum):      # types.rs:55-68; the value is the K granularity
    G32 = 32
    G128 = 128

    def k(self):
        return int(self)


class DgError(Exception):        # error.rs:6-15
    code = -1


class DriverError(DgError): code = 1
class InvalidArg(DgError): code = 3
class Unsupported(DgError): code = 4
class Mismatch(DgError): code = 5
class RuntimeLibError(DgError): code = 6
class DeviceTimeout(DgError): code = 8


_BY_CODE = {c.code: c for c in (DriverError, InvalidArg, Unsupported, Mismatch, RuntimeLibError, DeviceTimeout)}


def error_for(code, msg):
    return _BY_CODE.get(code, DgError)(msg)


@dataclass
class SfTensor:                  # types.rs:87-96
    rows: int                    # packed K rows = ceil(K / (gran * 4))
    cols: int                    # TMA-aligned MN
    gran: SfGran
    buf: torch.Tensor            # int32/uint32 device tensor [rows, cols]


@dataclass
class Operand:                   # types.rs:98-111
    dtype: Dtype
    major: Major
    rows: int
    k: int
    outer_stride: int            # elements (FP4: logical elements)
    sf: Optional[SfTensor]
    data: torch.Tensor

    @staticmethod
    def k_major(dtype, rows, k, outer_stride, sf, data):
        return Operand(dtype, Major.K, rows, k, outer_stride, sf, data)

    @staticmethod
    def mn_major(dtype, rows, k, outer_stride, sf, data):
        return Operand(dtype, Major.Mn, rows, k, outer_stride, sf, data)


@dataclass
class Output:                    # types.rs:113-121
    dtype: Dtype                 # Bf16 or F32
    rows: int
    cols: int
    stride: int
    data: torch.Tensor
