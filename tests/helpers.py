"""Shared builders for the GPU parity tests: seeded inputs, oracle-quantised operands uploaded
to the device, and the comparison helpers."""
import numpy as np
import torch

import oracle as o
from deepgemm import Dtype, Major, Operand, Output, SfGran, SfTensor

TOL = {"fp8": 1e-3, "fp4": 2e-3, "bf16": 1e-3}  # calc_diff bounds (FP8 / FP4 from the stated contract)


def randn(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape).astype(np.float32)


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.view(dtype)
    return t.cuda()


def sf_tensor(words, gran):
    return SfTensor(words.shape[0], words.shape[1], SfGran(gran), dev(words.view(np.int32)))


def quantised_operand(x, kind, gran, block128=False):
    """x f32 [rows, k] -> (device Operand, oracle GoldenOperand), quantised on the host by the oracle."""
    rows, k = x.shape
    if kind == "fp8":
        data, sf = o.quant_fp8_block128_host(x) if block128 else o.quant_mx_host(x, o.FP8, gran)
        op = Operand.k_major(Dtype.Fp8, rows, k, k, sf_tensor(sf, gran), dev(data))
        return op, o.GoldenOperand(data, sf, o.FP8, gran, k)
    data, sf = o.quant_mx_host(x, o.FP4, 32)
    op = Operand.k_major(Dtype.Fp4, rows, k, k, sf_tensor(sf, 32), dev(data))
    return op, o.GoldenOperand(data, sf, o.FP4, 32, k)


def bf16_operand(x):
    rows, k = x.shape
    t = torch.from_numpy(x).to(torch.bfloat16)
    return Operand.k_major(Dtype.Bf16, rows, k, k, None, t.cuda()), t.float().numpy()


def new_output(rows, cols, f32=False, stride=None, fill=None):
    stride = stride or cols
    dt = torch.float32 if f32 else torch.bfloat16
    t = torch.full((rows, stride), float("nan") if fill is None else fill, dtype=dt, device="cuda")
    return Output(Dtype.F32 if f32 else Dtype.Bf16, rows, cols, stride, t)


def to_f32(out):
    return out.data.float().cpu().numpy()[:, :out.cols]


def bf16_round(x):
    return o.bf16_bits_to_f32(o.f32_to_bf16_bits_np(x))


def assert_close_to_oracle(got, ref, kind, what=""):
    """calc_diff bound of the contract plus an element-wise bound that catches a single wrong
    tile, row or column (calc_diff alone averages it away)."""
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    d = o.calc_diff(got, ref)
    assert d <= TOL[kind], f"{what}: calc_diff {d:.3e} > {TOL[kind]}"
    scale = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))) + 1e-30
    err = np.abs(got - ref) / scale
    assert err.max() <= 0.05, f"{what}: element error {err.max():.3e} of rms at {np.unravel_index(err.argmax(), err.shape)}"
