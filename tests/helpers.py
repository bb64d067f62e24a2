"""Shared helpers of the GPU parity tests."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import humming_oracle as oracle  # noqa: E402

from humming_b200 import dtypes, runtime  # noqa: E402
from humming_b200.layer import HummingLayer  # noqa: E402
from humming_b200.utils import synthetic  # noqa: E402

TORCH_TO_NAME = {torch.float16: "float16", torch.bfloat16: "bfloat16"}

# Output tolerance of the 16-bit-activation path against the fp32 oracle
# (reference README: atol 0.1, rtol 0.01).
ATOL_16, RTOL_16 = 0.1, 0.01


def build_layer(case: synthetic.DenseW4A16Case, has_bias=False, signed=False, device="cuda:0"):
    """HummingLayer loaded from a synthetic case through the public API."""
    name = TORCH_TO_NAME[case.dtype]
    layer = HummingLayer(shape_n=case.n, shape_k=case.k, a_dtype=name, b_dtype="int4" if signed else "uint4",
                         c_dtype=name, bs_dtype=name, weight_scale_group_size=case.group_size,
                         has_dynamic_zp=case.zero_points is not None, has_bias=has_bias).to(device)
    codes = case.codes - 8 if signed else case.codes
    bias = None
    if has_bias:
        gen = torch.Generator(device="cpu").manual_seed(7)
        bias = torch.randn((case.n,), generator=gen).to(case.dtype)
    layer.load_weight(weight=codes.to(device), weight_scale=case.scales.to(device),
                      zero_point=None if case.zero_points is None else case.zero_points.to(device),
                      bias=None if bias is None else bias.to(device))
    layer.finish_load()
    return layer, bias


def oracle_weight(case: synthetic.DenseW4A16Case) -> np.ndarray:
    return oracle.weight_ref_int(case.codes.numpy(), case.scales.float().numpy(), case.group_size, 4,
                                 None if case.zero_points is None else case.zero_points.numpy())


def assert_close_16(out: torch.Tensor, ref: torch.Tensor, what=""):
    torch.testing.assert_close(out.float().cpu(), ref.float().cpu(), atol=ATOL_16, rtol=RTOL_16, msg=lambda m: f"{what}: {m}")
