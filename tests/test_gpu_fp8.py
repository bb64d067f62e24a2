"""GPU parity of the FP8-activation paths against the CPU oracle:
MXFP4 x FP8 (float4e2m1 weights, UE8M0 scales per 32, e4m3 activations with
per-token scales) and W4A8 (uint4 / int4 weights, 16-bit group-128 scales).
Bounds: atol 0.1, rtol 0.03 (the reference's FP8-activation tests,
tests/test_datatype.py:123)."""
import numpy as np
import pytest
import torch

from helpers import oracle
from humming_b200 import runtime
from humming_b200.layer import HummingLayer, HummingMethod

pytestmark = pytest.mark.gpu
ATOL, RTOL = 0.1, 0.03


def mxfp4_case(n, k, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    codes = torch.randint(0, 16, (n, k), generator=gen, dtype=torch.int32)
    exps = torch.randint(-8, -1, (n, k // 32), generator=gen)           # exponents uniform in [-8, -2]
    scale_codes = (exps + 127).to(torch.uint8)
    w = oracle.decode_fp(codes.numpy(), 2, 1, True) * np.repeat(oracle.e8m0_to_float(scale_codes.numpy()), 32, axis=-1)
    return codes, scale_codes.view(torch.float8_e8m0fnu), torch.from_numpy(w)


def quantized_acts(m, k, seed):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((m, k), generator=gen).bfloat16()
    q, s = oracle.quant_input_e4m3(x)
    return x, q, s


@pytest.mark.parametrize("n,k", [(128, 128), (512, 1024)])
def test_mxfp4_prepared_weights_decode_bit_exact(cuda_device, n, k):
    codes, scales, w_ref = mxfp4_case(n, k, seed=n)
    layer = HummingLayer(shape_n=n, shape_k=k, a_dtype="float8e4m3", b_dtype="float4e2m1", c_dtype="bfloat16",
                         bs_dtype="float8e8m0", weight_scale_group_size=32).to(cuda_device)
    layer.load_weight(weight=codes.to(cuda_device), weight_scale=scales.to(cuda_device))
    layer.finish_load()
    got = runtime.dequant_prepared(HummingMethod._desc(layer.meta), layer.weight, layer.weight_scale)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), w_ref.numpy().view(np.uint32))


@pytest.mark.parametrize("m", [1, 16, 100, 300, 1100])
def test_mxfp4_fp8_gemm(cuda_device, m):
    n, k = 1024, 2048
    codes, scales, w_ref = mxfp4_case(n, k, seed=1)
    layer = HummingLayer(shape_n=n, shape_k=k, a_dtype="float8e4m3", b_dtype="float4e2m1", c_dtype="bfloat16",
                         bs_dtype="float8e8m0", weight_scale_group_size=32).to(cuda_device)
    layer.load_weight(weight=codes.to(cuda_device), weight_scale=scales.to(cuda_device))
    layer.finish_load()
    x, q, s = quantized_acts(m, k, seed=m)
    out = layer(inputs=q.to(cuda_device), input_scale=s.to(cuda_device))
    layer.check_status()
    inputs_ref = q.float() * s                                    # reference humming/utils/test.py:24-64
    ref = oracle.gemm_ref(inputs_ref, w_ref, torch.bfloat16)
    torch.testing.assert_close(out.float().cpu(), ref.float(), atol=ATOL, rtol=RTOL)
    # un-quantized activations are quantized by the layer (dynamic per-token scales)
    out2 = layer(inputs=x.to(cuda_device))
    torch.testing.assert_close(out2.float().cpu(), ref.float(), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("m", [40, 300])
def test_mxfp4_fp8_gemm_cta_pair(cuda_device, m):
    """The two-CTA kernel gives bit-identical results for MXFP4 weights (no K split)."""
    from humming_b200 import native
    n, k = 1024, 2048
    codes, scales, w_ref = mxfp4_case(n, k, seed=2)
    layer = HummingLayer(shape_n=n, shape_k=k, a_dtype="float8e4m3", b_dtype="float4e2m1", c_dtype="bfloat16",
                         bs_dtype="float8e8m0", weight_scale_group_size=32).to(cuda_device)
    layer.load_weight(weight=codes.to(cuda_device), weight_scale=scales.to(cuda_device))
    layer.finish_load()
    _, q, s = quantized_acts(m, k, seed=m)
    outs = []
    for flags in (native.HM_FLAG_NO_SPLIT_K | native.HM_FLAG_NO_CTA_PAIR, native.HM_FLAG_NO_SPLIT_K | native.HM_FLAG_CTA_PAIR):
        layer.humming_kernel_options[""]["native_flags"] = flags
        outs.append(layer(inputs=q.to(cuda_device), input_scale=s.to(cuda_device)).clone())
    layer.check_status()
    ref = oracle.gemm_ref(q.float() * s, w_ref, torch.bfloat16)
    torch.testing.assert_close(outs[1].float().cpu(), ref.float(), atol=ATOL, rtol=RTOL)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("signed", [False, True])
@pytest.mark.parametrize("m", [7, 64, 400])
def test_w4a8_gemm(cuda_device, signed, m):
    n, k = 512, 1024
    gen = torch.Generator(device="cpu").manual_seed(3)
    codes = torch.randint(0, 16, (n, k), generator=gen, dtype=torch.int32)
    scales = (torch.randn((n, k // 128), generator=gen).abs() * 0.02 + 1e-3).bfloat16()
    layer = HummingLayer(shape_n=n, shape_k=k, a_dtype="float8e4m3", b_dtype="int4" if signed else "uint4", c_dtype="bfloat16",
                         bs_dtype="bfloat16", weight_scale_group_size=128).to(cuda_device)
    layer.load_weight(weight=(codes - 8 if signed else codes).to(cuda_device), weight_scale=scales.to(cuda_device))
    layer.finish_load()
    _, q, s = quantized_acts(m, k, seed=m)
    out = layer(inputs=q.to(cuda_device), input_scale=s.to(cuda_device))
    layer.check_status()
    w_ref = torch.from_numpy(oracle.weight_ref_int(codes.numpy(), scales.float().numpy(), 128, 4))
    ref = oracle.gemm_ref(q.float() * s, w_ref, torch.bfloat16)
    torch.testing.assert_close(out.float().cpu(), ref.float(), atol=ATOL, rtol=RTOL)


def test_fp8_inputs_need_scales(cuda_device):
    layer = HummingLayer(shape_n=128, shape_k=128, a_dtype="float8e4m3", b_dtype="uint4", c_dtype="bfloat16",
                         bs_dtype="bfloat16", weight_scale_group_size=128).to(cuda_device)
    layer.load_weight(weight=torch.zeros((128, 128), dtype=torch.int32, device=cuda_device),
                      weight_scale=torch.ones((128, 1), dtype=torch.bfloat16, device=cuda_device))
    layer.finish_load()
    q = torch.zeros((4, 128), dtype=torch.float8_e4m3fn, device=cuda_device)
    with pytest.raises(ValueError):
        layer(inputs=q, input_scale=torch.ones(3, device=cuda_device))
