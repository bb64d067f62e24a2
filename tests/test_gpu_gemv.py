"""GPU parity of the decode kernel that serves up to 16 tokens (weights decoded in
registers, warp-level MMA): against the CPU oracle (atol 0.1 / rtol 0.01 on 16-bit
outputs) and against the tcgen05 kernel."""
import pytest
import torch

from helpers import assert_close_16, build_layer
from humming_b200 import native, runtime
from humming_b200.layer import HummingMethod
from humming_b200.utils import synthetic
from test_gpu_gemm import run_case

pytestmark = pytest.mark.gpu


def plan_of(layer, m, flags=0):
    return runtime.gemm_plan(HummingMethod._desc(layer.meta, flags=flags), m)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("zp", [False, True])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8, 9, 13, 16])
def test_gemv_matches_oracle(cuda_device, dtype, zp, m):
    case = synthetic.dense_w4a16_case(512, 2048, dtype, zp, seed=17)
    out, ref, layer = run_case(case, m, cuda_device, flags=native.HM_FLAG_DECODE_KERNEL)
    assert plan_of(layer, m, native.HM_FLAG_DECODE_KERNEL).mode == 2
    assert (plan_of(layer, m).mode == 2) == (m <= 4)
    assert_close_16(out, ref, f"gemv m={m}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("zp", [False, True])
@pytest.mark.parametrize("m", [1])
def test_gemv_fma_form_matches_oracle(cuda_device, dtype, zp, m):
    """A single token runs the fp32 multiply-add form by default."""
    case = synthetic.dense_w4a16_case(512, 2048, dtype, zp, seed=19)
    out, ref, layer = run_case(case, m, cuda_device)
    assert plan_of(layer, m).mode == 2
    assert_close_16(out, ref, f"gemv fma m={m}")


@pytest.mark.parametrize("n,k,g", [(128, 128, 64), (128, 128, 128), (256, 4096, 128), (2048, 256, 64), (384, 1024, 0), (1536, 2048, 256),
                                   (128, 14336, 128)])
def test_gemv_shapes_and_groups(cuda_device, n, k, g):
    case = synthetic.dense_w4a16_case(n, k, torch.bfloat16, True, group_size=g or k, seed=5)
    for m, flags in ((3, native.HM_FLAG_DECODE_KERNEL), (11, native.HM_FLAG_DECODE_KERNEL), (1, 0), (2, 0)):
        out, ref, _ = run_case(case, m, cuda_device, flags=flags)
        assert_close_16(out, ref, f"gemv n={n} k={k} g={g} m={m}")


def test_gemv_bias_signed_weights_and_tensor_core_agreement(cuda_device):
    case = synthetic.dense_w4a16_case(1024, 4096, torch.bfloat16, True, seed=23)
    out, ref, layer = run_case(case, 2, cuda_device, has_bias=True)
    assert_close_16(out, ref, "gemv bias")
    x = synthetic.activations(2, case.k, case.dtype, seed=1).to(cuda_device)
    again = layer(inputs=x)
    assert torch.equal(again, out)                       # the K split is summed in a fixed order
    layer.humming_kernel_options[""]["native_flags"] = native.HM_FLAG_NO_GEMV
    assert plan_of(layer, 2, native.HM_FLAG_NO_GEMV).mode != 2
    tc = layer(inputs=x)
    layer.check_status()
    torch.testing.assert_close(tc.float(), out.float(), atol=0.1, rtol=0.01)
    signed = synthetic.dense_w4a16_case(256, 1024, torch.float16, False, seed=3)
    layer_s, _ = build_layer(signed, signed=True)
    xs = synthetic.activations(1, 1024, torch.float16, seed=2).to(cuda_device)
    got = layer_s(inputs=xs)
    layer_s.humming_kernel_options[""]["native_flags"] = native.HM_FLAG_NO_GEMV
    torch.testing.assert_close(got.float(), layer_s(inputs=xs).float(), atol=0.1, rtol=0.01)


@pytest.mark.parametrize("name", ["qkv", "o", "gate_up", "down"])
def test_gemv_llama_shapes_against_gpu_fp32(cuda_device, name):
    n, k = synthetic.LLAMA3_8B_SHAPES[name]
    case = synthetic.dense_w4a16_case(n, k, torch.bfloat16, True, seed=13)
    layer, _ = build_layer(case)
    layer.humming_kernel_options[""]["native_flags"] = native.HM_FLAG_DECODE_KERNEL
    w = runtime.dequant_prepared(HummingMethod._desc(layer.meta), layer.weight, layer.weight_scale, layer.zero_point)
    for m in (1, 4, 16, -1, -2):   # negative: default plan (fp32 multiply-add form for one or two tokens)
        layer.humming_kernel_options[""]["native_flags"] = native.HM_FLAG_DECODE_KERNEL if m > 0 else 0
        m = abs(m)
        x = synthetic.activations(m, k, torch.bfloat16).to(cuda_device)
        out = layer(inputs=x)
        assert_close_16(out, (x.float() @ w.T).to(torch.bfloat16), f"gemv {name} m={m}")
        assert torch.equal(layer(inputs=x * 2).float(), out.float() * 2)   # powers of two commute with every rounding
    layer.check_status()
