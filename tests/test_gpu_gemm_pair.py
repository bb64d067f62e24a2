"""GPU parity of the CTA-pair (cta_group::2) dense GEMM against the CPU oracle
and against the single-CTA kernel: same tolerance as the other GEMM tests
(atol 0.1 / rtol 0.01 on 16-bit outputs)."""
import pytest
import torch

from helpers import assert_close_16
from humming_b200 import native, runtime
from humming_b200.layer import HummingMethod
from humming_b200.utils import synthetic
from test_gpu_gemm import run_case

pytestmark = pytest.mark.gpu

PAIR = native.HM_FLAG_CTA_PAIR


def plan_of(layer, m):
    return runtime.gemm_plan(HummingMethod._desc(layer.meta, flags=layer.humming_kernel_options[""].get("native_flags", 0)), m)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("zp", [False, True])
@pytest.mark.parametrize("m", [1, 16, 33, 64, 100, 128, 234, 256, 300, 1000, 2500])
def test_pair_m_sweep(cuda_device, dtype, zp, m):
    case = synthetic.dense_w4a16_case(512, 1024, dtype, zp, seed=11)
    out, ref, layer = run_case(case, m, cuda_device, flags=PAIR)
    assert plan_of(layer, m).cta_pair == 1
    assert_close_16(out, ref, f"pair m={m}")


@pytest.mark.parametrize("m_tile", [32, 64, 128, 256])
@pytest.mark.parametrize("flags", [PAIR, PAIR | native.HM_FLAG_NO_SPLIT_K])
def test_pair_every_tile_size_and_schedule(cuda_device, m_tile, flags):
    case = synthetic.dense_w4a16_case(1024, 2048, torch.bfloat16, True, seed=21)
    out, ref, _ = run_case(case, 200, cuda_device, flags=flags, m_tile=m_tile)
    assert_close_16(out, ref, f"pair m_tile={m_tile} flags={flags}")


@pytest.mark.parametrize("n,k,g", [(256, 128, 64), (256, 4096, 128), (2048, 256, 64), (768, 1024, 0), (1536, 2048, 256)])
def test_pair_shapes_and_groups(cuda_device, n, k, g):
    case = synthetic.dense_w4a16_case(n, k, torch.bfloat16, True, group_size=g or k, seed=5)
    out, ref, _ = run_case(case, 48, cuda_device, flags=PAIR)
    assert_close_16(out, ref, f"pair n={n} k={k} g={g}")


def test_pair_falls_back_when_not_eligible(cuda_device):
    """N not a multiple of 256, or a token tile the pair kernel does not have:
    the single-CTA kernel runs and the answer is the same."""
    case = synthetic.dense_w4a16_case(384, 1024, torch.bfloat16, True, seed=3)
    out, ref, layer = run_case(case, 40, cuda_device, flags=PAIR)
    assert plan_of(layer, 40).cta_pair == 0
    assert_close_16(out, ref, "n=384")
    case = synthetic.dense_w4a16_case(512, 1024, torch.bfloat16, True, seed=3)
    out, ref, _ = run_case(case, 40, cuda_device, flags=PAIR, m_tile=16)
    assert_close_16(out, ref, "m_tile=16")
    out, ref, layer = run_case(case, 40, cuda_device, flags=PAIR | native.HM_FLAG_NO_CTA_PAIR)
    assert plan_of(layer, 40).cta_pair == 0


@pytest.mark.parametrize("m", [16, 200, 4096])
def test_pair_matches_single_cta_unsplit(cuda_device, m):
    """Without a K split both kernels accumulate each output in the same order."""
    case = synthetic.dense_w4a16_case(2048, 2048, torch.bfloat16, True, seed=8)
    one, ref, _ = run_case(case, m, cuda_device, flags=native.HM_FLAG_NO_SPLIT_K | native.HM_FLAG_NO_CTA_PAIR)
    two, _, _ = run_case(case, m, cuda_device, flags=native.HM_FLAG_NO_SPLIT_K | PAIR)
    assert_close_16(two, ref, f"pair m={m}")
    assert torch.equal(one, two)


def test_pair_split_k_is_deterministic(cuda_device):
    case = synthetic.dense_w4a16_case(512, 8192, torch.bfloat16, True, seed=4)
    a, ref, layer = run_case(case, 24, cuda_device, flags=PAIR)
    assert plan_of(layer, 24).mode == 1
    x = synthetic.activations(24, case.k, case.dtype, seed=1).to(cuda_device)
    for _ in range(3):
        assert torch.equal(layer(inputs=x), a)
    layer.check_status()
    assert_close_16(a, ref, "pair split-K")


@pytest.mark.parametrize("name,m", [("gate_up", 16), ("down", 64), ("qkv", 256), ("gate_up", 4096)])
def test_pair_llama_shapes_against_gpu_fp32(cuda_device, name, m):
    n, k = synthetic.LLAMA3_8B_SHAPES[name]
    case = synthetic.dense_w4a16_case(n, k, torch.bfloat16, True, seed=13)
    from helpers import build_layer
    layer, _ = build_layer(case)
    layer.humming_kernel_options[""]["native_flags"] = PAIR
    desc = HummingMethod._desc(layer.meta)
    w = runtime.dequant_prepared(desc, layer.weight, layer.weight_scale, layer.zero_point)
    x = synthetic.activations(m, k, torch.bfloat16).to(cuda_device)
    out = layer(inputs=x)
    layer.check_status()
    assert_close_16(out, (x.float() @ w.T).to(torch.bfloat16), f"pair {name} m={m}")
