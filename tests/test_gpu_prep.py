"""GPU parity of the load-path kernels against the CPU oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from helpers import oracle, oracle_weight, build_layer
from humming_b200 import dtypes, runtime
from humming_b200.layer import HummingMethod
from humming_b200.utils import synthetic

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_pack_unpack_match_oracle(cuda_device, bits):
    rng = np.random.default_rng(bits)
    codes = rng.integers(0, 1 << bits, size=(64, 256), dtype=np.int64).astype(np.int32)
    packed = runtime.pack_weight(torch.from_numpy(codes).to(cuda_device), bits)
    want = oracle.pack_bits(codes, bits).view(np.int32).reshape(64, -1)
    assert packed.shape == want.shape
    assert np.array_equal(packed.cpu().numpy(), want)
    back = runtime.unpack_weight(packed, bits)
    assert np.array_equal(back.cpu().numpy(), codes)


def test_pack_rejects_ragged_input(cuda_device):
    with pytest.raises(ValueError):
        runtime.pack_weight(torch.zeros((3, 40), dtype=torch.int32, device=cuda_device), 4)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("zp", [False, True])
@pytest.mark.parametrize("n,k,g", [(128, 128, 64), (256, 512, 128), (1024, 1024, 128), (384, 1024, 0)])
def test_prepared_weights_dequantize_bit_exact(cuda_device, dtype, zp, n, k, g):
    """finish_load's layout decoded by the GEMM's own device function equals
    weight_ref rounded once to the activation type, bit for bit."""
    case = synthetic.dense_w4a16_case(n, k, dtype, zp, group_size=g or k, seed=n + k)
    case.group_size = g or k
    layer, _ = build_layer(case)
    meta = layer.meta
    desc = HummingMethod._desc(meta)
    got = runtime.dequant_prepared(desc, layer.weight, layer.weight_scale, getattr(layer, "zero_point", None))
    ref = oracle.effective_weight_16(oracle_weight(case), str(meta.a_dtype))
    assert np.array_equal(got.cpu().numpy().view(np.uint32), ref.view(np.uint32))


def test_signed_int4_equals_offset_uint4(cuda_device):
    case = synthetic.dense_w4a16_case(256, 256, torch.bfloat16, False, seed=3)
    lu, _ = build_layer(case, signed=False)
    ls, _ = build_layer(case, signed=True)
    assert torch.equal(lu.weight, ls.weight)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("m,k", [(1, 64), (5, 1000), (33, 8192)])
def test_quant_input_matches_oracle(cuda_device, dtype, m, k):
    gen = torch.Generator(device="cpu").manual_seed(m * k)
    x = (torch.randn((m, k), generator=gen) * 3).to(dtype)
    if m > 1:
        x[1].zero_()  # all-zero row: scale floor 1e-30/448
    q, s = runtime.quant_input(x.to(cuda_device), "float8e4m3")
    q_ref, s_ref = oracle.quant_input_e4m3(x)
    assert torch.equal(s.cpu(), s_ref)
    # x * (1/scale) may differ from the oracle's by one fp32 ulp before rounding:
    # allow codes one e4m3 step apart on at most a handful of elements.
    a = q.cpu().view(torch.uint8).to(torch.int32)
    b = q_ref.view(torch.uint8).to(torch.int32)
    diff = (a - b).abs()
    assert int(diff.max()) <= 1
    assert int((diff != 0).sum()) <= max(2, a.numel() // 1000)
