"""The random test-data generators (``humming_b200.utils.test``, names and return tuples of the reference's
``humming/utils/test.py``) run on the CPU with the reference's seeds: they draw in the reference's order, so every
tensor they return equals, bit for bit, what the reference's own generators returned when the fixtures were made."""
import os

import numpy as np
import pytest
import torch

from humming_b200.utils import test as gen

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
RANDOM_WEIGHT_CASES = [("uint4", "float16", 128, False, None), ("uint4", "bfloat16", 128, True, None),
                       ("int4", "bfloat16", 128, False, 2), ("uint8", "float16", 128, True, None),
                       ("uint4", "bfloat16", 32, True, 3), ("int8", "float16", 128, False, None)]


@pytest.fixture(autouse=True)
def on_cpu(monkeypatch):
    monkeypatch.setattr(gen, "DEVICE", "cpu")


@pytest.mark.parametrize("i", range(len(RANDOM_WEIGHT_CASES)))
def test_generate_random_weight_reproduces_the_reference(i):
    b, s, group, zp, experts = RANDOM_WEIGHT_CASES[i]
    g = np.load(os.path.join(GOLD, "random_weight.npz"))
    torch.manual_seed(500 + i)
    w_orig, w_ref, q, scale, zero_point, gs = gen.generate_random_weight(8, 256, group, b, s, num_experts=experts, has_dynamic_zp=zp)
    assert gs is None
    assert np.array_equal(w_orig.numpy().view(np.uint32), g[f"c{i}_weight_orig"].view(np.uint32))
    assert np.array_equal(q.numpy(), g[f"c{i}_codes"])
    assert np.array_equal(scale.view(torch.int16).numpy(), g[f"c{i}_scale_bits"])
    assert np.array_equal(w_ref.numpy().view(np.uint32), g[f"c{i}_weight_ref"].view(np.uint32))
    if zp:
        assert np.array_equal(zero_point.numpy(), g[f"c{i}_zero_point"])
    else:
        assert zero_point is None


def test_generate_random_moe_tensors_reproduces_the_reference():
    g = np.load(os.path.join(GOLD, "moe_align.npz"))
    for i in range(5):
        m, e, k, blk = (int(v) for v in g[f"c{i}_shape"])
        torch.manual_seed(100 + i)
        topk_ids, topk_w, sorted_ids, expert_ids, total = gen.generate_random_moe_tensors(m, e, k, blk)
        assert np.array_equal(topk_ids.numpy(), g[f"c{i}_topk_ids"])
        assert np.array_equal(sorted_ids.numpy(), g[f"c{i}_sorted_token_ids"])
        assert np.array_equal(expert_ids.numpy(), g[f"c{i}_expert_ids"])
        assert int(total) == int(g[f"c{i}_num_tokens_post_padded"])
        assert topk_w.shape == (m, k) and topk_ids.dtype == sorted_ids.dtype == expert_ids.dtype == torch.int32


def test_generate_random_inputs_reproduces_the_reference():
    g = np.load(os.path.join(GOLD, "random_inputs.npz"))
    for i, (m, k, group, name) in enumerate([(5, 256, 0, "float16"), (3, 512, 128, "bfloat16")]):
        torch.manual_seed(700 + i)
        x_orig, x_ref, x, x_scale = gen.generate_random_inputs(m, k, group, name)
        assert x_scale is None
        assert np.array_equal(x_orig.numpy().view(np.uint32), g[f"c{i}_orig"].view(np.uint32))
        assert np.array_equal(x.view(torch.int16).numpy(), g[f"c{i}_bits"])
        assert np.array_equal(x_ref.numpy().view(np.uint32), g[f"c{i}_ref"].view(np.uint32))
    with pytest.raises(NotImplementedError):
        gen.generate_random_inputs(4, 256, 0, "int8")


def test_generate_random_bias():
    b = gen.generate_random_bias(64, "bfloat16")
    assert b.shape == (64,) and b.dtype == torch.bfloat16
    with pytest.raises(AssertionError):
        gen.generate_random_bias(64, "float32")
