"""Random test-data generators with the reference's names and return tuples
(``humming/utils/test.py``): quantized weights with their fp32 ``weight_ref``,
activations with ``inputs_ref``, biases and MoE routing tensors.

Only the cases this library builds are generated (integer weights, 16-bit or
e4m3 activations); the rest raise ``NotImplementedError``.
"""
import math

import torch

from humming_b200 import dtypes
from humming_b200 import runtime
from humming_b200.utils.weight import quantize_weight

DEVICE = "cuda:0"


def generate_random_inputs(m: int, k: int, group_size: int = 0, dtype: dtypes.DataType = dtypes.float32):
    """-> (inputs_orig fp32, inputs_ref fp32, inputs, input_scale)
    (``humming/utils/test.py:9-66``)."""
    dtype = dtypes.DataType.from_str(dtype)
    g = group_size if group_size > 0 else k
    assert k % g == 0
    torch.randn((m, k // g), dtype=torch.float32, device=DEVICE)  # the reference draws (and drops) this first: same seed, same data
    x = torch.randn((m, k), dtype=torch.float32, device=DEVICE)
    x = x * torch.rand((m, k // g), dtype=torch.float32, device=DEVICE).repeat_interleave(g, 1)
    x = x / x.std()
    if dtype in (dtypes.float16, dtypes.bfloat16):
        inputs = x.to(dtypes.torch_dtype_map[dtype])
        return x, inputs.float(), inputs, None
    if dtype == dtypes.float8e4m3 and g == k:
        q, scale = runtime.quant_input(x, "float8e4m3")
        return x, q.float() * scale, q, scale
    raise NotImplementedError(f"inputs of type {dtype} with group size {group_size} are not built")


def generate_random_weight(n, k, group_size, dtype, scale_dtype, num_experts=None, has_global_scale=False,
                           has_dynamic_zp=False):
    """-> (weight_orig, weight_ref, quanted_weight, weight_scale, zero_point, global_scale)
    (``humming/utils/test.py:69-144``).  ``weight_ref`` is the fp32 oracle
    ``(q - zp) * scale``; ``quanted_weight`` holds int32 codes (two's complement
    values for signed dtypes)."""
    dtype = dtypes.DataType.from_str(dtype)
    e = 1 if num_experts is None else num_experts
    g = group_size if group_size > 0 else k
    if has_dynamic_zp:
        assert dtype.is_integer_type and not dtype.is_signed, "dynamic zero point only supports for uint dtype"
    if not dtype.is_integer_type:
        raise NotImplementedError(f"random weights of type {dtype} are not built")
    q_dtype = dtypes.InergerType(False, dtype.num_bits)

    w = torch.randn((e, n, k), dtype=torch.float32, device=DEVICE)
    spread = torch.rand((e, n, k // g), dtype=torch.float32, device=DEVICE) + 0.01
    shift = torch.randn((e, n, k // g), dtype=torch.float32, device=DEVICE)
    w = (w + shift.repeat_interleave(g, -1)) * spread.repeat_interleave(g, -1)
    w = w / w.std()

    q, scale, zp, gs = quantize_weight(w, dtype=q_dtype, scale_dtype=scale_dtype, group_size=g,
                                       has_dynamic_zp=has_dynamic_zp, has_global_scale=has_global_scale)
    if has_dynamic_zp:
        ref = q.float() - zp.repeat_interleave(g, -1)
    else:
        ref = q.float() - 2 ** (dtype.num_bits - 1)
    ref = ref * scale.float().repeat_interleave(g, -1)
    if dtype.is_signed:
        q = q - 2 ** (dtype.num_bits - 1)
    if num_experts is None:
        w, ref, q, scale = w.squeeze(0), ref.squeeze(0), q.squeeze(0), scale.squeeze(0)
        zp = zp.squeeze(0) if zp is not None else None
    return w, ref, q, scale, zp, gs


def generate_random_bias(n, dtype):
    dtype = dtypes.DataType.from_str(dtype)
    assert dtype in (dtypes.float16, dtypes.bfloat16)
    return torch.randn((n,), dtype=dtypes.torch_dtype_map[dtype], device=DEVICE)


def generate_random_moe_tensors(m, num_experts, topk, block_size):
    """Random routing + block-aligned token order
    (``humming/utils/test.py:154-183``): returns ``(topk_ids, topk_weights,
    sorted_token_ids, expert_ids, num_tokens_post_padded)`` where
    ``sorted_token_ids`` lists flat (token, slot) ids grouped by expert and padded
    per expert to a multiple of ``block_size`` with the sentinel ``m * topk``."""
    logits = torch.randn((m, num_experts), dtype=torch.float32, device=DEVICE)
    topk_weights, topk_ids = logits.topk(topk, 1)
    topk_ids = topk_ids.int()
    flat = topk_ids.view(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    blocks = (counts + block_size - 1) // block_size
    padded = blocks * block_size
    starts = torch.cumsum(padded, 0) - padded
    total = int(padded.sum())
    sorted_token_ids = torch.full((total,), flat.numel(), dtype=torch.int32, device=DEVICE)
    src_starts = torch.cumsum(counts, 0) - counts
    expert_of = flat[order]
    pos = torch.arange(flat.numel(), device=DEVICE) - src_starts[expert_of] + starts[expert_of]
    sorted_token_ids[pos] = order.int()
    expert_ids = torch.repeat_interleave(torch.arange(num_experts, device=DEVICE, dtype=torch.int32), blocks)
    num_tokens_post_padded = torch.tensor(total, dtype=torch.int32, device=DEVICE)
    return topk_ids, topk_weights, sorted_token_ids, expert_ids, num_tokens_post_padded
