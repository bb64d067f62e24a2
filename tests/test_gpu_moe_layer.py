"""GPU parity of the whole MoE layer (routing, alignment, both GEMMs, SiLU*mul,
sum over top-k) against a CPU reference with the same rounding points."""
import pytest
import torch

from humming_b200 import runtime
from humming_b200.moe import HummingMoE
from moe_common import make_expert_weights, moe_layer_reference

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,experts,top_k", [(1, 8, 2), (33, 16, 4), (257, 128, 8)])
def test_route_matches_torch(cuda_device, tokens, experts, top_k):
    gen = torch.Generator(device="cpu").manual_seed(tokens)
    logits = torch.randn((tokens, experts), generator=gen)
    ids, w = runtime.moe_route(logits.to(cuda_device), top_k)
    pw, pid = torch.softmax(logits, -1).topk(top_k, 1)
    pw = pw / pw.sum(-1, keepdim=True)
    assert torch.equal(ids.cpu().long(), pid)
    torch.testing.assert_close(w.cpu(), pw, rtol=1e-4, atol=1e-6)
    ids2, w2 = runtime.moe_route(logits.to(cuda_device), top_k, use_softmax=False, renormalize=False)
    rw, rid = logits.topk(top_k, 1)
    assert torch.equal(ids2.cpu().long(), rid) and torch.equal(w2.cpu(), rw)


def test_silu_mul_and_topk_sum(cuda_device):
    gen = torch.Generator(device="cpu").manual_seed(1)
    x = torch.randn((37, 2 * 96), generator=gen).bfloat16()
    got = runtime.silu_mul(x.to(cuda_device)).cpu()
    want = (torch.nn.functional.silu(x[:, :96].float()) * x[:, 96:].float()).bfloat16()
    torch.testing.assert_close(got.float(), want.float(), rtol=1e-2, atol=1e-2)
    y = torch.randn((19, 8, 64), generator=gen).bfloat16()
    assert torch.equal(runtime.topk_sum(y.to(cuda_device)).cpu(), y.float().sum(1).bfloat16())


@pytest.mark.parametrize("tokens", [1, 32, 300])
def test_moe_layer_single_gpu(cuda_device, tokens):
    experts, top_k, hidden, inter = 16, 4, 512, 256
    weights = make_expert_weights(experts, hidden, inter, seed=3)
    moe = HummingMoE(hidden, inter, experts, top_k).to(cuda_device)
    for e in range(experts):
        moe.load_expert(e, weights[0][e].to(cuda_device), weights[1][e].to(cuda_device), weights[2][e].to(cuda_device),
                        weights[3][e].to(cuda_device))
    moe.finish_load()
    gen = torch.Generator(device="cpu").manual_seed(tokens)
    x = torch.randn((tokens, hidden), generator=gen).bfloat16()
    logits = torch.randn((tokens, experts), generator=gen)
    out = moe(x.to(cuda_device), logits.to(cuda_device))
    moe.check_status()
    ref, _, _ = moe_layer_reference(x, logits, weights, top_k)
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=0.05, atol=0.1)


@pytest.mark.parametrize("tokens", [5, 200])
def test_moe_layer_w4a8(cuda_device, tokens):
    """int4 weights, e4m3 activations with per-token scales re-quantized between the two GEMMs."""
    experts, top_k, hidden, inter = 8, 2, 512, 256
    weights = make_expert_weights(experts, hidden, inter, seed=5)
    moe = HummingMoE(hidden, inter, experts, top_k, b_dtype="int4", a_dtype="float8e4m3").to(cuda_device)
    for e in range(experts):
        moe.load_expert(e, (weights[0][e] - 8).to(cuda_device), weights[1][e].to(cuda_device), (weights[2][e] - 8).to(cuda_device),
                        weights[3][e].to(cuda_device))
    moe.finish_load()
    gen = torch.Generator(device="cpu").manual_seed(tokens)
    x = torch.randn((tokens, hidden), generator=gen).bfloat16()
    logits = torch.randn((tokens, experts), generator=gen)
    out = moe(x.to(cuda_device), logits.to(cuda_device))
    moe.check_status()
    ref, _, _ = moe_layer_reference(x, logits, weights, top_k, fp8=True)
    torch.testing.assert_close(out.float().cpu(), ref.float(), rtol=0.05, atol=0.1)
