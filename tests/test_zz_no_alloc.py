"""hm_gemm_static_scratch: the GEMM entry point for callers that cannot allocate.

Some callers of this library have no way to obtain device memory at call time:
a serving loop whose memory pool is frozen after warm-up, or a plugin that a host
engine hands fixed buffers and no allocator.  For them the library carries an
8 MiB scratch array inside its own device image.  This test drives that entry
point straight through the C ABI and checks it against the regular hm_gemm
path (which uses a caller-owned workspace) on two calls in a row, because the
second call finds the array dirty from the first.

The file name makes pytest collect it last, so a run that stops at the first
failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

from helpers import ATOL_16, RTOL_16, build_layer
from humming_b200 import native
from humming_b200.layer import HummingMethod
from humming_b200.utils import synthetic

pytestmark = pytest.mark.gpu


def _call_static(layer, desc, x, out):
    stream = ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    return native.lib.hm_gemm_static_scratch(
        ctypes.byref(desc), x.size(0), ptr(x), x.stride(0), None, ptr(layer.weight), ptr(layer.weight_scale),
        ptr(getattr(layer, "zero_point", None)), None, ptr(out), out.stride(0), stream)


def test_static_scratch_matches_workspace_path_twice(cuda_device):
    # 4096 x 4096 at 16 rows: 32 tiles spread over all SMs, so every tile's K range
    # is split and the scratch (counters + fp32 partial sums) really is used.
    case = synthetic.dense_w4a16_case(4096, 4096, torch.bfloat16, True, seed=31)
    layer, _ = build_layer(case)
    desc = HummingMethod._desc(layer.meta)
    plan = native.Plan()
    native.check(native.lib.hm_gemm_plan(ctypes.byref(desc), 16, ctypes.byref(plan)))
    assert plan.mode == 1 and 0 < plan.workspace_bytes <= native.HM_STATIC_SCRATCH_BYTES

    x1 = synthetic.activations(16, 4096, torch.bfloat16, seed=41).to(cuda_device)
    x2 = synthetic.activations(16, 4096, torch.bfloat16, seed=42).to(cuda_device)
    want1 = layer(inputs=x1).clone()   # regular entry point, caller-owned workspace
    want2 = layer(inputs=x2).clone()
    layer.check_status()

    got1 = torch.empty_like(want1)
    got2 = torch.empty_like(want2)
    native.check(_call_static(layer, desc, x1, got1))
    native.check(_call_static(layer, desc, x2, got2))   # second call: scratch holds call one's leftovers
    torch.cuda.synchronize()
    torch.testing.assert_close(got1.float(), want1.float(), atol=ATOL_16, rtol=RTOL_16)
    torch.testing.assert_close(got2.float(), want2.float(), atol=ATOL_16, rtol=RTOL_16)
    assert not torch.equal(got1, got2)

    # A different, smaller shape right after: its counter region overlaps what the
    # previous shape used for partial sums, and must have been cleared.
    small = synthetic.dense_w4a16_case(1024, 1024, torch.bfloat16, True, seed=32)
    layer_s, _ = build_layer(small)
    desc_s = HummingMethod._desc(layer_s.meta)
    xs = synthetic.activations(7, 1024, torch.bfloat16, seed=43).to(cuda_device)
    want_s = layer_s(inputs=xs).clone()
    got_s = torch.empty_like(want_s)
    native.check(_call_static(layer_s, desc_s, xs, got_s))
    torch.cuda.synchronize()
    torch.testing.assert_close(got_s.float(), want_s.float(), atol=ATOL_16, rtol=RTOL_16)


def test_static_scratch_serves_the_decode_kernels(cuda_device):
    """One and three tokens are planned for the decode kernels (mode 2), whose counters and partial sums
    live in the same array; twice in a row, after a tensor-core call has left its own data there."""
    case = synthetic.dense_w4a16_case(1024, 4096, torch.bfloat16, True, seed=33)
    layer, _ = build_layer(case)
    desc = HummingMethod._desc(layer.meta)
    x16 = synthetic.activations(16, 4096, torch.bfloat16, seed=44).to(cuda_device)
    native.check(_call_static(layer, desc, x16, torch.empty((16, 1024), dtype=torch.bfloat16, device=cuda_device)))
    for m in (1, 3):
        plan = native.Plan()
        native.check(native.lib.hm_gemm_plan(ctypes.byref(desc), m, ctypes.byref(plan)))
        assert plan.mode == 2 and plan.workspace_bytes <= native.HM_STATIC_SCRATCH_BYTES
        x = synthetic.activations(m, 4096, torch.bfloat16, seed=45 + m).to(cuda_device)
        want = layer(inputs=x).clone()
        for _ in range(2):
            got = torch.empty_like(want)
            native.check(_call_static(layer, desc, x, got))
            torch.cuda.synchronize()
            assert torch.equal(got, want)
    layer.check_status()


def test_static_scratch_refuses_shapes_beyond_its_size(cuda_device):
    # a long K with few tiles: planned as a K split whose partial tiles exceed the static array
    case = synthetic.dense_w4a16_case(2048, 8192, torch.bfloat16, True, seed=31)
    layer, _ = build_layer(case)
    desc = HummingMethod._desc(layer.meta)
    x = synthetic.activations(256, 8192, torch.bfloat16).to(cuda_device)
    out = torch.empty((256, 2048), dtype=torch.bfloat16, device=cuda_device)
    plan = native.Plan()
    native.check(native.lib.hm_gemm_plan(ctypes.byref(desc), 256, ctypes.byref(plan)))
    assert plan.workspace_bytes > native.HM_STATIC_SCRATCH_BYTES
    rc = _call_static(layer, desc, x, out)
    assert rc == native.HM_ERR_WORKSPACE
    msg = native.last_error()
    assert str(plan.workspace_bytes) in msg and str(native.HM_STATIC_SCRATCH_BYTES) in msg
