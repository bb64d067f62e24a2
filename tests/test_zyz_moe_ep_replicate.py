"""The replicated-token expert-parallel mode (all-gather, local experts only, reduce-scatter) on two GPUs over NCCL
against the single-process CPU reference; the ranks hold different token counts and pad to the larger one.  Skipped
where fewer than two GPUs are visible."""
import os

import pytest
import torch
import torch.multiprocessing as mp

from test_gpu_moe_ep import _free_port, _worker

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_replicated_expert_parallel_moe_two_gpus(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), "replicate"), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
