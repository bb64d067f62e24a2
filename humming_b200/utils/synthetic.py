"""Seeded synthetic tensors with the shapes and value distributions of the
benchmark configurations (no checkpoints or datasets are involved; model names
only fix shapes).  Used by the tests, ``bench.py`` and ``smoke()``; generated on
CPU with a fixed seed so that GPU and CPU sides see identical values.
"""
import dataclasses
from typing import Optional

import torch

# (N, K) of the Llama-3-8B-shaped dense projections.
LLAMA3_8B_SHAPES = {
    "qkv": (6144, 4096),
    "o": (4096, 4096),
    "gate_up": (28672, 4096),
    "down": (4096, 14336),
}


@dataclasses.dataclass
class DenseW4A16Case:
    n: int
    k: int
    group_size: int
    dtype: torch.dtype            # activation / scale / output type
    codes: torch.Tensor           # (N, K) int32 in [0, 15]
    scales: torch.Tensor          # (N, K/g) in `dtype`
    zero_points: Optional[torch.Tensor]  # (N, K/g) int32 in [0, 15] or None (implicit 8)

    def weight_ref(self) -> torch.Tensor:
        """fp32 ``(q - zp) * s`` (reference humming/utils/test.py:109-128)."""
        g = self.group_size
        w = self.codes.float()
        if self.zero_points is not None:
            w = w - self.zero_points.float().repeat_interleave(g, -1)
        else:
            w = w - 8.0
        return w * self.scales.float().repeat_interleave(g, -1)


def dense_w4a16_case(n: int, k: int, dtype: torch.dtype, dynamic_zp: bool, group_size: int = 128,
                     seed: int = 0) -> DenseW4A16Case:
    """uint4 codes uniform in [0, 15]; scales |N(0,1)| * 0.02 + 1e-3 in `dtype`;
    zero-point codes uniform in [0, 15] when ``dynamic_zp``."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    codes = torch.randint(0, 16, (n, k), generator=gen, dtype=torch.int32)
    scales = (torch.randn((n, k // group_size), generator=gen).abs() * 0.02 + 1e-3).to(dtype)
    zps = torch.randint(0, 16, (n, k // group_size), generator=gen, dtype=torch.int32) if dynamic_zp else None
    return DenseW4A16Case(n, k, group_size, dtype, codes, scales, zps)


def activations(m: int, k: int, dtype: torch.dtype, seed: int = 1) -> torch.Tensor:
    """N(0,1) activations in `dtype`."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn((m, k), generator=gen).to(dtype)
