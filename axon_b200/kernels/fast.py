"""The tuned sm_100a kernels of the bfloat16 path.

Each function returns True when it ran and False when it refuses the sizes or
dtypes, in which case the caller takes the plain kernel.
"""

from __future__ import annotations

from typing import Optional

import torch


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor],
         accumulate: bool) -> bool:
    return False


def gemm_swiglu(h: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor) -> bool:
    return False


def attention(q, kv, ctx, out, heads: int, scale: float) -> bool:
    return False
