"""Stand-alone online rotation y = x @ U on the bf16 tensor cores (tcgen05), with the call
signature of the reference's rotation kernels (speedup/kernels/bf16_rotation.py:35-66,
int8_rotation.py:194-241, fp8_rotation.py) so report scripts can swap it in."""
from __future__ import annotations

import torch

from . import ops


def prepare_U_bf16(U: torch.Tensor):
    """Returns (U_prepared, None).  The prepared tensor is U transposed, contiguous, bf16: the
    K-major operand layout the kernel's TMA descriptor expects."""
    assert U.dim() == 2 and U.shape[0] == U.shape[1]
    return U.t().contiguous().to(torch.bfloat16), None


def bf16_rotation_forward(x: torch.Tensor, U_prepared: torch.Tensor, scale_U=None, *, scale_x=None) -> torch.Tensor:
    """y [M, N] = x [M, K] @ U, bf16.  ``scale_U`` / ``scale_x`` are accepted and ignored, as in the
    reference's bf16 variant."""
    assert x.dim() == 2 and x.dtype == torch.bfloat16
    return ops.rotate(x.contiguous(), U_prepared)
