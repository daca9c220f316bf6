"""Host-side helpers shared by fmmv / fdmmv: contiguity checks and output allocation.

Semantics follow the reference: a tensor is acceptable when one of its strides is 1
(falkon/mmv_ops/utils.py:36-39, falkon/utils/tensor_helpers.py:210-213); a missing ``out`` is
created on the first CUDA input's device, else on the CPU (pinned), with the memory order of X1
(falkon/mmv_ops/utils.py:124-155, falkon/utils/tensor_helpers.py:128-141).
"""
from typing import Optional, Sequence, Tuple

import torch

__all__ = ("is_contig", "is_f_contig", "check_contiguity", "create_output_mat", "create_same_stride")


def is_contig(tensor: torch.Tensor) -> bool:
    return any(s == 1 for s in tensor.stride())


def is_f_contig(tensor: torch.Tensor, strict: bool = False) -> bool:
    """Column-major test with the reference's treatment of degenerate shapes
    (falkon/utils/tensor_helpers.py:164-207)."""
    strides, sizes = tensor.stride(), tensor.shape
    if len(sizes) == 0:
        return True
    if len(sizes) == 1:
        return strides[0] == 1
    if sizes[-2] == 1:
        if strict:
            return strides[-2] == 1
        return strides[-1] == 1 or strides[-2] == 1
    if sizes[-1] == 1:
        if strict:
            return strides[-2] == 1 and strides[-1] >= sizes[-2]
        return strides[-2] == 1
    return strides[-2] == 1 and strides[-1] >= strides[-2]


def check_contiguity(*named: Tuple[Optional[torch.Tensor], str]) -> None:
    for tensor, name in named:
        if tensor is not None and not is_contig(tensor):
            raise ValueError(f"Tensor '{name}' must be memory contiguous")


def create_same_stride(shape, other: torch.Tensor, dtype, device, pin_memory: bool = False) -> torch.Tensor:
    """Empty 2-D tensor in Fortran order if ``other`` is (strictly) column-major, else C order."""
    pin = pin_memory and torch.device(device).type == "cpu" and torch.cuda.is_available()
    if is_f_contig(other, strict=True):
        return torch.empty_strided(shape, (1, shape[0]), dtype=dtype, device=device, pin_memory=pin)
    if is_contig(other):
        return torch.empty(shape, dtype=dtype, device=device, pin_memory=pin)
    raise ValueError("Desired stride is not contiguous, cannot create.")


def create_output_mat(
    out: Optional[torch.Tensor],
    data_devs: Sequence[torch.device],
    shape: Tuple[int, int],
    dtype: torch.dtype,
    comp_dev_type: str,
    other_mat: torch.Tensor,
) -> torch.Tensor:
    if out is not None:
        return out
    out_dev = torch.device("cpu")
    for ddev in data_devs:
        if ddev.type == "cuda":
            out_dev = ddev
            break
    return create_same_stride(
        shape, other_mat, dtype, device=out_dev, pin_memory=out_dev.type != "cuda" and comp_dev_type == "cuda"
    )
