"""Nystrom centre selection (falkon/center_selection.py:18-270): uniform sampling without replacement
driven by a numpy generator, and a selector for centres fixed in advance.  With the same seed the
uniform selector picks the same rows as the reference: both call ``Generator.choice(N, size=M,
replace=False)`` on ``numpy.random.default_rng(seed)``."""
import warnings
from abc import ABC, abstractmethod
from typing import Optional, Union

import numpy as np
import torch

__all__ = ("CenterSelector", "FixedSelector", "UniformSelector")


def _as_generator(random_gen) -> np.random.Generator:
    if isinstance(random_gen, np.random.Generator):
        return random_gen
    return np.random.default_rng(random_gen)


class CenterSelector(ABC):
    def __init__(self, random_gen):
        self.random_gen = _as_generator(random_gen)

    @abstractmethod
    def select(self, X, Y):
        ...

    @abstractmethod
    def select_indices(self, X, Y):
        ...


class FixedSelector(CenterSelector):
    """Returns the centres given at construction (and their targets / indices when supplied)."""

    def __init__(self, centers: torch.Tensor, y_centers: Optional[torch.Tensor] = None,
                 idx_centers: Optional[torch.Tensor] = None):
        super().__init__(random_gen=None)
        self.centers = centers
        self.idx_centers = idx_centers
        self.y_centers = y_centers

    def select(self, X, Y):
        if Y is not None:
            if self.y_centers is None:
                raise RuntimeError("FixedSelector has no y-centers available, but `Y` is not None.")
            return self.centers, self.y_centers
        return self.centers

    def select_indices(self, X, Y):
        if self.idx_centers is None:
            raise RuntimeError("`select_indices` method called but no indices were provided.")
        if Y is not None:
            if self.y_centers is None:
                raise RuntimeError("FixedSelector has no y-centers available, but `Y` is not None.")
            return self.centers, self.y_centers, self.idx_centers
        return self.centers, self.idx_centers


class UniformSelector(CenterSelector):
    """Chooses ``num_centers`` rows uniformly at random without replacement."""

    def __init__(self, random_gen: Union[None, int, np.random.Generator], num_centers: int):
        self.num_centers = num_centers
        super().__init__(random_gen)

    def select_indices(self, X, Y):
        N = X.shape[0]
        num_centers = self.num_centers
        if num_centers > N:
            warnings.warn(
                f"Number of centers M greater than the number of data-points. Setting `num_centers` to {N}",
                stacklevel=2,
            )
            num_centers = N
        idx = self.random_gen.choice(N, size=num_centers, replace=False)
        th_idx = torch.from_numpy(idx.astype(np.int64)).to(X.device)
        Xc = torch.index_select(X, 0, th_idx)
        if X.dim() == 2 and X.stride(0) == 1 and X.shape[1] > 1:  # keep column-major inputs column-major
            Xc = Xc.T.contiguous().T
        if Y is not None:
            Yc = torch.index_select(Y, 0, th_idx.to(Y.device))
            return Xc, Yc, th_idx
        return Xc, th_idx

    def select(self, X, Y):
        out = self.select_indices(X, Y)
        if len(out) == 2:
            return out[0]
        return out[0], out[1]
