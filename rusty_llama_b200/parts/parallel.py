"""A mixer made of several mixers that read the same input side by side."""

from __future__ import annotations

from typing import Mapping

import torch

from ..errors import ConfigError
from ..kernels.linear import linear_to_stream
from ..spec import PartSpec
from .base import MIXERS, Mixer


@MIXERS.register("parallel")
class ParallelMixers(Mixer):
    """result = sum_i scale_i * branch_i(xn).

    Every branch is a mixer that ends in a projection and can leave it to the caller (`forward_unprojected`).  The branches
    write what their projections would read into one row, side by side, and ONE product with the projections' matrices side
    by side makes the sum: no branch's result is stored or added on its own.  A branch's scale is handed to it as its
    `out_scale`, so it is applied in 32-bit where the branch forms its last values; biases of the branches' projections
    are summed into one row (`output_bias`).  Each branch keeps the cache storage it asks for; this mixer's need is the
    tuple of theirs.

    params: branches: a list of (PartSpec, scale); a branch's prefix is relative to this mixer's."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        branches = self._param("branches")
        if not branches:
            raise ConfigError("parallel: no branches")
        self.branches = []
        for b, scale in branches:
            if not isinstance(b, PartSpec):
                raise ConfigError("parallel: a branch must be a PartSpec")
            cls = MIXERS.get(b.kind)
            if not getattr(cls, "takes_out", False):
                raise ConfigError(f"parallel: mixer '{b.kind}' cannot leave its last projection to the caller")
            params = dict(b.params)
            params["out_scale"] = float(params.get("out_scale", 1.0)) * float(scale)
            self.branches.append(MIXERS.build(PartSpec(b.kind, params, self.prefix + b.prefix), runtime))
        self._needs = [b.cache_need() for b in self.branches]
        self.w_o = None
        self.bias = None

    def children(self):
        return tuple(self.branches)

    def cache_need(self):
        needs = tuple(n for n in self._needs if n is not None)
        return needs or None

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        # children are loaded by the model after this part; their matrices are put side by side at the first step
        self.w_o = None

    def output_bias(self):
        return self.bias

    def _assemble(self) -> None:
        self.w_o = torch.cat([b.w_o for b in self.branches], dim=1).contiguous()
        rows = [b.output_bias() for b in self.branches]
        rows = [r for r in rows if r is not None]
        self.bias = None if not rows else torch.stack(rows).sum(dim=0).contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        if shared_cache:
            raise ConfigError("parallel: its branches fill caches of their own")
        if self.w_o is None:
            self._assemble()
        views = list(cache) if isinstance(cache, (tuple, list)) else [cache]
        T = xn.shape[0]
        a = torch.empty((T, self.w_o.shape[1]), dtype=xn.dtype, device=xn.device)
        at = 0
        for b, need in zip(self.branches, self._needs):
            k = b.w_o.shape[1]
            b.forward_unprojected(xn, step, views.pop(0) if need is not None else None, False, out=a[:, at : at + k])
            at += k
        return linear_to_stream(a, self.w_o)
