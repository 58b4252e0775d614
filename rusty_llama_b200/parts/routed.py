"""A feed-forward that sends each token to a few of many small gated feed-forwards."""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.linear import linear, linear_swiglu
from .base import FEED_FORWARDS, FeedForward, ParamInfo

_NAMES = {
    "expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "router": "router", "bias": "correction",
    "shared": "shared.", "shared_gate": "shared.sg",
}


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """E experts f_e(x) = W_down[e] (silu(W_gate[e] x) * (W_up[e] x)); every token uses `top` of them.

        s = softmax(W_r x) over all experts, in 32-bit
        chosen = the `top` experts with the largest s + bias (the bias only chooses)
        y = sum over chosen e of s_e f_e(x)            (s_e / sum of the chosen s if `renormalize`)
          + sigmoid(w_sg . x) * f_shared(x)            (if there is a shared expert; without w_sg it is added as it is)

    params: hidden_size, n_experts, top, expert_ff, bias (bool), renormalize (bool),
            shared_ff (0: none), shared_gate (bool), names (optional).
    tensors: <prefix>e<i>.gate [ff, d], e<i>.up [ff, d], e<i>.down [d, ff], router [E, d], correction [E],
             shared.gate / shared.up / shared.down, shared.sg [1, d]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.E = int(self._param("n_experts"))
        self.top = int(self._param("top"))
        self.ff = int(self._param("expert_ff"))
        self.has_bias = bool(spec.params.get("bias", False))
        self.renormalize = bool(spec.params.get("renormalize", False))
        self.shared_ff = int(spec.params.get("shared_ff", 0))
        self.shared_gate = bool(spec.params.get("shared_gate", False)) and self.shared_ff > 0
        self.names = dict(_NAMES, **dict(spec.params.get("names", {})))
        if not 0 < self.top <= self.E:
            raise ConfigError(f"routed_experts: {self.top} of {self.E} experts per token")
        if self.ff <= 0:
            raise ConfigError(f"routed_experts: expert size {self.ff}")

    def _expert(self, i: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(i) + self.names[which]

    def _shared(self, which: str) -> str:
        return self.prefix + self.names["shared"] + self.names[which]

    def param_infos(self) -> Dict[str, ParamInfo]:
        infos = {}
        for i in range(self.E):
            infos[self._expert(i, "gate")] = ParamInfo((self.ff, self.d))
            infos[self._expert(i, "up")] = ParamInfo((self.ff, self.d))
            infos[self._expert(i, "down")] = ParamInfo((self.d, self.ff))
        infos[self.prefix + self.names["router"]] = ParamInfo((self.E, self.d), "scalars")
        if self.has_bias:
            infos[self.prefix + self.names["bias"]] = ParamInfo((self.E,), "scalars")
        if self.shared_ff:
            infos[self._shared("gate")] = ParamInfo((self.shared_ff, self.d))
            infos[self._shared("up")] = ParamInfo((self.shared_ff, self.d))
            infos[self._shared("down")] = ParamInfo((self.d, self.shared_ff))
        if self.shared_gate:
            infos[self.prefix + self.names["shared_gate"]] = ParamInfo((1, self.d), "scalars")
        return infos

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        stack = lambda which: torch.stack([tensors[self._expert(i, which)] for i in range(self.E)], dim=0).contiguous()  # noqa: E731
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        rows = [tensors[self.prefix + self.names["router"]]]
        if self.shared_gate:
            rows.append(tensors[self.prefix + self.names["shared_gate"]])  # one more row of the router's product
        self.w_router = torch.cat(rows, dim=0).contiguous()
        self.bias = tensors[self.prefix + self.names["bias"]].contiguous() if self.has_bias else None
        if self.shared_ff:
            gate, up = tensors[self._shared("gate")], tensors[self._shared("up")]
            self.shared_fused = self.rt.dtype == torch.bfloat16
            if self.shared_fused:  # gate and up rows alternate: the product's kernel applies the activation (see GatedMLP)
                self.ws_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.shared_ff, self.d).contiguous()
            else:
                self.ws_gate_up = torch.cat([gate, up], dim=0).contiguous()
            self.ws_down = tensors[self._shared("down")].contiguous()

    def forward(self, xn: torch.Tensor, step) -> torch.Tensor:
        T = xn.shape[0]
        ids, weights, gate = ops.moe_router(xn, self.w_router, self.bias, self.E, self.top, self.renormalize)
        # the height of a row tile: 128 once the experts get that many rows on average (a prompt step), else 32; the plain
        # kernels of a 32-bit run have their own
        tile_rows = 0
        if xn.dtype == torch.bfloat16 and self.d % 8 == 0 and self.ff % 8 == 0:  # (else the plain products, 16-byte rows or not)
            tile_rows = 128 if T * self.top >= 64 * self.E else 32
        order, place, tiles, max_tiles = ops.moe_plan(ids, self.E, tile_rows)
        h = ops.moe_gemm(xn, self.w_gate, tiles, max_tiles, T * self.top, order=order, gather_div=self.top, w2=self.w_up, tile_rows=tile_rows)
        y = ops.moe_gemm(h, self.w_down, tiles, max_tiles, T * self.top, out_dtype=torch.float32, tile_rows=tile_rows)
        shared = None
        if self.shared_ff:
            hs = linear_swiglu(xn, self.ws_gate_up) if self.shared_fused else ops.swiglu(linear(xn, self.ws_gate_up))
            shared = linear(hs, self.ws_down)
        return ops.moe_combine(y, place, weights, shared, gate)
