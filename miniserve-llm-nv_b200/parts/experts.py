"""A feed-forward of routed experts (``routed_experts``).

``experts`` small feed-forward layers without biases, of which every token uses ``top``:

* router logits ``z = W_r h + b`` in float32 (the router's weight and bias are kept in float32);
* the ``top`` experts with the largest logits are chosen (a tie goes to the lower index), and their weights are the
  softmax over the chosen logits alone;
* expert ``e`` computes ``W_down,e act(W_up,e h)``; the output is the weighted sum of the chosen experts' outputs;
* a shared expert of the same form (its own inner size), if any, runs for every token and is added.

``activation``: ``relu_square`` (``act(z) = max(z, 0)^2``), the only one implemented.

Everything happens on the device, so a step never waits for the host to learn the choice and a captured decode
step can hold the layer: the (token, choice) pairs are sorted by expert (``kernels.expert_route``), each expert's
two products run over its segment of rows (``kernels.expert_linear``, the first gathering its rows from the tokens and
applying the activation as it stores), and one kernel adds a token's weighted results and the shared expert's
(``kernels.expert_combine``, float32 sums).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, register_feed_forward
from .context import StepContext


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    def __init__(self, *, prefix: str, hidden_size: int, experts: int, top: int, expert_size: int,
                 shared_size: Optional[int] = None, router_bias: bool = True, activation: str = "relu_square",
                 router_name: str = "router", router_bias_name: str = "router.b", expert_name: str = "e{index}.",
                 shared_name: str = "shared.", up_name: str = "up", down_name: str = "down") -> None:
        if activation != "relu_square":
            raise ValueError(f"routed_experts implements the 'relu_square' activation, not {activation!r}")
        if not 1 <= top <= experts:
            raise ValueError(f"every token uses {top} of {experts} experts: not possible")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.experts, self.top, self.expert_size, self.shared_size = experts, top, expert_size, shared_size
        self.router_bias = bool(router_bias)
        self.names = dict(router=prefix + router_name, bias=prefix + router_bias_name,
                          up=[prefix + expert_name.format(index=e) + up_name for e in range(experts)],
                          down=[prefix + expert_name.format(index=e) + down_name for e in range(experts)],
                          shared_up=prefix + shared_name + up_name, shared_down=prefix + shared_name + down_name)
        self.router_weight: Optional[torch.Tensor] = None    # float32 [E, hidden]
        self.router_b: Optional[torch.Tensor] = None         # float32 [E]
        self.up: Optional[torch.Tensor] = None               # [E, expert_size, hidden]
        self.down: Optional[torch.Tensor] = None             # [E, hidden, expert_size]
        self.shared_up: Optional[torch.Tensor] = None
        self.shared_down: Optional[torch.Tensor] = None

    def param_specs(self) -> list[ParamSpec]:
        h, names = self.hidden_size, self.names
        specs = []
        for e in range(self.experts):
            specs += [ParamSpec(names["up"][e], (self.expert_size, h)), ParamSpec(names["down"][e], (h, self.expert_size))]
        specs.append(ParamSpec(names["router"], (self.experts, h), "matrix_f32"))
        if self.router_bias:
            specs.append(ParamSpec(names["bias"], (self.experts,), "vector"))
        if self.shared_size:
            specs += [ParamSpec(names["shared_up"], (self.shared_size, h)), ParamSpec(names["shared_down"], (h, self.shared_size))]
        return specs

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        names = self.names
        self.router_weight = tensors[names["router"]].float().contiguous()
        self.router_b = tensors[names["bias"]].float().contiguous() if self.router_bias else None
        self.up = torch.stack([tensors[name] for name in names["up"]]).contiguous()
        self.down = torch.stack([tensors[name] for name in names["down"]]).contiguous()
        if self.shared_size:
            self.shared_up, self.shared_down = tensors[names["shared_up"]], tensors[names["shared_down"]]

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        n, top, width = x.shape[0], self.top, self.hidden_size
        pairs = n * top
        ids = ctx.buffer("experts.ids", (n, top), torch.int32)
        weights = ctx.buffer("experts.weights", (n, top), torch.float32)
        logits = ctx.buffer("experts.logits", (n, self.experts), torch.float32)
        kernels.router_topk(x, self.router_weight, self.router_b, top, ids, weights, logits)
        offsets = ctx.buffer("experts.offsets", (self.experts + 1,), torch.int32)
        order = ctx.buffer("experts.order", (pairs,), torch.int32)
        place = ctx.buffer("experts.place", (pairs,), torch.int32)
        kernels.expert_route(ids, self.experts, offsets, order, place)
        hidden = ctx.buffer("experts.hidden", (pairs, self.expert_size), x.dtype)
        kernels.expert_linear(x, order, top, self.up, hidden, offsets, relu_square=True)
        results = ctx.buffer("experts.results", (pairs, width), x.dtype)
        kernels.expert_linear(hidden, None, top, self.down, results, offsets)
        shared = None
        if self.shared_size:
            shared_hidden = ctx.buffer("experts.shared_hidden", (n, self.shared_size), x.dtype)
            kernels.linear(x, self.shared_up, shared_hidden)
            kernels.relu_square(shared_hidden)
            shared = ctx.buffer("experts.shared", (n, width), x.dtype)
            kernels.linear(shared_hidden, self.shared_down, shared)
        out = ctx.buffer("experts.out", (n, width), x.dtype)
        kernels.expert_combine(results, place, weights, shared, out)
        return out
