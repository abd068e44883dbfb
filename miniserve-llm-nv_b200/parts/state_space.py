"""The selective state-space mixer (``state_space``): a linear recurrence per head whose decay, input and output maps
depend on the token, in the form known as Mamba-2.

With ``h`` the mixer's input, ``H`` heads of ``P`` channels, a state of ``N`` numbers per channel and ``G`` groups
(head ``k`` uses group ``k // (H / G)``), ``inner = H * P``:

* ``W_in h`` is laid out as ``[z: inner | x: inner | B: G*N | C: G*N | dt: H]`` (one product; zero rows pad the weight
  to a multiple of eight rows).
* ``x``, ``B`` and ``C`` together pass a causal convolution per channel (``taps`` taps with a bias; the last tap is the
  current token's) and SiLU.
* ``dt = softplus(dt + dt_bias)``; per head ``S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T`` (``S`` is ``N x P``)
  and ``y_t = S_t^T C_t + D x_t``.
* ``y`` (heads concatenated) is multiplied by ``silu(z)``, divided by its root mean square in ``norm_groups`` equal
  parts, multiplied by a weight, and ``W_o`` maps it back.

What a request carries from token to token is one float32 vector per layer (:class:`~.base.StateNeed`, zero at
admission): the last ``taps - 1`` inputs of the convolution, then the states of all heads.  Decay, step size, the
recurrence, its output and the gated norm are float32 whatever the compute type; the projections are in the compute
type.  Prompt portions, single tokens and mixed batches run the same three kernels
(``kernels.causal_conv_silu``, ``kernels.selective_scan``, ``kernels.gated_group_norm``), which walk each request's
tokens in order from the state its slot holds.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import ParamSpec, Part, StateNeed, register_mixer
from .context import StateView, StepContext


@register_mixer("state_space")
class StateSpace(Part):
    def __init__(self, *, prefix: str, hidden_size: int, heads: int, head_dim: int, state: int, groups: int, taps: int,
                 norm_groups: int, eps: float, in_name: str = "in", conv_name: str = "conv", conv_bias_name: str = "conv.b",
                 dt_bias_name: str = "dt_bias", a_log_name: str = "A_log", d_name: str = "D", norm_name: str = "norm",
                 o_name: str = "o") -> None:
        if min(hidden_size, heads, head_dim, state, groups, taps, norm_groups) < 1:
            raise ValueError("state_space: every size must be positive")
        if heads % groups or (heads * head_dim) % norm_groups:
            raise ValueError(f"state_space: {heads} heads in {groups} groups, {heads * head_dim} channels in {norm_groups} norm groups")
        if state > kernels.MAX_SCAN_STATE:
            raise ValueError(f"state_space: a state of {state} numbers per channel exceeds {kernels.MAX_SCAN_STATE}")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.heads, self.head_dim, self.state, self.groups, self.taps = heads, head_dim, state, groups, taps
        self.norm_groups, self.eps = norm_groups, float(eps)
        self.inner = heads * head_dim
        self.conv_channels = self.inner + 2 * groups * state
        self.z_col, self.conv_col, self.dt_col = 0, self.inner, self.inner + self.conv_channels
        rows = self.dt_col + heads
        self.in_rows = (rows + 7) // 8 * 8
        self.conv_state = (taps - 1) * self.conv_channels      # the request's vector: [conv inputs | head states]
        self.names = dict(inp=prefix + in_name, conv=prefix + conv_name, conv_b=prefix + conv_bias_name,
                          dt_bias=prefix + dt_bias_name, a_log=prefix + a_log_name, d=prefix + d_name,
                          norm=prefix + norm_name, o=prefix + o_name)
        self.in_weight: Optional[torch.Tensor] = None
        self.conv_weight = self.conv_bias = self.dt_bias = self.a_log = self.d = self.norm_weight = None
        self.o_weight: Optional[torch.Tensor] = None

    def param_specs(self) -> list[ParamSpec]:
        names, h = self.names, self.hidden_size
        return [ParamSpec(names["inp"], (self.dt_col + self.heads, h)),
                ParamSpec(names["conv"], (self.conv_channels, self.taps)),
                ParamSpec(names["conv_b"], (self.conv_channels,), "vector"),
                ParamSpec(names["dt_bias"], (self.heads,), "vector"),
                ParamSpec(names["a_log"], (self.heads,), "vector"),
                ParamSpec(names["d"], (self.heads,), "vector"),
                ParamSpec(names["norm"], (self.inner,), "vector"),
                ParamSpec(names["o"], (h, self.inner))]

    def cache_need(self) -> StateNeed:
        return StateNeed((self.conv_state + self.heads * self.head_dim * self.state,), torch.float32)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        names = self.names
        weight = tensors[names["inp"]]
        padding = self.in_rows - weight.shape[0]
        if padding:
            weight = torch.cat([weight, torch.zeros((padding, self.hidden_size), dtype=weight.dtype, device=weight.device)], dim=0)
        self.in_weight = weight.contiguous()
        # everything that enters the recurrence is float32 (the stored values widen exactly)
        self.conv_weight = tensors[names["conv"]].float().contiguous()
        self.conv_bias = tensors[names["conv_b"]].float().contiguous()
        self.dt_bias = tensors[names["dt_bias"]].float().contiguous()
        self.a_log = tensors[names["a_log"]].float().contiguous()
        self.d = tensors[names["d"]].float().contiguous()
        self.norm_weight = tensors[names["norm"]].float().contiguous()
        self.o_weight = tensors[names["o"]]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateView) -> torch.Tensor:
        n = x.shape[0]
        proj = ctx.buffer("state_space.proj", (n, self.in_rows), x.dtype)
        kernels.linear(x, self.in_weight, proj)
        conv = ctx.buffer("state_space.conv", (n, self.conv_channels), torch.float32)
        kernels.causal_conv_silu(proj, self.conv_col, self.conv_weight, self.conv_bias, cache.states, 0, ctx.state_slots,
                                 ctx.query_start, ctx.max_query_len, conv)
        y = ctx.buffer("state_space.y", (n, self.inner), torch.float32)
        kernels.selective_scan(conv, proj, self.dt_col, self.dt_bias, self.a_log, self.d, cache.states, self.conv_state,
                               ctx.state_slots, ctx.query_start, self.heads, self.head_dim, self.state, self.groups, y,
                               max_query_len=ctx.max_query_len)
        gated = ctx.buffer("state_space.gated", (n, self.inner), x.dtype)
        kernels.gated_group_norm(y, proj, self.z_col, self.norm_weight, self.norm_groups, self.eps, gated)
        out = ctx.buffer("state_space.out", (n, self.hidden_size), x.dtype)
        kernels.linear(gated, self.o_weight, out)
        return out
