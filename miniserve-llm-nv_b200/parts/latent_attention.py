"""The latent-attention mixer: attention whose keys and values are linear in one cached vector per token.

With ``h`` the mixer's input, ``H`` heads, per head ``dim`` unrotated and ``rot_dim`` rotated query/key entries,
``vdim`` value entries and a latent of ``kv_rank`` entries:

* ``q = W_q h``, head by head ``[q_h (dim) ; q_r,h (rot_dim)]``; ``q_r,h`` is rotated by the position encoding.
* ``W_dkv h`` has ``kv_rank + rot_dim`` entries: the first ``kv_rank``, RMS-normed with a weight, are the latent
  ``c``; the last ``rot_dim``, rotated, are a key part ``k_r`` that all heads share.  ``[c ; k_r]`` is all that
  the cache keeps of a token (:class:`~.base.PagedLatentNeed`).
* head ``h`` has keys ``U_h c`` and values ``V_h c``; the score of query i and key j is
  ``(q_h(i) . U_h c(j) + q_r,h(i) . k_r(j)) * scale``, causal, ordinary softmax.
* the head's output is multiplied by ``sigmoid(W_g h)_h`` (optional), and ``W_o`` maps the concatenated heads back.

The keys and values of the heads are never formed.  ``q_h . U_h c = (U_h^T q_h) . c``, so the query is taken to the
latent space (one small product per head) and attends to the cached rows directly
(``kernels.latent_attention``); the weighted sum of the ``c(j)`` is then multiplied by ``V_h`` (again one small
product per head).  A step therefore reads ``kv_rank + rot_dim`` numbers per cached token, whatever the number of
heads, in prompt portions and in decoding alike.

The three projections of ``h`` (queries, latent with key part, gate logits) run as one matrix product over a
row-concatenated weight, padded with zero rows to a multiple of eight.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import POSITIONS, PagedLatentNeed, ParamSpec, Part, register_mixer
from .context import PagedLatentView, StepContext
from .spec import PartSpec


@register_mixer("latent_attention")
class LatentAttention(Part):
    def __init__(self, *, prefix: str, hidden_size: int, num_heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, eps: float, position: PartSpec, output_gate: bool = True, window: Optional[int] = None,
                 q_name: str = "q", dkv_name: str = "dkv", latent_norm_name: str = "dkv.norm", uk_name: str = "uk",
                 uv_name: str = "uv", gate_name: str = "g", o_name: str = "o") -> None:
        if min(hidden_size, num_heads, dim, vdim, kv_rank) < 1 or rot_dim < 0:
            raise ValueError("latent attention: every size must be positive (the rotated part may be empty)")
        self.prefix, self.hidden_size, self.num_heads = prefix, hidden_size, num_heads
        self.dim, self.rot_dim, self.vdim, self.kv_rank = dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.window, self.output_gate = float(scale), float(eps), window, bool(output_gate)
        self.position = None
        if rot_dim and position.kind != "none":
            self.position = POSITIONS.build(position, head_dim=rot_dim) if "head_dim" not in position.args \
                else POSITIONS.build(position)
            if getattr(self.position, "interleaved", False) or not hasattr(self.position, "tables"):
                raise ValueError("latent attention rotates by a table of half-split pairs (position kind 'rope')")
        self.names = dict(q=prefix + q_name, dkv=prefix + dkv_name, norm=prefix + latent_norm_name, uk=prefix + uk_name,
                          uv=prefix + uv_name, g=prefix + gate_name, o=prefix + o_name)
        q_rows, dkv_rows = num_heads * (dim + rot_dim), kv_rank + rot_dim
        self.q_col, self.dkv_col, self.gate_col = 0, q_rows, q_rows + dkv_rows
        rows = q_rows + dkv_rows + (num_heads if self.output_gate else 0)
        self.in_rows = (rows + 7) // 8 * 8
        self.in_weight: Optional[torch.Tensor] = None       # [in_rows, hidden]: q ; dkv ; gate ; zero rows
        self.norm_weight: Optional[torch.Tensor] = None
        self.uk_t: Optional[torch.Tensor] = None            # [H, kv_rank, dim]: U_h^T, the map of a query to the latent space
        self.uv: Optional[torch.Tensor] = None              # [H, vdim, kv_rank]
        self.o_weight: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ declaration
    def param_specs(self) -> list[ParamSpec]:
        h, n = self.hidden_size, self.num_heads
        specs = [ParamSpec(self.names["q"], (n * (self.dim + self.rot_dim), h)),
                 ParamSpec(self.names["dkv"], (self.kv_rank + self.rot_dim, h)),
                 ParamSpec(self.names["norm"], (self.kv_rank,), "vector"),
                 ParamSpec(self.names["uk"], (n * self.dim, self.kv_rank)),
                 ParamSpec(self.names["uv"], (n * self.vdim, self.kv_rank)),
                 ParamSpec(self.names["o"], (h, n * self.vdim))]
        if self.output_gate:
            specs.insert(5, ParamSpec(self.names["g"], (n, h)))
        return specs

    def cache_need(self) -> PagedLatentNeed:
        return PagedLatentNeed(self.kv_rank, self.rot_dim, self.window)

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        names = self.names
        pieces = [tensors[names["q"]], tensors[names["dkv"]]]
        if self.output_gate:
            pieces.append(tensors[names["g"]])
        padding = self.in_rows - sum(p.shape[0] for p in pieces)
        if padding:
            pieces.append(torch.zeros((padding, self.hidden_size), dtype=pieces[0].dtype, device=pieces[0].device))
        self.in_weight = torch.cat(pieces, dim=0).contiguous()
        self.norm_weight = tensors[names["norm"]]
        n = self.num_heads
        self.uk_t = tensors[names["uk"]].view(n, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = tensors[names["uv"]].view(n, self.vdim, self.kv_rank).contiguous()
        self.o_weight = tensors[names["o"]]

    # ------------------------------------------------------------------ work
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: PagedLatentView) -> torch.Tensor:
        n, heads = x.shape[0], self.num_heads
        rank, rot, dim, vdim = self.kv_rank, self.rot_dim, self.dim, self.vdim
        proj = ctx.buffer("latent.proj", (n, self.in_rows), x.dtype)
        kernels.linear(x, self.in_weight, proj)
        # queries to the latent space: q_full[n, h] = [U_h^T q_h ; rotated q_r,h]
        q_full = ctx.buffer("latent.q", (n, heads, rank + rot), x.dtype)
        q_heads = proj[:, :heads * (dim + rot)].view(n, heads, dim + rot)
        kernels.linear_batched(q_heads[:, :, :dim].transpose(0, 1), self.uk_t, q_full[:, :, :rank].transpose(0, 1))
        table, rot_dims = (None, 0) if self.position is None else (self.position.tables(ctx), self.position.rotary_dim)
        slots = cache.slots if cache.writable else torch.full_like(cache.slots, -1)
        kernels.latent_prepare(proj, self.q_col, self.dkv_col, heads, dim, rot, rank, slots, self.norm_weight, self.eps,
                               table, rot_dims, cache.pool, q_full)
        mixed = ctx.buffer("latent.mixed", (n, heads, rank), x.dtype)
        kernels.latent_attention(q_full, cache.pool, cache.block_tables, ctx.request_of_token, ctx.positions, ctx.query_start,
                                 ctx.context_lens, ctx.max_query_len, ctx.max_context_len, rank, self.scale, self.window, mixed)
        # back from the latent space: head h's output is V_h (sum_j p_j c_j)
        attended = ctx.buffer("latent.attended", (n, heads, vdim), x.dtype)
        kernels.linear_batched(mixed.transpose(0, 1), self.uv, attended.transpose(0, 1))
        if self.output_gate:
            kernels.head_gate(attended, proj, self.gate_col)
        out = ctx.buffer("latent.out", (n, self.hidden_size), x.dtype)
        kernels.linear(attended.view(n, heads * vdim), self.o_weight, out)
        return out
