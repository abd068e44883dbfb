"""Zozezen: a decoder whose layers alternate, in an order that ``config.json`` gives, between two mixers (grouped-query
attention with a sink in the softmax and a gate per head; a selective state-space recurrence) and whose feed-forward is
a mixture of clamped gated experts with identity experts, a group-limited choice and a gated shared expert.  Every
sublayer has a norm before it and a norm of its own output; all norms of the stream store their weight around zero
(``1 + w``).  An attention layer may read the keys and values of an earlier attention layer instead of making its own.

``config.json`` lists the layers one by one; tensor names are ``embed``, ``final.norm``, ``head`` and, for layer i,
``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.{q,k,v,q.norm,k.norm,g,o}`` or
``l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}``, and
``l<i>.mlp.{router,correction,e<j>.gate,e<j>.up,e<j>.down,shared.gate,shared.up,shared.down,shared.sg}``.
"""

from __future__ import annotations

from ..config.model_config import ZozezenConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartSpec

# The design gives positions no upper limit; this is the engine's own bound on a request's length (it sizes the block
# tables of captured decode steps), which `max_model_len` lowers.
NOMINAL_MAX_POSITIONS = 131072


def build_zozezen_spec(config: ZozezenConfig) -> ModelSpec:
    width, eps = config.width, config.eps

    def stream_norm(name: str) -> PartSpec:
        return PartSpec("rms", dict(name=name, size=width, eps=eps, one_plus=True))

    layers, order, unused = [], [], []
    for index, layer in enumerate(config.layers):
        m = layer.mixer
        cache_of = None
        if layer.type == "attention":
            position = PartSpec("none") if m.rot.dims == 0 else PartSpec(
                "rope", dict(head_dim=m.dim, theta=m.rot.base, rotary_dim=m.rot.dims, frequencies="float64"))
            mixer = PartSpec("attention", dict(
                hidden_size=width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim, qk_norm=True,
                eps=eps, position=position, scale=m.scale, sink=True, output_gate=True, own_kv=m.kv_from is None,
                q_name="mix.q", k_name="mix.k", v_name="mix.v", o_name="mix.o", q_norm_name="mix.q.norm",
                k_norm_name="mix.k.norm", gate_name="mix.g"))
            cache_of = m.kv_from            # layers run once each, in order: a layer's index is its place in the order
        else:
            mixer = PartSpec("state_space", dict(
                hidden_size=width, heads=m.heads, head_dim=m.vdim, state=m.state, groups=m.groups, taps=m.conv,
                norm_groups=m.norm_groups, eps=eps, in_name="mix.in", conv_name="mix.conv", conv_bias_name="mix.conv.b",
                dt_bias_name="mix.dt_bias", a_log_name="mix.A_log", d_name="mix.D", norm_name="mix.norm", o_name="mix.o"))
        feed_forward = None
        if layer.mlp is not None:
            f = layer.mlp
            feed_forward = PartSpec("routed_experts", dict(
                hidden_size=width, experts=f.experts, top=f.top, expert_size=f.ff, shared_size=f.shared_ff, router_bias=False,
                activation="clamped_glu", limit=f.limit, shared_limit=f.shared_limit, identity=f.identity,
                scoring="all_softmax", correction_name="mlp.correction", groups=(f.group_count, f.group_keep),
                shared_gate_name="mlp.shared.sg", router_name="mlp.router", expert_name="mlp.e{index}.",
                shared_name="mlp.shared."))
        layers.append(LayerSpec(
            prefix=f"l{index}.", mixer=mixer, feed_forward=feed_forward, mixer_norm=stream_norm("norm1"),
            feed_forward_norm=None if feed_forward is None else stream_norm("norm2"), block=PartSpec("sandwich"),
            mixer_post_norm=stream_norm("norm1b"),
            feed_forward_post_norm=None if feed_forward is None else stream_norm("norm2b")))
        order.append(LayerRun(index, cache_of))
        if feed_forward is None:
            unused += [f"l{index}.norm2", f"l{index}.norm2b"]       # a checkpoint may carry them although nothing reads them
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, embedding_name="embed", layers=tuple(layers), order=tuple(order),
        final_norm=stream_norm("final.norm"), output_name="head", max_positions=NOMINAL_MAX_POSITIONS,
        nominal_max_positions=True, optional_names=tuple(unused))


register_architecture("Zozezen", ZozezenConfig, build_zozezen_spec)
