"""Vesidra: a decoder of parallel blocks (one RMS norm per layer, read by the mixer and by the feed-forward, whose
outputs are added to the stream together), latent attention with a YaRN-scaled rotation and a gate per head, and a
feed-forward that is a gated MLP (SiLU) in some layers and a mixture of squared-ReLU experts with a shared expert in
others.  The embedding is scaled as it enters the stream and is also the output matrix (without the scale).

``config.json`` lists the layers one by one; tensor names are ``embed``, ``final.norm`` and, for layer i,
``l<i>.norm1``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}`` and ``l<i>.mlp.{gate,up,down}`` or
``l<i>.mlp.{router,router.b,e<j>.up,e<j>.down,shared.up,shared.down}``.
"""

from __future__ import annotations

from ..config.model_config import VesidraConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartSpec

# The design gives positions no upper limit; this is the engine's own bound on a request's length (it sizes the block
# tables of captured decode steps), which `max_model_len` lowers.
NOMINAL_MAX_POSITIONS = 131072


def build_vesidra_spec(config: VesidraConfig) -> ModelSpec:
    width = config.width
    layers = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        m = layer.mixer
        position = PartSpec("rope", dict(head_dim=m.rot_dim, theta=m.rot.base, rotary_dim=m.rot.dims, scaling=m.rot.scaling_dict()))
        mixer = PartSpec("latent_attention", dict(
            hidden_size=width, num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
            eps=config.eps, position=position, output_gate=True, q_name="mix.q", dkv_name="mix.dkv",
            latent_norm_name="mix.dkv.norm", uk_name="mix.uk", uv_name="mix.uv", gate_name="mix.g", o_name="mix.o"))
        if layer.mlp is None:
            feed_forward = None
        elif layer.mlp.kind == "dense":
            feed_forward = PartSpec("gated_mlp", dict(hidden_size=width, intermediate_size=layer.mlp.ff, activation="silu",
                                                      gate_name="mlp.gate", up_name="mlp.up", down_name="mlp.down"))
        else:
            feed_forward = PartSpec("routed_experts", dict(
                hidden_size=width, experts=layer.mlp.experts, top=layer.mlp.top, expert_size=layer.mlp.ff,
                shared_size=layer.mlp.shared_ff, router_bias=True, activation="relu_square", router_name="mlp.router",
                router_bias_name="mlp.router.b", expert_name="mlp.e{index}.", shared_name="mlp.shared."))
        layers.append(LayerSpec(prefix=prefix, mixer=mixer, feed_forward=feed_forward,
                                mixer_norm=PartSpec("rms", dict(name="norm1", size=width, eps=config.eps)),
                                feed_forward_norm=None, block=PartSpec("parallel")))
    return ModelSpec(
        vocab_size=config.vocab, hidden_size=width, embedding_name="embed", layers=tuple(layers),
        order=tuple(LayerRun(index) for index in range(len(layers))),
        final_norm=PartSpec("rms", dict(name="final.norm", size=width, eps=config.eps)),
        output_name=None, max_positions=NOMINAL_MAX_POSITIONS, nominal_max_positions=True,
        embedding_scale=config.embedding_scale)


register_architecture("Vesidra", VesidraConfig, build_vesidra_spec)
