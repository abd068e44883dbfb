"""Small Zozezen configurations for the tests, with weights made so that the routing is never a close call."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def attn(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, kv_from=None):
    out = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=dict(base=base, dims=rot_dims))
    if kv_from is not None:
        out["kv_from"] = kv_from
    return dict(type="attention", mixer=out)


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups))


def moe(experts, identity, top, ff, limit, count, keep, shared=None, shared_limit=1.5):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit),
                router=dict(experts=experts, identity=identity, top=top, groups=dict(count=count, keep=keep)),
                shared=None if shared is None else dict(ff=shared, limit=shared_limit))


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


# Sizes that differ from one another everywhere: an attention layer first, two layers that borrow keys (one of them right
# behind the lender, one across a state-space layer), rotation over part of a head and over all of it, a layer without a
# feed-forward, more value than key entries and the other way round, groups of which two are kept, no identity experts
# in one layer and no shared expert in another.
ZOZEZEN_A = dict(architecture="Zozezen", vocab=211, width=96, norm=dict(eps=1e-5), layers=[
    layer(attn(6, 3, 24, 40, 0.23, 16, 5000.0), moe(6, 3, 2, 24, 0.8, 3, 2, 40, 1.7)),
    layer(attn(3, 3, 24, 40, 0.31, 16, 5000.0, kv_from=0), None),
    layer(ssm(6, 12, 20, 3, 4, 2), moe(8, 0, 3, 16, 1.2, 2, 1, None)),
    layer(attn(6, 3, 24, 40, 0.23, 16, 5000.0, kv_from=0), moe(5, 1, 2, 40, 0.9, 1, 1, 24, 0.6)),
    layer(ssm(2, 40, 8, 1, 2, 1), moe(6, 3, 2, 24, 0.8, 3, 2, 40, 1.7)),
    layer(attn(4, 1, 32, 8, 0.2, 32, 300.0), moe(4, 2, 4, 8, 1.0, 2, 2, 16, 1.0)),
])
# One head and one group everywhere; every router output chosen (top = experts + identity); odd sizes (nothing a multiple of
# eight but the width); a convolution of one tap (no inputs kept) and one of five; a state-space layer first.
ZOZEZEN_B = dict(architecture="Zozezen", vocab=157, width=72, norm=dict(eps=1e-6), layers=[
    layer(ssm(1, 20, 6, 1, 1, 1), moe(2, 1, 3, 20, 0.7, 1, 1, 12, 2.5)),
    layer(attn(1, 1, 12, 10, 0.4, 6, 100.0), moe(3, 0, 1, 10, 1.1, 3, 1, None)),
    layer(ssm(3, 6, 36, 3, 5, 3), None),
    layer(attn(5, 5, 6, 14, 0.17, 2, 20000.0), moe(3, 3, 2, 12, 0.5, 2, 1, 20, 0.9)),
    layer(attn(5, 5, 6, 14, 0.5, 2, 20000.0, kv_from=3), moe(3, 3, 2, 12, 0.5, 2, 1, 20, 0.9)),
])
# Sizes of the kind real models have in small: heads of 64 and 128 with values of the same size, eight query heads per
# key/value head, a state of 64 and of 128 numbers, many experts.
ZOZEZEN_C = dict(architecture="Zozezen", vocab=300, width=128, norm=dict(eps=1e-6), layers=[
    layer(ssm(8, 16, 64, 2, 4, 4), moe(16, 0, 4, 32, 7.0, 4, 2, 64, 7.0)),
    layer(attn(8, 1, 64, 64, 0.125, 64, 1000000.0), moe(12, 4, 2, 32, 1.0, 4, 1, 32, 1.0)),
    layer(ssm(4, 32, 128, 1, 4, 1), moe(16, 0, 4, 32, 7.0, 4, 2, 64, 7.0)),
    layer(attn(4, 2, 128, 128, 0.09, 64, 10000.0), moe(12, 4, 2, 32, 1.0, 4, 1, 32, 1.0)),
    layer(attn(8, 2, 128, 128, 0.09, 64, 10000.0, kv_from=3), moe(12, 4, 2, 32, 1.0, 4, 1, 32, 1.0)),
])
# Head sizes that are multiples of 16 but neither equal for keys and values nor among 32 / 64 / 128: the tensor-core kernel
# whose head sizes are run-time numbers; a layer on borrowed keys with four times the lender's query heads.
ZOZEZEN_D = dict(architecture="Zozezen", vocab=180, width=112, norm=dict(eps=1e-5), layers=[
    layer(attn(4, 2, 48, 80, 0.15, 32, 10000.0), moe(6, 2, 2, 16, 1.0, 2, 1, 24, 1.0)),
    layer(ssm(4, 16, 32, 2, 4, 2), moe(5, 0, 2, 16, 1.0, 1, 1, None)),
    layer(attn(16, 2, 48, 80, 0.2, 32, 10000.0, kv_from=0), moe(6, 2, 2, 16, 1.0, 2, 1, 24, 1.0)),
    layer(attn(2, 2, 112, 16, 0.1, 16, 500.0), None),
])
CONFIGS = {"a": ZOZEZEN_A, "b": ZOZEZEN_B, "c": ZOZEZEN_C, "d": ZOZEZEN_D}

POST_NORM_WEIGHT = -0.85     # the stored weight of the sublayers' output norms (1 + w = 0.15): what a sublayer adds stays small


def steer_routers(tensors: dict, config: dict) -> None:
    """Makes every router's choice clear.  Every routed layer gets columns of its own in the embedding: a token's row carries
    the marks 16, 12, 9, ... in the columns of the router outputs id, id + 1, ... (mod the number of outputs), as many as the
    layer chooses, and nothing in the layer's other columns.  The router reads only its own columns (weight one quarter), the
    correction of the choice is ``-0.3 - index / 512`` (all choice scores negative, no two outputs level, and the steps survive
    a bfloat16 checkpoint), and the norms of the sublayers' outputs have small weights, and exactly none in the columns of the
    marks: the stream keeps the marks through all layers untouched, so outputs without a mark score exactly alike and the
    correction alone ranks them.  In place."""
    vocab, width = config["vocab"], config["width"]
    ids = torch.arange(vocab)
    embed = tensors["embed"].float()
    column = 0
    for index, entry in enumerate(config["layers"]):
        for name in (f"l{index}.norm1b", f"l{index}.norm2b"):
            if name in tensors:
                tensors[name] = (POST_NORM_WEIGHT + 0.05 * torch.randn(width, generator=torch.Generator().manual_seed(index))).to(tensors[name].dtype)
        if f"l{index}.mix.A_log" in tensors:
            # decays around 0.75 a token, so that the state remembers a dozen tokens and a lost state shows
            heads = tensors[f"l{index}.mix.A_log"].shape[0]
            tensors[f"l{index}.mix.A_log"] = (-1.5 + 0.3 * torch.randn(heads, generator=torch.Generator().manual_seed(50 + index))).to(
                tensors[f"l{index}.mix.A_log"].dtype)
        mlp = entry["mlp"]
        if not mlp:
            continue
        router = mlp["router"]
        total, top = router["experts"] + router["identity"], router["top"]
        embed[:, column:column + total] = 0
        for choice in range(top):
            embed[ids, column + (ids + choice) % total] = 16.0 * 0.75 ** choice
        name = f"l{index}.mlp.router"
        weight = torch.zeros(total, width)
        weight[:, column:column + total] = 0.25 * torch.eye(total)
        tensors[name] = weight.to(tensors[name].dtype)
        tensors[f"l{index}.mlp.correction"] = (-0.3 - torch.arange(total, dtype=torch.float32) / 512).to(tensors[f"l{index}.mlp.correction"].dtype)
        column += total
    if column > width:
        raise ValueError("the width is too small for the marks of all routed layers")
    for name in tensors:
        if name.endswith((".norm1b", ".norm2b")):
            tensors[name][:column] = -1.0
    tensors["embed"] = embed.to(tensors["embed"].dtype)


def make_folder(tmp_path, name: str, seed: int = 0, stored_dtype: str = "bfloat16", matrix_std: float = 0.08) -> Path:
    import miniserve_b200  # noqa: F401
    from miniserve_b200.weights import random_tensors
    from safetensors.torch import save_file

    folder = Path(tmp_path) / f"zozezen_{name}_{seed}_{stored_dtype}"
    if not folder.exists():
        folder.mkdir(parents=True)
        config = CONFIGS[name]
        tensors = random_tensors(config, seed, stored_dtype, matrix_std)
        steer_routers(tensors, config)
        (folder / "config.json").write_text(json.dumps(config, indent=1))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
