"""Small Vesidra configurations for the tests, with weights made so that the routing is never a close call."""

from __future__ import annotations

import json
from pathlib import Path

import torch


def rot(dims, base=10000.0, scaling=None):
    return dict(base=base, dims=dims, scaling=scaling)


def mixer(heads, dim, rot_dim, vdim, kv_rank, scale, rotation):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale, rot=rotation)


def moe(experts, top, ff, shared):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top), shared=None if shared is None else dict(ff=shared))


def layer(mix, mlp):
    return dict(type="latent_attention", mixer=mix, mlp=mlp)


YARN_A = dict(factor=2.5, original=64, fast=8.0, slow=1.0)      # a short "original" context: the stretched range is met at once
YARN_B = dict(factor=8.0, original=48, fast=4.0, slow=0.5)

# Sizes that differ from one another everywhere; rotated parts that are only partly rotated (dims < rot_dim), a layer
# without feed-forward, a rotation without scaling, experts with and without a shared one.
VESIDRA_A = dict(architecture="Vesidra", vocab=211, width=96, embedding=dict(scale=3.5), norm=dict(eps=1e-5), layers=[
    layer(mixer(3, 24, 16, 20, 40, 0.21, rot(8, 5000.0, YARN_A)), dict(kind="dense", ff=136)),
    layer(mixer(3, 24, 16, 20, 40, 0.21, rot(8, 5000.0, YARN_A)), moe(5, 2, 24, 40)),
    layer(mixer(2, 16, 32, 40, 56, 0.3, rot(32, 300.0, None)), None),
    layer(mixer(3, 24, 16, 20, 40, 0.21, rot(16, 5000.0, YARN_B)), moe(6, 3, 16, None)),
])
# One head; every expert chosen (top = experts); embedding scale 1; odd sizes (nothing a multiple of eight but the width).
VESIDRA_B = dict(architecture="Vesidra", vocab=157, width=72, embedding=dict(scale=1.0), norm=dict(eps=1e-6), layers=[
    layer(mixer(1, 12, 6, 10, 22, 0.4, rot(6, 100.0, dict(factor=3.0, original=32, fast=6.0, slow=2.0))), moe(3, 3, 20, 12)),
    layer(mixer(5, 6, 10, 14, 18, 0.17, rot(10, 20000.0, None)), dict(kind="dense", ff=100)),
])
# Sizes that the tensor-core kernels take (latent and rotated part multiples of 16, up to 16 heads), many heads.
VESIDRA_C = dict(architecture="Vesidra", vocab=300, width=128, embedding=dict(scale=6.0), norm=dict(eps=1e-6), layers=[
    layer(mixer(8, 32, 16, 32, 64, 0.15, rot(16, 10000.0, YARN_A)), moe(8, 2, 32, 64)),
    layer(mixer(16, 16, 32, 24, 96, 0.2, rot(32, 10000.0, YARN_B)), dict(kind="dense", ff=192)),
    layer(mixer(4, 64, 64, 64, 128, 0.1, rot(64, 500000.0, None)), moe(4, 1, 48, None)),
])
# A width that is no multiple of eight (rows that start off 16-byte boundaries), tiny heads, two rotated entries.
VESIDRA_D = dict(architecture="Vesidra", vocab=97, width=100, embedding=dict(scale=10.0), norm=dict(eps=1e-6), layers=[
    layer(mixer(3, 10, 4, 6, 14, 0.27, rot(2, 50.0, dict(factor=2.0, original=16, fast=2.0, slow=1.0))), moe(4, 2, 10, 6)),
    layer(mixer(2, 7, 3, 5, 11, 0.31, rot(2, 10000.0, None)), dict(kind="dense", ff=50)),
])
CONFIGS = {"a": VESIDRA_A, "b": VESIDRA_B, "c": VESIDRA_C, "d": VESIDRA_D}


def steer_routers(tensors: dict, config: dict) -> None:
    """Makes every router's choice clear.  Every routed layer gets columns of its own in the embedding: a token's row
    carries the marks 16, 12, 9, ... (over the embedding scale) in the columns of the experts id, id + 1, id + 2, ... (mod E)
    that it is to choose, first to last, and nothing in the layer's other columns; the residual stream keeps them (the
    matrices that write into the stream are halved, so that what the layers add stays small beside the marks).  The
    router reads its columns with weight one quarter on top of small random weights, and has a small bias.  In place."""
    vocab, scale = config["vocab"], float(config["embedding"]["scale"])
    ids = torch.arange(vocab)
    embed = tensors["embed"].float()
    column = 0
    for index, entry in enumerate(config["layers"]):
        mlp = entry["mlp"]
        if not mlp or mlp["kind"] != "moe":
            continue
        experts, top = mlp["router"]["experts"], mlp["router"]["top"]
        embed[:, column:column + experts] = 0
        for choice in range(top):
            embed[ids, column + (ids + choice) % experts] = (16.0 * 0.75 ** choice) / scale
        name = f"l{index}.mlp.router"
        router = tensors[name].float() * 0.1
        router[:, column:column + experts] = 0.25 * torch.eye(experts)
        tensors[name] = router.to(tensors[name].dtype)
        tensors[name + ".b"] = (0.02 * torch.arange(experts, dtype=torch.float32)).to(tensors[name + ".b"].dtype)
        column += experts
    for name in tensors:
        if name.endswith((".mix.o", ".down")):
            tensors[name] = (tensors[name].float() * 0.5).to(tensors[name].dtype)
    if column > config["width"]:
        raise ValueError("the width is too small for the marks of all routed layers")
    tensors["embed"] = embed.to(tensors["embed"].dtype)


def make_folder(tmp_path, name: str, seed: int = 0, stored_dtype: str = "bfloat16", matrix_std: float = 0.08) -> Path:
    import miniserve_b200  # noqa: F401
    from miniserve_b200.weights import random_tensors
    from safetensors.torch import save_file

    folder = Path(tmp_path) / f"vesidra_{name}_{seed}_{stored_dtype}"
    if not folder.exists():
        folder.mkdir(parents=True)
        config = CONFIGS[name]
        tensors = random_tensors(config, seed, stored_dtype, matrix_std)
        steer_routers(tensors, config)
        (folder / "config.json").write_text(json.dumps(config, indent=1))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder
