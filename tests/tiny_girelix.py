"""Tiny Girelix configurations of the tests' own, and a folder of random weights shaped so that faults show.

Sizes differ from layer to layer and between the configurations: query heads over 1, 2, 3 or as many key/value
heads, head sizes that the tensor-core kernels take and that they do not, rotations of a whole head, of a part of it
and of nothing, 1 to 3 heads of linear attention with key sizes below, at and above a warp's width, experts with and
without identities, one group or several, all groups kept or some, one expert per token or several, layers without a
feed-forward, widths that are no multiple of 8.
"""

import json
from pathlib import Path

import torch

LEFT = dict(heads=6, kv_heads=2, dim=24, vdim=24, scale=0.31, rot=dict(base=10000.0, dims=16))
LEFT_FULL = dict(heads=4, kv_heads=4, dim=16, vdim=16, scale=0.4, rot=dict(base=500.0, dims=16))
LEFT_ODD = dict(heads=3, kv_heads=1, dim=20, vdim=20, scale=0.27, rot=dict(base=1000000.0, dims=6))
LEFT_WIDE = dict(heads=36, kv_heads=2, dim=8, vdim=8, scale=0.5, rot=dict(base=100.0, dims=0))
LEFT_RAGGED = dict(heads=3, kv_heads=3, dim=12, vdim=12, scale=0.33, rot=dict(base=77.0, dims=4))
RIGHT = dict(heads=3, dim=20, vdim=24, decay=[0.55, 0.9, 0.995])
RIGHT_ONE = dict(heads=1, dim=72, vdim=40, decay=[0.97])
RIGHT_SMALL = dict(heads=2, dim=8, vdim=5, decay=[1.0, 0.25])
RIGHT_RAGGED = dict(heads=2, dim=12, vdim=10, decay=[0.8, 0.99])
RIGHT_LONG = dict(heads=1, dim=136, vdim=72, decay=[0.98])  # keys longer than the chunked recurrence takes


def moe(experts, identity, top, count, keep, ff):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, identity=identity, top=top,
                                                            groups=dict(count=count, keep=keep)))


def layer(left, right, mlp, left_scale=1.3, right_scale=0.8):
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale), mlp=mlp)


def model(width, vocab, layers, eps=1e-5, mult=0.6):
    return dict(architecture="Girelix", width=width, vocab=vocab, norm=dict(eps=eps), residual_mult=mult, layers=layers)


CONFIGS = {
    "mix": model(80, 200, [
        layer(LEFT, RIGHT, moe(10, 2, 3, 4, 2, 48)),
        layer(LEFT_ODD, RIGHT_ONE, None),
        layer(LEFT_FULL, RIGHT_SMALL, moe(5, 0, 1, 1, 1, 24), left_scale=0.7, right_scale=1.1),
        layer(LEFT_WIDE, RIGHT, moe(6, 3, 4, 3, 3, 40)),
    ]),
    "odd": model(52, 90, [layer(LEFT_ODD, RIGHT_SMALL, moe(7, 1, 2, 2, 1, 20)), layer(LEFT, RIGHT_ONE, moe(3, 1, 4, 1, 1, 36))],
                 eps=1e-6, mult=1.0),
    # sizes that are multiples of nothing much: rows of 50 and 77, heads of 12, experts of 10
    "ragged": model(50, 77, [layer(LEFT_RAGGED, RIGHT_RAGGED, moe(3, 0, 2, 1, 1, 10)), layer(LEFT_ODD, RIGHT_LONG, moe(4, 2, 2, 3, 2, 14))],
                    eps=1e-3, mult=-0.8),
    "bare": model(48, 120, [layer(LEFT_FULL, RIGHT, None), layer(LEFT, RIGHT_SMALL, None)], mult=0.9),
}
PAGE = {"mix": 8, "odd": 16, "ragged": 32, "bare": 64}
LENGTHS = {"mix": [1, 45, 2, 97, 33, 130, 64], "odd": [70, 3, 41, 100], "ragged": [75, 2, 140], "bare": [90, 1, 37]}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}  # largest |difference| over largest |reference logit|
# A routing margin (in units of the scores, which lie in 0..1) below this may fall the other way in bfloat16, the more
# so in a late layer, whose input carries the rounding of the layers before it.
CLOSE_CALL = 0.05


def make_folder(config, seed, folder, sharp=True):
    """A model folder with random weights. ``sharp``: attention's q and k large enough for peaked scores, sinks of
    both signs and of the scores' size, routers and corrections wide enough that the choice is seldom close."""
    from safetensors.torch import save_file

    from akas_b200.config import config_from_dict
    from akas_b200.weights import random_tensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config_from_dict(config), seed=seed, std=0.08, dtype="float32")
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(tensors):
        if sharp and name.endswith(("left.q", "left.k")):
            tensors[name] = tensors[name] * 2.0
        if name.endswith("left.sink"):
            tensors[name] = torch.randn(tensors[name].shape, generator=g) * 2.0
        if name.endswith("mlp.router"):
            tensors[name] = tensors[name] * 6.0
        if name.endswith("mlp.correction"):
            tensors[name] = torch.randn(tensors[name].shape, generator=g) * 0.5
        if name.endswith((".ls1", ".ls2")):
            tensors[name] = 1.0 + torch.randn(tensors[name].shape, generator=g) * 0.3
    tensors = {k: v.to(torch.bfloat16).contiguous() for k, v in tensors.items()}  # stored as a checkpoint stores them
    save_file(tensors, str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(config))
    return folder, {k: v.to(torch.float64) for k, v in tensors.items()}


def plant(folder, config, key_token, query_token, channel=20, strength=0.7):
    """Rewrites a one-layer folder so that ``query_token``'s queries and ``key_token``'s keys are long along one
    channel that the rotation leaves alone (``channel`` >= rot.dims): wherever the two stand, the query's score for
    that key is far above the others', so the key is felt among hundreds. The two tokens' embeddings are two
    orthogonal vectors of +-1 (the layer's norm keeps them); every query head's row for the channel points along the
    query token's, every key head's along the key token's. Returns the weights."""
    from safetensors.torch import load_file, save_file

    left = config["layers"][0]["mixer"]["left"]
    assert left["rot"]["dims"] <= channel < left["dim"]
    tensors = load_file(str(Path(folder) / "model.safetensors"))
    c = config["width"]
    assert c % 4 == 0
    u, u2 = torch.ones(c), torch.ones(c)
    u[1::2] = -1.0
    u2[2::4] = u2[3::4] = -1.0
    tensors["embed"][key_token] = u.to(torch.bfloat16)
    tensors["embed"][query_token] = u2.to(torch.bfloat16)
    for a in range(left["heads"]):
        tensors["l0.mix.left.q"][a * left["dim"] + channel] = (strength * u2 / c ** 0.5).to(torch.bfloat16)
    for a in range(left["kv_heads"]):
        tensors["l0.mix.left.k"][a * left["dim"] + channel] = (strength * u / c ** 0.5).to(torch.bfloat16)
    save_file(tensors, str(Path(folder) / "model.safetensors"))
    return {k: v.to(torch.float64) for k, v in tensors.items()}


def prompts(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
