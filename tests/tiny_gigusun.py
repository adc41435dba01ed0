"""Tiny Gigusun configurations of the tests' own, and a folder of random weights shaped so that faults show.

Sizes differ from layer to layer and between the configurations: query heads over 1, 2 or as many key/value heads,
value heads larger and smaller than key heads, windows that are no multiple of a page, more kept tokens than a
window holds, none at all, convolutions of 1, 2 and 4 taps, layers without a feed-forward, a rank of the decay pair
that only the checkpoint's shapes give.
"""

import json
from pathlib import Path

import torch

ATT = dict(heads=6, kv_heads=2, dim=24, vdim=40, scale=0.35, softcap=12.0, mask=dict(size=20, keep_first=3))
ATT_WIDE = dict(heads=4, kv_heads=4, dim=16, vdim=8, scale=0.5, softcap=30.0, mask=dict(size=37, keep_first=0))
ATT_KEPT = dict(heads=2, kv_heads=1, dim=40, vdim=24, scale=0.3, softcap=8.0, mask=dict(size=9, keep_first=11))
GLA = dict(heads=3, dim=20, vdim=24, tau=8.0, rank=6)
GLA_BIG = dict(heads=2, dim=72, vdim=136, tau=4.0, rank=5)
DELTA = dict(heads=4, kv_heads=4, dim=16, vdim=12, conv=4)
DELTA_SHARED = dict(heads=6, kv_heads=2, dim=40, vdim=20, conv=2)
DELTA_ONE_TAP = dict(heads=2, kv_heads=1, dim=24, vdim=28, conv=1)


def layer(kind, mixer, ff=112):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(ff=ff, kind="dense"))


CONFIGS = {
    "mix": dict(architecture="Gigusun", width=80, vocab=200, max_positions=512, norm=dict(eps=1e-5), layers=[
        layer("delta", DELTA), layer("attention", ATT), layer("gla", GLA, ff=None), layer("attention", ATT_KEPT, ff=96),
        layer("delta", DELTA_SHARED), layer("gla", GLA_BIG)]),
    "attention": dict(architecture="Gigusun", width=48, vocab=120, max_positions=512, norm=dict(eps=1e-6),
                      layers=[layer("attention", ATT, ff=None), layer("attention", ATT_WIDE, ff=64)]),
    "gla": dict(architecture="Gigusun", width=56, vocab=90, max_positions=512, norm=dict(eps=1e-6),
                layers=[layer("gla", GLA, ff=None), layer("gla", GLA_BIG, ff=72)]),
    "delta": dict(architecture="Gigusun", width=64, vocab=100, max_positions=512, norm=dict(eps=1e-4),
                  layers=[layer("delta", DELTA_SHARED, ff=None), layer("delta", DELTA, ff=40), layer("delta", DELTA_ONE_TAP, ff=None)]),
}
PAGE = {"mix": 8, "attention": 16, "gla": 64, "delta": 8}
LENGTHS = {"mix": [1, 45, 2, 97, 33, 130, 64], "attention": [70, 3, 41, 100], "gla": [90, 1, 37], "delta": [5, 80, 2, 33]}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}  # largest |difference| over largest |reference logit|


def make_folder(config, seed, folder, slow=False):
    """A model folder with random weights: attention's q and k large enough for peaked scores, decays near one
    (``slow``: so near that a token is still felt hundreds of tokens later)."""
    from safetensors.torch import save_file

    from akas_b200.config import config_from_dict
    from akas_b200.weights import random_tensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = random_tensors(config_from_dict(config), seed=seed, std=0.08, dtype="float32")
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(tensors):
        kind = config["layers"][int(name[1:].split(".")[0])]["type"] if name[0] == "l" and name[1].isdigit() else None
        if kind == "attention" and name.endswith(("mix.q", "mix.k")):
            tensors[name] = tensors[name] * 4.0
        if name.endswith(".r2"):
            tensors[name] = tensors[name].abs() + 0.1
        if name.endswith(".r1"):
            tensors[name] = torch.rand(tensors[name].shape, generator=g) * 0.8
        if name.endswith("A_log"):
            tensors[name] = tensors[name] - (7.0 if slow else 2.0)
        if name.endswith("a2.b") and slow:
            tensors[name] = tensors[name] + 4.0
        if name.endswith(".act"):
            tensors[name] = torch.tensor([0.7, 0.4, 0.2, 0.05]) + tensors[name]
    tensors = {k: v.to(torch.bfloat16).contiguous() for k, v in tensors.items()}  # stored as a checkpoint stores them
    save_file(tensors, str(folder / "model.safetensors"))
    stored = json.loads(json.dumps(config))
    for entry in stored["layers"]:
        entry["mixer"].pop("rank", None)  # the checkpoint's shapes give it
    (folder / "config.json").write_text(json.dumps(stored))
    return folder, {k: v.to(torch.float64) for k, v in tensors.items()}


def prompts(vocab, lengths, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
