"""Small Sedopel configurations and model folders for the tests.  The sizes differ between
them in everything, none is a power-of-two family throughout, and each choice of the
design appears in several values: one and several key/value heads under the softmax
attention and under the delta rule, values narrower and wider than keys, a rotation over
nothing, a part and the whole of a head, one to five taps, lightning attention with one to
three heads and decays from fast to none, layers with and without a feed-forward in every
order."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def softmax(heads, kv_heads, dim, vdim, rot_dims, scale, base=10000.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"base": base, "dims": rot_dims}}


def lightning(dim, vdim, decay):
    return {"heads": len(decay), "dim": dim, "vdim": vdim, "decay": list(decay)}


def parallel(left, right, ff=None):
    return {"type": "parallel", "mixer": {"left": left, "right": right},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta(heads, kv_heads, dim, vdim, taps, ff=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(vocab, width, eps, layers):
    return {"architecture": "Sedopel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# both mixers, feed-forwards on some layers only, a delta layer first
MIXED = config(307, 96, 1e-5, [
    delta(4, 2, 24, 16, 4, ff=72),
    parallel(softmax(6, 3, 24, 40, 8, 0.3, base=1000.0), lightning(16, 24, (0.9, 0.999, 0.5)), ff=56),
    parallel(softmax(4, 1, 32, 16, 32, 0.25), lightning(40, 8, (0.97,))),
    delta(3, 3, 16, 48, 2),
    parallel(softmax(2, 2, 16, 16, 0, 0.5), lightning(24, 24, (1.0, 0.8)), ff=40),
])
# sizes that are no multiples of eight or four
ODD = config(211, 76, 1e-6, [
    parallel(softmax(3, 3, 10, 34, 4, 0.4, base=50.0), lightning(18, 6, (0.6, 0.99)), ff=52),
    delta(2, 1, 22, 10, 5),
    delta(6, 2, 12, 36, 1, ff=20),
    parallel(softmax(5, 1, 18, 6, 18, 0.2, base=2000.0), lightning(10, 30, (0.95, 0.95, 0.3, 0.999))),
])
# one mechanism each
ONLY_SOFTMAX = config(150, 64, 1e-5, [
    parallel(softmax(4, 2, 16, 24, 8, 0.5, base=100.0), lightning(8, 8, (0.9,))),
    parallel(softmax(8, 1, 12, 40, 12, 0.6, base=30.0), lightning(8, 8, (0.5,)))])
ONLY_LIGHTNING = config(150, 64, 1e-5, [
    parallel(softmax(1, 1, 8, 8, 2, 0.5), lightning(32, 16, (0.999, 0.7))),
    parallel(softmax(1, 1, 8, 8, 2, 0.5), lightning(72, 40, (0.99,))),
    parallel(softmax(1, 1, 8, 8, 2, 0.5), lightning(128, 64, (1.0, 0.9)))])
ONLY_DELTA = config(150, 64, 1e-5, [delta(2, 1, 32, 32, 3), delta(4, 4, 8, 70, 4), delta(2, 2, 136, 20, 2),
                                    delta(1, 1, 256, 33, 3)])
ONLY_DENSE = config(150, 72, 1e-5, [delta(1, 1, 8, 8, 2, ff=88)])
# softmax attention made sharp: large scores, so that most of a query's weight lies on one key
SHARP = config(150, 64, 1e-5, [
    parallel(softmax(4, 2, 16, 16, 8, 2.0, base=100.0), lightning(8, 8, (0.9,))),
    parallel(softmax(2, 1, 24, 8, 24, 1.5, base=10000.0), lightning(8, 8, (0.9,)))])
# key and value heads of 64 and of 128: the sizes of the tensor-core prompt attention
HEADS_64 = config(150, 64, 1e-5, [
    parallel(softmax(4, 2, 64, 64, 32, 0.2, base=100.0), lightning(64, 64, (0.98, 0.9)), ff=40),
    delta(2, 1, 64, 64, 4),
    parallel(softmax(2, 1, 128, 128, 128, 0.15, base=5000.0), lightning(32, 32, (0.999,)))])
CONFIGS: Dict[str, dict] = {"mixed": MIXED, "odd": ODD, "heads64": HEADS_64, "softmax": ONLY_SOFTMAX,
                            "lightning": ONLY_LIGHTNING, "delta": ONLY_DELTA, "dense": ONLY_DENSE, "sharp": SHARP}


def make_model(tmp_dir: str, cfg: dict, seed: int) -> str:
    """A model folder with random weights whose activations and scores are of order one.
    Tensors that random numbers around zero or one would make harmless are moved to where they
    matter: the delta rule's decays spread between fast and very slow, temperatures, the depth
    weights and the two output norms of a pair of mixers all differ clearly from one another."""
    from nnis_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    write_random_model(cfg, seed, tmp_dir, std=1.0, norm_std=0.1, std_by_fan_in=True)
    path = os.path.join(tmp_dir, "model.safetensors")
    w = load_file(path)
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(w):
        t = w[name].float()
        if name.endswith(".mix.A_log"):     # decays exp(-exp(A_log) * softplus(.)) from about 0.4 up to 0.999
            t = torch.empty_like(t).uniform_(-7.0, 0.0, generator=g)
        elif name.endswith(".mix.dt_bias"):
            t = torch.empty_like(t).uniform_(-1.0, 1.0, generator=g)
        elif name.endswith(".temp") or name.endswith(".out"):
            t = torch.empty_like(t).uniform_(0.4, 1.6, generator=g)
        elif name.endswith(".dwa"):
            t = torch.empty_like(t).uniform_(0.15, 0.9, generator=g) * (1 - 2 * (torch.rand(t.shape, generator=g) < 0.2).float())
        elif name.endswith(".conv"):        # taps of order one: the inputs before the current one matter
            t = torch.empty_like(t).uniform_(-1.0, 1.0, generator=g)
        w[name] = t.to(torch.bfloat16)
    save_file(w, path)
    return tmp_dir


def load_weights(model_dir: str, as_bf16: bool):
    from safetensors.torch import load_file
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: (v.to(torch.bfloat16).float() if as_bf16 else v.float()) for k, v in w.items()}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)
