"""Small Selovik configurations and model folders for the tests.  The sizes differ between them
in everything, none is a power-of-two family throughout, and each choice of the design appears in
several values: one and several key/value heads, one to three query heads a key/value head, maps
and values of unequal sizes, a rotation over nothing, a part and the whole of a map, with and
without scaled frequencies, windows shorter than a page, of a page and a token, and longer than
the prompts, dense and expert feed-forwards and none, routers with and without groups, identity
experts, a shared expert; loops over the first layers, the last ones, all of them, and none."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch


def attention(heads, kv_heads, dim, vdim, window, rot_dims, scale, diff=0.5, base=10000.0, scaling=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
            "mask": {"size": window}, "rot": {"base": base, "dims": rot_dims, "scaling": scaling}}


def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, groups=None, shared=None):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router, "shared": {"ff": shared} if shared else None}


def layer(mixer, mlp=None):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def config(vocab, width, eps, layers, loop=None, scale=1.0, bigram=None, logit_scale=1.0):
    cfg = {"architecture": "Selovik", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": scale}, "logit_scale": logit_scale, "layers": layers}
    if bigram:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# every feed-forward, a loop over the middle layers three times, a pair table
MIXED = config(307, 96, 1e-5, [
    layer(attention(6, 3, 24, 40, 50, 8, 0.3, diff=0.3, base=1000.0, scaling=yarn(4.0, 64, 8.0, 1.0)), dense(72)),
    layer(attention(4, 1, 16, 16, 9, 16, 0.4, diff=0.8), moe(5, 3, 24, identity=3, groups=(4, 2), shared=40)),
    layer(attention(2, 2, 32, 24, 200, 0, 0.25, diff=0.5)),
    layer(attention(3, 1, 8, 48, 65, 4, 0.5, diff=0.1, base=50.0), moe(6, 2, 32)),
], loop=(1, 3, 3), scale=3.0, bigram=(101, 7, 13), logit_scale=0.7)
# sizes that are no multiples of eight or four; no loop, no pair table; a window of one token
ODD = config(211, 76, 1e-6, [
    layer(attention(3, 3, 10, 34, 64, 4, 0.4, diff=0.25, base=50.0), moe(3, 1, 20, identity=1, shared=28)),
    layer(attention(5, 1, 18, 6, 1, 18, 0.2, diff=0.6, base=2000.0, scaling=yarn(2.0, 16, 4.0, 0.5)), dense(52)),
    layer(attention(2, 1, 6, 10, 33, 2, 0.7, diff=0.9), moe(7, 4, 12, identity=5, groups=(3, 1))),
], scale=0.5, logit_scale=1.5)
# the whole model is one loop, passed twice; experts only
LOOP_ALL = config(150, 64, 1e-5, [
    layer(attention(4, 2, 16, 24, 30, 8, 0.5, diff=0.4, base=100.0), moe(4, 2, 16, identity=4, groups=(2, 1), shared=24)),
    layer(attention(8, 1, 12, 40, 70, 12, 0.3, diff=0.7, base=30.0), moe(9, 3, 8, groups=(3, 2))),
], loop=(0, 2, 2), scale=2.0, bigram=(31, 3, 5))
# a loop of one pass over the last layer (its row is still added), dense only
LOOP_ONCE = config(150, 72, 1e-5, [
    layer(attention(1, 1, 8, 8, 40, 2, 0.5), dense(88)),
    layer(attention(2, 1, 20, 12, 100, 20, 0.35, diff=0.2, scaling=yarn(8.0, 32, 2.0, 1.0)), dense(24)),
], loop=(1, 2, 1), bigram=(1, 1, 1), logit_scale=2.5)
# attention made sharp: large scores, so that most of a query's weight lies on one key of each map
SHARP = config(150, 64, 1e-5, [
    layer(attention(4, 2, 16, 16, 300, 8, 2.0, diff=0.5, base=100.0), dense(40)),
    layer(attention(2, 1, 24, 8, 129, 24, 1.5, diff=0.3), dense(40)),
    layer(attention(2, 2, 8, 32, 64, 0, 2.5, diff=0.6), None)], bigram=(17, 2, 3))
# maps of 64 and 128 and of 32 with values of 128: the sizes of the tensor-core prompt attention
HEADS_64 = config(150, 64, 1e-5, [
    layer(attention(4, 2, 64, 64, 100, 32, 0.2, diff=0.5, base=100.0), dense(40)),
    layer(attention(2, 1, 32, 128, 70, 32, 0.25, diff=0.4, base=5000.0, scaling=yarn(4.0, 128, 16.0, 1.0)),
          moe(4, 2, 64, identity=2, shared=64)),
    layer(attention(2, 1, 128, 128, 500, 64, 0.15, diff=0.2), dense(64)),
    layer(attention(6, 2, 64, 128, 64, 64, 0.2, diff=0.7), None)], loop=(1, 3, 2), scale=4.0, bigram=(53, 5, 11))
CONFIGS: Dict[str, dict] = {"mixed": MIXED, "odd": ODD, "loop_all": LOOP_ALL, "loop_once": LOOP_ONCE,
                            "sharp": SHARP, "heads64": HEADS_64}


def make_model(tmp_dir: str, cfg: dict, seed: int) -> str:
    """A model folder with random weights whose activations and scores are of order one.
    Tensors that random numbers around zero would make harmless are moved to where they matter:
    the four vectors behind lambda so that the two exponentials differ clearly, the routers'
    corrections large enough to change choices, the pair table and the loop's rows of the size of
    the embedding, norm weights some way off zero."""
    from nnis_b200.weights import write_random_model
    from safetensors.torch import load_file, save_file
    write_random_model(cfg, seed, tmp_dir, std=1.0, norm_std=0.1, std_by_fan_in=True)
    path = os.path.join(tmp_dir, "model.safetensors")
    w = load_file(path)
    g = torch.Generator().manual_seed(seed + 1)
    for name in list(w):
        t = w[name].float()
        if name.rsplit(".", 1)[-1] in ("lq1", "lk1", "lq2", "lk2"):
            t = torch.empty_like(t).uniform_(-1.0, 1.0, generator=g) * (1.2 / t.numel() ** 0.5)
        elif name.endswith(".correction"):
            t = torch.empty_like(t).uniform_(-0.15, 0.15, generator=g)
        elif name.endswith(".router"):
            t = torch.randn(t.shape, generator=g) * (2.0 / t.shape[1] ** 0.5)
        elif "norm" in name:
            t = torch.empty_like(t).uniform_(-0.4, 0.4, generator=g)
        elif name in ("bigram", "loop.step"):
            t = torch.randn(t.shape, generator=g) * 0.7
        elif name == "embed":
            t = torch.randn(t.shape, generator=g) * 0.5
        w[name] = t.to(torch.bfloat16)
    save_file(w, path)
    return tmp_dir


def load_weights(model_dir: str, as_bf16: bool):
    from safetensors.torch import load_file
    w = load_file(os.path.join(model_dir, "model.safetensors"))
    return {k: (v.to(torch.bfloat16).double() if as_bf16 else v.double()) for k, v in w.items()}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)
