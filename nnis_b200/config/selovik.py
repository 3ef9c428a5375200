"""Typed configuration of the Selovik decoder, read from config.json.

config.json gives ``architecture`` ("Selovik"), ``vocab``, ``width``, ``norm`` {eps},
``embedding`` {scale, bigram {buckets, mul_prev, mul_cur} (optional)}, ``logit_scale``, ``loop``
{start, stop, times} (optional) and ``layers``: a list whose entries name the layer's mixer
(``type``: "attention"), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``:
``kind`` "dense" with ``ff``; ``kind`` "moe" with ``expert`` {ff}, ``router`` {experts, top, identity,
groups {count, keep}} and ``shared`` {ff} or null; or null for no feed-forward).  Every size and
every constant that may differ between models comes from there, layer by layer.

The model.  Embedding: table row times ``scale``, plus a row of a second table picked by a hash of
(token before, token), then the model's norm.  Every norm is an RMS norm whose stored weight lies
around zero (multiplier 1 + w).  Layers are parallel with a norm per branch,
x += mixer(norm1(x)) + ff(norm2(x)), both of the same x.  Layers ``start .. stop - 1`` run
``times`` times in a row with the same weights and a cache per pass; before every pass but the first
the embedding output is added to the stream, and before every pass row t of ``loop.step``.  The mixer
is differential attention (two softmax maps a head over the same values, rotation of the first
``rot.dims`` values of every map in the rotate-half pairing with frequencies blended by index and a
magnitude on cosine and sine, a sliding window, the maps' difference normed per head, a sigmoid gate
per output value).  Feed-forwards: down(relu(up(x))^2), or experts down(silu(gate(x)) * up(x)) chosen
by softmax scores plus a correction within the best groups, the router's last outputs standing for
experts that hand their input on, plus a shared expert.  Head: the model's norm, the embedding table,
times ``logit_scale``.

Tensor names: ``embed``, ``bigram``, ``embed.norm``, ``loop.step``, ``final.norm`` and ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.{q,k,v,g,o,lq1,lk1,lq2,lk2}``, ``l<i>.mlp.{up,down}`` or
``l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down}}``, with no ``.weight``
ending; weights are stored in bfloat16.  Positions have no bound of the model's own.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, StreamEnter

# angles are float32 products position * frequency; beyond 2^24 a position is no exact float32
MAX_POSITIONS = 1 << 24
# constants that the design fixes
NORM_OFFSET = 1.0  # a norm's multiplier is NORM_OFFSET + the stored weight


def _int(raw: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {least}; got {value!r}")
    return value


def _number(raw: Mapping[str, Any], key: str, where: str, positive: bool = True) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) \
            or (positive and value <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a finite{' positive' if positive else ''} number; "
                          f"got {value!r}")
    return float(value)


def _object(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json: {where}.{key} must be an object")
    return value


def _check_attention(m: Mapping[str, Any], where: str) -> None:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    dim = _int(m, "dim", where)
    _int(m, "vdim", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads={heads} is no multiple of kv_heads={kv_heads}")
    _number(m, "scale", where)
    _number(m, "diff", where, positive=False)
    _int(_object(m, "mask", where), "size", where + ".mask")
    rot = _object(m, "rot", where)
    dims = rot.get("dims")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {dim}; got {dims!r}")
    _number(rot, "base", where + ".rot")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, Mapping):
            raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
        for key in ("factor", "original", "fast", "slow"):
            _number(scaling, key, where + ".rot.scaling")
        if float(rot["base"]) <= 1.0:
            raise ConfigError(f"config.json: {where}.rot.base must exceed 1 where frequencies are scaled")


def _check_mlp(mlp: Mapping[str, Any], where: str) -> None:
    kind = mlp.get("kind")
    if kind == "dense":
        _int(mlp, "ff", where)
        return
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design (dense, moe)")
    _int(_object(mlp, "expert", where), "ff", where + ".expert")
    r = _object(mlp, "router", where)
    experts, top = _int(r, "experts", where + ".router", 0), _int(r, "top", where + ".router")
    identity = _int(r, "identity", where + ".router", 0) if r.get("identity") is not None else 0
    outputs = experts + identity
    count, keep = 1, 1
    if r.get("groups") is not None:
        g = _object(r, "groups", where + ".router")
        count, keep = _int(g, "count", where + ".router.groups"), _int(g, "keep", where + ".router.groups")
    if outputs <= 0 or outputs % count or keep > count or top > keep * (outputs // count):
        raise ConfigError(f"config.json: {where}.router: {outputs} outputs in {count} groups (keep {keep}) cannot "
                          f"give top={top}")
    if mlp.get("shared") is not None:
        _int(_object(mlp, "shared", where), "ff", where + ".shared")


@dataclass(frozen=True)
class SelovikLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class SelovikConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    bigram: Optional[Mapping[str, int]]
    logit_scale: float
    loop: Optional[Tuple[int, int, int]]  # start, stop, times
    layers: Tuple[SelovikLayer, ...]
    raw: Mapping[str, Any]

    architecture = "Selovik"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SelovikConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"config.json: architecture must be {cls.architecture!r}; "
                              f"got {raw.get('architecture')!r}")
        vocab, width = _int(raw, "vocab", "config"), _int(raw, "width", "config")
        eps = _number(_object(raw, "norm", "config"), "eps", "norm")
        emb = raw.get("embedding") if raw.get("embedding") is not None else {}
        if not isinstance(emb, Mapping):
            raise ConfigError("config.json: embedding must be an object")
        scale = _number(emb, "scale", "embedding", positive=False) if emb.get("scale") is not None else 1.0
        bigram = None
        if emb.get("bigram") is not None:
            b = _object(emb, "bigram", "embedding")
            bigram = {"buckets": _int(b, "buckets", "embedding.bigram"),
                      "mul_prev": _int(b, "mul_prev", "embedding.bigram", 0),
                      "mul_cur": _int(b, "mul_cur", "embedding.bigram", 0)}
        logit_scale = _number(raw, "logit_scale", "config", positive=False) \
            if raw.get("logit_scale") is not None else 1.0
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers must be a list of at least one layer")
        layers: List[SelovikLayer] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with type, mixer and mlp")
            kind, mixer = entry.get("type"), entry["mixer"]
            if kind != "attention":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (attention)")
            _check_attention(mixer, where + ".mixer")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"config.json: {where}.mlp must be null or an object")
                _check_mlp(mlp, where + ".mlp")
            layers.append(SelovikLayer(kind, mixer, mlp))
        loop = None
        if raw.get("loop") is not None:
            lp = _object(raw, "loop", "config")
            start, stop = _int(lp, "start", "loop", 0), _int(lp, "stop", "loop", 0)
            times = _int(lp, "times", "loop", 1)
            if not start <= stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within {len(layers)} layers")
            loop = (start, stop, times)
        return cls(vocab, width, eps, scale, bigram, logit_scale, loop, tuple(layers), dict(raw))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        def plain(x):
            return {k: plain(v) for k, v in x.items()} if isinstance(x, Mapping) else x
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale, **({"bigram": dict(self.bigram)} if self.bigram else {})},
               "logit_scale": self.logit_scale,
               "layers": [{"type": l.type, "mixer": plain(l.mixer),
                           "mlp": None if l.mlp is None else plain(l.mlp)} for l in self.layers]}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    # ------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name, "leaf": "",
                                    "offset": NORM_OFFSET})

    def _mixer(self, m: Mapping[str, Any]) -> PartSpec:
        rot = m["rot"]
        scaling = None
        if rot.get("scaling") is not None:
            scaling = {"ramp": "index", **{k: rot["scaling"][k] for k in ("factor", "original", "fast", "slow")}}
        position = PartSpec("rope_frequencies", {"dims": rot["dims"], "base": rot["base"], "pairing": "half",
                                                 "scaling": scaling})
        return PartSpec("differential_attention", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
            "vdim": m["vdim"], "scale": m["scale"], "window": m["mask"]["size"], "diff": m["diff"], "gate": True,
            "eps": self.norm_eps, "position": position, "leaf": "",
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "o": "mix.o", "gate": "mix.g", "lq1": "mix.lq1",
                      "lk1": "mix.lk1", "lq2": "mix.lq2", "lk2": "mix.lk2"}})

    def _ffn(self, mlp: Mapping[str, Any]) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("mlp", {"hidden_size": self.width, "intermediate_size": mlp["ff"], "activation": "relu2",
                                    "leaf": "", "names": {"up": "mlp.up", "down": "mlp.down"}})
        r = mlp["router"]
        groups = r.get("groups") or {"count": 1, "keep": 1}
        shared = None
        if mlp.get("shared") is not None:
            shared = PartSpec("gated_mlp", {
                "hidden_size": self.width, "intermediate_size": mlp["shared"]["ff"], "activation": "silu", "leaf": "",
                "names": {"gate": "mlp.shared.gate", "up": "mlp.shared.up", "down": "mlp.shared.down"}})
        return PartSpec("moe", {
            "hidden_size": self.width, "experts": r["experts"], "top": r["top"], "ff": mlp["expert"]["ff"],
            "activation": "silu_gated", "scores": "softmax_all", "weight_on": "output",
            "identity": r.get("identity") or 0, "groups": groups["count"], "keep": groups["keep"], "shared": shared,
            "leaf": "",
            "names": {"router": "mlp.router", "correction": "mlp.correction", "expert": "mlp.e{e}", "gate": "gate",
                      "up": "up", "down": "down"}})

    def run_order(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, pass number if it is the first layer of a pass through the loop) in run order."""
        n = len(self.layers)
        if self.loop is None or self.loop[0] == self.loop[1]:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    def to_spec(self) -> ModelSpec:
        layers = []
        for i, layer in enumerate(self.layers):
            parts = {"norm": self._norm("norm1"), "mixer": self._mixer(layer.mixer)}
            params: Dict[str, Any] = {}
            if layer.mlp is not None:
                parts["ffn_norm"] = self._norm("norm2")
                parts["ffn"] = self._ffn(layer.mlp)
            else:
                params["tolerated"] = ("norm2",)
            layers.append(LayerSpec(prefix=f"l{i}", block="parallel", parts=parts, params=params))
        times = self.loop[2] if self.loop is not None else 0
        schedule = []
        for i, t in self.run_order():
            enter = None
            if t is not None:  # the first layer of pass t: the embedding output again (not the first time), the pass's row
                enter = StreamEnter(embedding=t > 0, tensor="loop.step", rows=times, row=t)
            schedule.append(ScheduleEntry(i, enter=enter))
        embedding = {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed", "leaf": "",
                     "scale": self.embedding_scale, "norm": self._norm("embed.norm")}
        if self.bigram is not None:
            embedding["pair"] = {"name": "bigram", **self.bigram}
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=self.width,
            vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("pair_hash_embedding", embedding),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width, "name": "embed",
                                          "tied_to": "embed", "leaf": "", "scale": self.logit_scale}),
            stop_token_ids=(),
            stored_dtype="bfloat16",
        )
        spec.validate()
        return spec
