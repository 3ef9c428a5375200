"""Typed configuration of the Sedopel decoder, read from config.json.

config.json gives ``architecture`` ("Sedopel"), ``vocab``, ``width``, ``norm`` {eps} and ``layers``:
a list whose entries name the layer's mixer (``type``: "parallel" or "delta"), the mixer's sizes
and constants (``mixer``) and its feed-forward (``mlp``: ``kind`` "dense" with ``ff``, or null for
none).  Every size and every constant that may differ between models comes from there, layer by
layer.

The model: token embedding; layers with a norm before and a norm after each sub-layer,
x += norm1b(mixer(norm1(x))), x += norm2b(ff(norm2(x))); after every layer the stream is replaced
by a learned weighted sum of the embedding output and the results of all layers so far (layer i
has i + 2 weights, ``l<i>.dwa``); the model's norm and the head.

Mixers.  "parallel": two mixers read the same input, softmax attention (``left``: grouped queries,
rotation of the first ``rot.dims`` values of every head in the rotate-half pairing, then an RMS norm
of every q and k head without a weight, scores times ``scale`` and a learned number per head, a
sigmoid gate per output value) and lightning attention (``right``: silu on q, k and v, a fixed decay
per head, one norm over the joined heads, a sigmoid gate); each output is RMS-normed over the
width with a weight of its own and the result is half their sum.  "delta": the gated delta rule
with short convolutions on q, k and v.  Feed-forward: down(gelu(up(x))) with the erf gelu.

Tensor names: ``embed``, ``head``, ``final.norm`` and ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``,
``l<i>.norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa`` with no ``.weight`` ending; weights are
stored in bfloat16.  Positions have no bound of the model's own.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .llama import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# angles are float32 products position * frequency; beyond 2^24 a position is no exact float32
MAX_POSITIONS = 1 << 24
# constants that the design fixes
UNIT_EPS = 1e-6     # q and k of the delta rule: x / sqrt(sum(x^2) + UNIT_EPS)
PAIR_WEIGHT = 0.5   # the parallel mixer is half the sum of its two normed outputs


def _int(raw: Mapping[str, Any], key: str, where: str, least: int = 1) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {least}; got {value!r}")
    return value


def _float(raw: Mapping[str, Any], key: str, where: str) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) \
            or value <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be finite and positive; got {value!r}")
    return float(value)


def _object(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"config.json: {where}.{key} must be an object")
    return value


def _check_softmax(m: Mapping[str, Any], where: str) -> None:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    dim = _int(m, "dim", where)
    _int(m, "vdim", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads={heads} is no multiple of kv_heads={kv_heads}")
    _float(m, "scale", where)
    rot = _object(m, "rot", where)
    dims = rot.get("dims")
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {dim}; got {dims!r}")
    _float(rot, "base", where + ".rot")


def _decays(m: Mapping[str, Any], heads: int, where: str) -> Tuple[float, ...]:
    """One decay per head; a single number stands for all heads."""
    decay = m.get("decay")
    if not isinstance(decay, list):
        decay = [decay] * heads
    if len(decay) != heads:
        raise ConfigError(f"config.json: {where}.decay must be one number or one per head ({heads})")
    for d in decay:
        if isinstance(d, bool) or not isinstance(d, (int, float)) or not 0 < d <= 1:
            raise ConfigError(f"config.json: {where}.decay values lie in (0, 1]; got {d!r}")
    return tuple(float(d) for d in decay)


def _check_lightning(m: Mapping[str, Any], where: str) -> None:
    heads = _int(m, "heads", where)
    _int(m, "dim", where)
    _int(m, "vdim", where)
    _decays(m, heads, where)


def _check_delta(m: Mapping[str, Any], where: str) -> None:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    for key in ("dim", "vdim", "conv"):
        _int(m, key, where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads={heads} is no multiple of kv_heads={kv_heads}")


@dataclass(frozen=True)
class SedopelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class SedopelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SedopelLayer, ...]
    raw: Mapping[str, Any]

    architecture = "Sedopel"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "SedopelConfig":
        if raw.get("architecture") != cls.architecture:
            raise ConfigError(f"config.json: architecture must be {cls.architecture!r}; "
                              f"got {raw.get('architecture')!r}")
        vocab, width = _int(raw, "vocab", "config"), _int(raw, "width", "config")
        eps = _float(_object(raw, "norm", "config"), "eps", "norm")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers must be a list of at least one layer")
        layers: List[SedopelLayer] = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(entry, Mapping) or not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with type, mixer and mlp")
            kind, mixer = entry.get("type"), entry["mixer"]
            if kind == "parallel":
                _check_softmax(_object(mixer, "left", where + ".mixer"), where + ".mixer.left")
                _check_lightning(_object(mixer, "right", where + ".mixer"), where + ".mixer.right")
            elif kind == "delta":
                _check_delta(mixer, where + ".mixer")
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  f"(parallel, delta)")
            mlp = entry.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp must be null or an object of kind 'dense'")
                _int(mlp, "ff", where + ".mlp")
            layers.append(SedopelLayer(kind, mixer, mlp))
        return cls(vocab, width, eps, tuple(layers), dict(raw))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        def plain(x):
            return {k: plain(v) for k, v in x.items()} if isinstance(x, Mapping) else x
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps},
                "layers": [{"type": l.type, "mixer": plain(l.mixer),
                            "mlp": None if l.mlp is None else plain(l.mlp)} for l in self.layers]}

    # ------------------------------------------------------------------
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": name, "leaf": ""})

    def _softmax(self, m: Mapping[str, Any], stem: str) -> PartSpec:
        position = PartSpec("rope_frequencies", {"dims": m["rot"]["dims"], "base": m["rot"]["base"],
                                                 "pairing": "half"})
        return PartSpec("sink_attention", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
            "vdim": m["vdim"], "scale": m["scale"], "softcap": 0.0, "chunk": 0, "window": 0, "sink": False,
            "gate": "value", "qk_norm": "head", "head_scale": True, "eps": self.norm_eps, "position": position,
            "kv": "own", "leaf": "",
            "names": {"q": f"{stem}.q", "k": f"{stem}.k", "v": f"{stem}.v", "o": f"{stem}.o", "gate": f"{stem}.g",
                      "head_scale": f"{stem}.temp"}})

    def _lightning(self, m: Mapping[str, Any], stem: str) -> PartSpec:
        return PartSpec("retention", {
            "hidden_size": self.width, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
            "decay": _decays(m, int(m["heads"]), "mixer.right"), "eps": self.norm_eps,
            "position": PartSpec("rope_frequencies", {"dims": 0, "base": 1.0}),
            "activation": "silu", "key_scale": 1.0, "norm": "joined", "gate": "sigmoid", "leaf": "",
            "names": {"q": f"{stem}.q", "k": f"{stem}.k", "v": f"{stem}.v", "g": f"{stem}.g", "o": f"{stem}.o",
                      "norm": f"{stem}.norm"}})

    def _mixer(self, layer: SedopelLayer) -> PartSpec:
        m = layer.mixer
        if layer.type == "parallel":
            return PartSpec("mixer_pair", {
                "hidden_size": self.width, "eps": self.norm_eps, "weight": PAIR_WEIGHT,
                "left": self._softmax(m["left"], "mix.left"), "right": self._lightning(m["right"], "mix.right"),
                "leaf": "", "names": {"left_norm": "mix.left.out", "right_norm": "mix.right.out"}})
        return PartSpec("gated_delta_rule", {
            "hidden_size": self.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"],
            "vdim": m["vdim"], "taps": m["conv"], "eps": self.norm_eps, "unit_eps": UNIT_EPS, "leaf": "",
            "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "q_conv": "mix.q.conv", "k_conv": "mix.k.conv",
                      "v_conv": "mix.v.conv", "b": "mix.b", "a": "mix.a", "a_log": "mix.A_log",
                      "dt_bias": "mix.dt_bias", "g": "mix.g", "norm": "mix.norm", "o": "mix.o"}})

    def to_spec(self) -> ModelSpec:
        layers, schedule = [], []
        most = len(self.layers) + 1
        for i, layer in enumerate(self.layers):
            parts = {"mixer_norm": self._norm("norm1"), "mixer": self._mixer(layer),
                     "mixer_post_norm": self._norm("norm1b")}
            if layer.mlp is not None:
                parts["ffn_norm"] = self._norm("norm2")
                parts["ffn"] = PartSpec("mlp", {
                    "hidden_size": self.width, "intermediate_size": layer.mlp["ff"], "activation": "gelu",
                    "leaf": "", "names": {"up": "mlp.up", "down": "mlp.down"}})
                parts["ffn_post_norm"] = self._norm("norm2b")
            layers.append(LayerSpec(prefix=f"l{i}", block="sandwich", parts=parts,
                                    params={"depth_mix": {"name": "dwa", "terms": i + 2, "most": most}}))
            schedule.append(ScheduleEntry(i))
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=self.width,
            vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "name": "embed", "leaf": ""}),
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": self.width,
                                          "name": "head", "tied_to": None, "leaf": ""}),
            stop_token_ids=(),
            stored_dtype="bfloat16",
        )
        spec.validate()
        return spec
