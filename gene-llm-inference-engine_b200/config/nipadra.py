"""Configuration of the Nipadra design, read from its own config.json keys.

Keys: ``architecture`` ("Nipadra"), ``width``, ``vocab``, ``norm.eps``, ``postln_alpha`` and ``layers``, a list
whose entries give ``type`` ("lightning" or "parallel"), the mixer's sizes under ``mixer`` and the feed-forward
under ``mlp`` (null for a layer without one; ``kind`` "dense" with ``ff`` and an optional ``act``, "relu" when
absent). Every size and every constant that the file gives is kept as it stands; nothing is assumed equal to
anything else. The design has no context length of its own: ``max_position`` (optional) only sets the engine's default.

Translation into parts (``model_spec``): every layer is a ``post_norm`` block (x <- N(alpha x + sublayer(x)))
with ``rmsnorm`` norms whose weights are stored around zero; "lightning" becomes a ``linear_attention`` mixer;
"parallel" a ``parallel`` mixer of an ``attention`` mixer (values taken from the keys, per-head query/key norm,
interleaved partial rotation with angles computed on the device, sliding window, a sink in the softmax, a
sigmoid gate per head) beside a ``state_space`` mixer; the feed-forward a ``gated_mlp``. The head is the
embedding table.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_INT_LIMIT = 100_000_000
DEFAULT_CONTEXT = 32768
ACTIVATIONS = ("relu", "silu", "gelu_tanh")


def _obj(j: Any, what: str) -> Dict[str, Any]:
    if not isinstance(j, dict):
        raise ConfigError(f"config.json: {what} is not an object")
    return j


def _int(j: Dict[str, Any], key: str, what: str) -> int:
    v = j.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or v != int(v) or not (0 < int(v) <= _INT_LIMIT):
        raise ConfigError(f"config.json: {what} needs a positive integer '{key}' (got {v!r})")
    return int(v)


def _num(j: Dict[str, Any], key: str, what: str) -> float:
    v = j.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"config.json: {what} needs a number '{key}' (got {v!r})")
    return float(v)


@dataclass(frozen=True)
class LightningSizes:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_json(self):
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class WindowAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int
    rot_base: float
    rot_dims: int
    scale: float

    def to_json(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "mask": {"size": self.window}, "rot": {"base": self.rot_base, "dims": self.rot_dims}, "scale": self.scale}


@dataclass(frozen=True)
class StateSpaceSizes:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state

    def to_json(self):
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}


@dataclass(frozen=True)
class ParallelSizes:
    left: WindowAttentionSizes
    right: StateSpaceSizes
    left_scale: float
    right_scale: float

    def to_json(self):
        return {"left": self.left.to_json(), "right": self.right.to_json(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class NipadraLayer:
    type: str                          # "lightning" | "parallel"
    mixer: Any                         # LightningSizes | ParallelSizes
    ff: Optional[int]                  # None: the layer has no feed-forward
    act: str = "relu"

    def to_json(self):
        mlp = None if self.ff is None else {"ff": self.ff, "kind": "dense"}
        if mlp is not None and self.act != "relu":
            mlp["act"] = self.act
        return {"type": self.type, "mixer": self.mixer.to_json(), "mlp": mlp}


def _lightning(m: Dict[str, Any], what: str) -> LightningSizes:
    heads = _int(m, "heads", what)
    decay = m.get("decay")
    if not isinstance(decay, list) or len(decay) != heads or any(
            isinstance(d, bool) or not isinstance(d, (int, float)) or not (0.0 <= d <= 1.0) for d in decay):
        raise ConfigError(f"config.json: {what} needs 'decay', one number in [0, 1] per head")
    return LightningSizes(heads, _int(m, "dim", what), _int(m, "vdim", what), tuple(float(d) for d in decay))


def _window_attention(m: Dict[str, Any], what: str) -> WindowAttentionSizes:
    heads, kv_heads, dim, vdim = (_int(m, k, what) for k in ("heads", "kv_heads", "dim", "vdim"))
    if heads % kv_heads:
        raise ConfigError(f"config.json: {what}: heads must be a multiple of kv_heads")
    if vdim != dim:
        raise ConfigError(f"config.json: {what}: the values are the keys, so vdim ({vdim}) must equal dim ({dim})")
    rot = _obj(m.get("rot"), what + ".rot")
    dims = _int(rot, "dims", what + ".rot")
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {what}.rot.dims must be even and at most dim")
    base = _num(rot, "base", what + ".rot")
    if not base > 0:
        raise ConfigError(f"config.json: {what}.rot.base must be positive")
    return WindowAttentionSizes(heads, kv_heads, dim, vdim, _int(_obj(m.get("mask"), what + ".mask"), "size", what + ".mask"),
                                base, dims, _num(m, "scale", what))


def _state_space(m: Dict[str, Any], what: str) -> StateSpaceSizes:
    s = StateSpaceSizes(*(_int(m, k, what) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
    if s.heads % s.groups:
        raise ConfigError(f"config.json: {what}: heads must be a multiple of groups")
    if s.inner % s.norm_groups:
        raise ConfigError(f"config.json: {what}: heads * vdim must split into norm_groups equal parts")
    return s


@dataclass(frozen=True)
class NipadraConfig:
    width: int
    vocab: int
    eps: float
    alpha: float
    layers: Tuple[NipadraLayer, ...]
    max_position: int = DEFAULT_CONTEXT

    architecture = "Nipadra"
    model_type = "nipadra"

    @classmethod
    def from_json(cls, j: Any) -> "NipadraConfig":
        j = _obj(j, "the configuration")
        width, vocab = _int(j, "width", "the model"), _int(j, "vocab", "the model")
        eps = _num(_obj(j.get("norm"), "norm"), "eps", "norm")
        if not eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        alpha = _num(j, "postln_alpha", "the model")
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[NipadraLayer] = []
        for i, entry in enumerate(raw):
            what = f"layer {i}"
            entry = _obj(entry, what)
            kind = entry.get("type")
            m = _obj(entry.get("mixer"), what + ".mixer")
            if kind == "lightning":
                mixer = _lightning(m, what + ".mixer")
            elif kind == "parallel":
                mixer = ParallelSizes(_window_attention(_obj(m.get("left"), what + ".mixer.left"), what + ".mixer.left"),
                                      _state_space(_obj(m.get("right"), what + ".mixer.right"), what + ".mixer.right"),
                                      _num(m, "left_scale", what + ".mixer"), _num(m, "right_scale", what + ".mixer"))
            else:
                raise ConfigError(f"config.json: {what} has the unknown type {kind!r} (known: lightning, parallel)")
            mlp = entry.get("mlp")
            ff, act = None, "relu"
            if mlp is not None:
                mlp = _obj(mlp, what + ".mlp")
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {what}.mlp has the unknown kind {mlp.get('kind')!r} (known: dense)")
                ff = _int(mlp, "ff", what + ".mlp")
                act = mlp.get("act", "relu")
                if act not in ACTIVATIONS:
                    raise ConfigError(f"config.json: {what}.mlp.act {act!r} is unknown (known: {', '.join(ACTIVATIONS)})")
            layers.append(NipadraLayer(kind, mixer, ff, act))
        max_position = DEFAULT_CONTEXT if j.get("max_position") is None else _int(j, "max_position", "the model")
        return cls(width, vocab, eps, alpha, tuple(layers), max_position)

    def to_json(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
               "postln_alpha": self.alpha, "layers": [l.to_json() for l in self.layers]}
        if self.max_position != DEFAULT_CONTEXT:
            out["max_position"] = self.max_position
        return out

    # ------------------------------------------------------------------ translation into parts
    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = PartSpec("rmsnorm", {"size": D, "eps": self.eps, "weight_offset": 1.0})
        specs = []
        for layer in self.layers:
            if layer.type == "lightning":
                m = layer.mixer
                mixer = PartSpec("linear_attention", {
                    "hidden_size": D, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay": list(m.decay),
                    "activation": "silu", "norm_eps": self.eps, "gate": "sigmoid"})
            else:
                a, s = layer.mixer.left, layer.mixer.right
                rope = PartSpec("rope_on_device", {"head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base,
                                                   "pairing": "interleaved"})
                left = PartSpec("attention", {
                    "hidden_size": D, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                    "scale": a.scale, "window": a.window, "position": rope, "values": "keys", "qk_norm_eps": self.eps,
                    "sink": True, "head_gate": True})
                right = PartSpec("state_space", {
                    "hidden_size": D, "num_heads": s.heads, "head_dim": s.vdim, "state_size": s.state, "groups": s.groups,
                    "conv_taps": s.conv, "norm_groups": s.norm_groups, "norm_eps": self.eps})
                mixer = PartSpec("parallel", {"branches": [("left", left, layer.mixer.left_scale),
                                                           ("right", right, layer.mixer.right_scale)]})
            ffn = None if layer.ff is None else PartSpec("gated_mlp", {
                "hidden_size": D, "intermediate_size": layer.ff, "activation": layer.act})
            specs.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                   feed_forward_norm=None if ffn is None else norm, block="post_norm",
                                   block_params={"alpha": self.alpha}))
        return ModelSpec(architecture=self.architecture, hidden_size=D, vocab_size=self.vocab,
                         max_position=self.max_position, layers=specs,
                         schedule=[ScheduleEntry(i) for i in range(len(specs))], final_norm=norm,
                         tie_word_embeddings=True, open_ended=True)
