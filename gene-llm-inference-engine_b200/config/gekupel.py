"""Configuration of the Gekupel design, read from its own config.json keys.

Keys: ``architecture`` ("Gekupel"), ``width``, ``vocab``, ``norm.eps``, ``embedding.scale`` and ``layers``, a list whose
entries give ``type`` ("attention", "latent_attention" or "latent_attention_2"), the mixer's sizes under ``mixer``, the
feed-forward under ``mlp`` (null for none; ``kind`` "dense" with ``ff``, or "moe" with ``expert.ff``, ``router.experts``
and ``router.top``) and optionally ``weights_of``: j, a layer without tensors of its own that runs layer j's with a cache
of its own. Every size and constant that the file gives is kept as it stands. The design has no context length of its
own: ``max_position`` (optional) only sets the engine's default.

Translation into parts (``model_spec``): every layer is an ``output_norm`` block (x <- x + N(sublayer(x)), the sublayers
read x itself) with ``rmsnorm`` norms. "attention" becomes the ``attention`` mixer without rotation, with queries and
keys at unit RMS per head (no weights), a distance bias whose slope for head h of H is 2^(-8 (h + 1) / H), blocks of
``mask.size`` positions that do not see each other, and a learned sink per head. The two latent kinds become the
``latent_attention`` mixer over a window of ``mask.size`` positions with an interleaved rotation of the ``rot_dim`` part
computed on the device; "latent_attention_2" adds the long-context ramp scaling of the frequencies and a learned sink.
A dense feed-forward is a ``gated_mlp`` with tanh-GELU, a mixture a ``routed_experts`` with SiLU. The head is a
matrix of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .nipadra import DEFAULT_CONTEXT, _int, _num, _obj

MIXER_TYPES = ("attention", "latent_attention", "latent_attention_2")


def distance_slopes(heads: int) -> List[float]:
    """The slope of the distance bias of head h = 0 .. H-1: 2^(-8 (h + 1) / H)."""
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


@dataclass(frozen=True)
class ChunkedAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    chunk: int
    scale: float

    def to_json(self):
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "mask": {"size": self.chunk},
                "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class RampScaling:
    factor: float
    original: float
    fast: float
    slow: float

    def to_json(self):
        original = int(self.original) if self.original == int(self.original) else self.original
        return {"factor": self.factor, "fast": self.fast, "original": original, "slow": self.slow}


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    window: int
    scale: float
    rot_base: float
    scaling: Optional[RampScaling]      # the second kind only
    sink: bool                          # the second kind only

    def to_json(self):
        rot: Dict[str, Any] = {"base": self.rot_base, "dims": self.rot_dim}
        if self.scaling is not None:
            rot["scaling"] = self.scaling.to_json()
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "mask": {"size": self.window},
                "q_rank": self.q_rank, "rot": rot, "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class GekupelFeedForward:
    kind: str                   # "dense" | "moe"
    ff: int                     # of the dense feed-forward, or of one expert
    experts: int = 0
    top: int = 0

    def to_json(self):
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class GekupelLayer:
    type: str
    mixer: Any                              # ChunkedAttentionSizes | LatentAttentionSizes
    mlp: Optional[GekupelFeedForward]
    weights_of: Optional[int] = None

    def to_json(self):
        out = {"mixer": self.mixer.to_json(), "mlp": None if self.mlp is None else self.mlp.to_json(), "type": self.type}
        if self.weights_of is not None:
            out["weights_of"] = self.weights_of
        return out


def _chunked_attention(m: Dict[str, Any], what: str) -> ChunkedAttentionSizes:
    heads, kv_heads, dim, vdim = (_int(m, k, what) for k in ("heads", "kv_heads", "dim", "vdim"))
    if heads % kv_heads:
        raise ConfigError(f"config.json: {what}: heads must be a multiple of kv_heads")
    return ChunkedAttentionSizes(heads, kv_heads, dim, vdim, _int(_obj(m.get("mask"), what + ".mask"), "size", what + ".mask"),
                                 _num(m, "scale", what))


def _latent_attention(m: Dict[str, Any], what: str, second: bool) -> LatentAttentionSizes:
    heads, dim, rot_dim, vdim, q_rank, kv_rank = (_int(m, k, what) for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"))
    rot = _obj(m.get("rot"), what + ".rot")
    if _int(rot, "dims", what + ".rot") != rot_dim:
        raise ConfigError(f"config.json: {what}: rot.dims must equal rot_dim (the whole rotated part turns)")
    if rot_dim % 2:
        raise ConfigError(f"config.json: {what}: rot_dim must be even")
    base = _num(rot, "base", what + ".rot")
    if not base > 1:
        raise ConfigError(f"config.json: {what}.rot.base must exceed 1")
    scaling = None
    if second:
        sc = _obj(rot.get("scaling"), what + ".rot.scaling")
        scaling = RampScaling(*(_num(sc, k, what + ".rot.scaling") for k in ("factor", "original", "fast", "slow")))
        if not (scaling.factor > 0 and scaling.original > 0 and scaling.fast > 0 and scaling.slow > 0):
            raise ConfigError(f"config.json: {what}.rot.scaling: every number must be positive")
    return LatentAttentionSizes(heads, dim, rot_dim, vdim, q_rank, kv_rank,
                                _int(_obj(m.get("mask"), what + ".mask"), "size", what + ".mask"), _num(m, "scale", what), base,
                                scaling, second)


def _feed_forward(mlp: Any, what: str) -> Optional[GekupelFeedForward]:
    if mlp is None:
        return None
    mlp = _obj(mlp, what)
    kind = mlp.get("kind")
    if kind == "dense":
        return GekupelFeedForward("dense", _int(mlp, "ff", what))
    if kind == "moe":
        router = _obj(mlp.get("router"), what + ".router")
        experts, top = _int(router, "experts", what + ".router"), _int(router, "top", what + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {what}.router.top exceeds the number of experts")
        return GekupelFeedForward("moe", _int(_obj(mlp.get("expert"), what + ".expert"), "ff", what + ".expert"), experts, top)
    raise ConfigError(f"config.json: {what} has the unknown kind {kind!r} (known: dense, moe)")


@dataclass(frozen=True)
class GekupelConfig:
    width: int
    vocab: int
    eps: float
    embedding_scale: float
    layers: Tuple[GekupelLayer, ...]
    max_position: int = DEFAULT_CONTEXT

    architecture = "Gekupel"
    model_type = "gekupel"

    @classmethod
    def from_json(cls, j: Any) -> "GekupelConfig":
        j = _obj(j, "the configuration")
        width, vocab = _int(j, "width", "the model"), _int(j, "vocab", "the model")
        eps = _num(_obj(j.get("norm"), "norm"), "eps", "norm")
        if not eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        scale = _num(_obj(j.get("embedding"), "embedding"), "scale", "embedding")
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[GekupelLayer] = []
        for i, entry in enumerate(raw):
            what = f"layer {i}"
            entry = _obj(entry, what)
            kind = entry.get("type")
            m = _obj(entry.get("mixer"), what + ".mixer")
            if kind == "attention":
                mixer = _chunked_attention(m, what + ".mixer")
            elif kind in ("latent_attention", "latent_attention_2"):
                mixer = _latent_attention(m, what + ".mixer", kind == "latent_attention_2")
            else:
                raise ConfigError(f"config.json: {what} has the unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            mlp = _feed_forward(entry.get("mlp"), what + ".mlp")
            owner = entry.get("weights_of")
            if owner is not None:
                if isinstance(owner, bool) or not isinstance(owner, int) or not (0 <= owner < len(raw)) or owner == i:
                    raise ConfigError(f"config.json: {what}.weights_of must name another layer")
            layers.append(GekupelLayer(kind, mixer, mlp, owner))
        for i, layer in enumerate(layers):
            if layer.weights_of is not None:
                o = layers[layer.weights_of]
                if o.weights_of is not None:
                    raise ConfigError(f"config.json: layer {i} takes the weights of layer {layer.weights_of}, which has none of its own")
                if (o.type, o.mixer, o.mlp) != (layer.type, layer.mixer, layer.mlp):
                    raise ConfigError(f"config.json: layer {i} takes the weights of layer {layer.weights_of} but is described differently")
        max_position = DEFAULT_CONTEXT if j.get("max_position") is None else _int(j, "max_position", "the model")
        return cls(width, vocab, eps, scale, tuple(layers), max_position)

    def to_json(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": [l.to_json() for l in self.layers], "norm": {"eps": self.eps}, "vocab": self.vocab, "width": self.width}
        if self.max_position != DEFAULT_CONTEXT:
            out["max_position"] = self.max_position
        return out

    # ------------------------------------------------------------------ translation into parts
    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = PartSpec("rmsnorm", {"size": D, "eps": self.eps})
        specs, schedule, shared = [], [], {}
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if layer.type == "attention":
                mixer = PartSpec("attention", {
                    "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                    "scale": m.scale, "window": None, "chunk": m.chunk, "position": PartSpec("none", {}),
                    "qk_norm_eps": self.eps, "qk_norm_weights": False, "distance_slopes": distance_slopes(m.heads),
                    "sink": "learned"})
            else:
                rope = PartSpec("rope_on_device", {
                    "head_dim": m.rot_dim, "rotary_dim": m.rot_dim, "theta": m.rot_base, "pairing": "interleaved",
                    "ramp_scaling": None if m.scaling is None else {"factor": m.scaling.factor, "original": m.scaling.original,
                                                                     "fast": m.scaling.fast, "slow": m.scaling.slow}})
                mixer = PartSpec("latent_attention", {
                    "hidden_size": D, "num_heads": m.heads, "head_dim": m.dim, "rotary_dim": m.rot_dim, "value_dim": m.vdim,
                    "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "window": m.window, "norm_eps": self.eps,
                    "position": rope, "sink": "learned" if m.sink else None})
            ffn = None
            if layer.mlp is not None and layer.mlp.kind == "dense":
                ffn = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": layer.mlp.ff, "activation": "gelu_tanh"})
            elif layer.mlp is not None:
                ffn = PartSpec("routed_experts", {"hidden_size": D, "intermediate_size": layer.mlp.ff, "experts": layer.mlp.experts,
                                                  "top": layer.mlp.top, "activation": "silu"})
            specs.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                   feed_forward_norm=None if ffn is None else norm, block="output_norm"))
            if layer.weights_of is None:
                schedule.append(ScheduleEntry(i))
            else:
                shared[i] = layer.weights_of
                schedule.append(ScheduleEntry(layer.weights_of, cache_of=i))
        return ModelSpec(architecture=self.architecture, hidden_size=D, vocab_size=self.vocab, max_position=self.max_position,
                         layers=specs, schedule=schedule, final_norm=norm, tie_word_embeddings=False,
                         embedding_scale=self.embedding_scale, open_ended=True, shared_layers=shared)
