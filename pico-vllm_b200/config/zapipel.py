"""Configuration of the Zapipel decoder, read from its config.json keys.

config.json of this design names the model in ``architecture`` and describes the stack layer by layer:
``layers[i] = {"type": mixer kind, "mixer": its sizes, "mlp": its feed-forward or null}``.  Model-wide keys:
``vocab``, ``width``, ``norm.eps``, ``logit_scale``, ``logit_softcap``.  Keys of the one mixer kind,
``latent_attention``: ``heads``, ``dim`` (query/key size per head), ``vdim`` (value size per head), ``q_rank``
and ``kv_rank`` (sizes of the query latent and of the cached key/value latent), ``scale`` (the factor on
q.k) and optionally ``kv_from`` (the layer whose cached latents this layer reads instead of making its own).
Feed-forward: ``{"kind": "dense", "ff": n}`` or ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts":
E, "top": k}}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import KeyReader

ARCHITECTURE = "Zapipel"
MIXER_KINDS = ("latent_attention",)


@dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    kv_from: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "q_rank": self.q_rank,
             "kv_rank": self.kv_rank, "scale": self.scale}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                  # "dense" or "moe"
    ff: int                    # inner size (of each expert, for "moe")
    experts: int = 0
    top: int = 0

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: LatentAttentionSpec
    mlp: Optional[FeedForwardSpec]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class ZapipelConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    logit_softcap: Optional[float]
    layers: Tuple[LayerSpec, ...]
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "ZapipelConfig":
        r = KeyReader(raw, where)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        norm = r.any("norm")
        if not isinstance(norm, dict):
            raise ConfigError(f"{where}: key 'norm' must be an object with 'eps'")
        eps = KeyReader(norm, f"{where}: norm").number("eps", positive=True)
        logit_scale = r.number("logit_scale", default=1.0)
        softcap = r.number("logit_softcap", default=None, positive=True)
        layers_raw = r.any("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        layers = []
        for i, item in enumerate(layers_raw):
            at = f"{where}: layers[{i}]"
            lr = KeyReader(item, at)
            kind = lr.string("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"{at}: 'type' {kind!r} is not a mixer of {ARCHITECTURE} (have {list(MIXER_KINDS)})")
            mixer = _read_mixer(lr.any("mixer"), f"{at}.mixer", i, layers)
            layers.append(LayerSpec(kind, mixer, _read_ff(lr.any("mlp"), f"{at}.mlp")))
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default="bfloat16")
        return cls(vocab=vocab, width=width, norm_eps=eps, logit_scale=logit_scale, logit_softcap=softcap,
                   layers=tuple(layers), torch_dtype=dtype, bos_token_id=r.integer("bos_token_id", default=None),
                   eos_token_id=r.integer("eos_token_id", default=None))

    def to_dict(self) -> Dict[str, Any]:
        """config.json content that :meth:`from_dict` reads back to an equal object."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "logit_scale": self.logit_scale, "layers": [l.to_dict() for l in self.layers]}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        for k in ("bos_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                d[k] = getattr(self, k)
        return d


def _read_mixer(raw, at: str, index: int, earlier) -> LatentAttentionSpec:
    if not isinstance(raw, dict):
        raise ConfigError(f"{at}: must be an object with the mixer's sizes")
    m = KeyReader(raw, at)
    spec = LatentAttentionSpec(heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1),
                               vdim=m.integer("vdim", minimum=1), q_rank=m.integer("q_rank", minimum=1),
                               kv_rank=m.integer("kv_rank", minimum=1), scale=m.number("scale"),
                               kv_from=m.integer("kv_from", default=None, minimum=0))
    if spec.kv_from is not None:
        if spec.kv_from >= index:
            raise ConfigError(f"{at}: 'kv_from' {spec.kv_from} must name an earlier layer")
        src = earlier[spec.kv_from].mixer
        if src.kv_from is not None:
            raise ConfigError(f"{at}: 'kv_from' {spec.kv_from} names a layer that keeps no latents of its own")
        if src.kv_rank != spec.kv_rank:
            raise ConfigError(f"{at}: 'kv_rank' {spec.kv_rank} differs from layer {spec.kv_from}'s {src.kv_rank}")
    return spec


def _read_ff(raw, at: str) -> Optional[FeedForwardSpec]:
    if raw is None:
        return None
    if not isinstance(raw, dict):
        raise ConfigError(f"{at}: must be null or an object")
    f = KeyReader(raw, at)
    kind = f.string("kind")
    if kind == "dense":
        return FeedForwardSpec("dense", f.integer("ff", minimum=1))
    if kind == "moe":
        expert, router = f.any("expert"), f.any("router")
        if not isinstance(expert, dict) or not isinstance(router, dict):
            raise ConfigError(f"{at}: a 'moe' feed-forward needs the objects 'expert' and 'router'")
        rr = KeyReader(router, f"{at}.router")
        experts, top = rr.integer("experts", minimum=1), rr.integer("top", minimum=1)
        if top > experts:
            raise ConfigError(f"{at}.router: 'top' {top} exceeds 'experts' {experts}")
        return FeedForwardSpec("moe", KeyReader(expert, f"{at}.expert").integer("ff", minimum=1), experts, top)
    raise ConfigError(f"{at}: 'kind' {kind!r} is not a feed-forward of {ARCHITECTURE} (have ['dense', 'moe'])")
