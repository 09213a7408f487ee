"""Configuration of the Zikupel decoder, read from its config.json keys.

config.json of this design names the model in ``architecture`` and describes the stack layer by layer:
``layers[i] = {"type": mixer kind, "mixer": its sizes and constants, "mlp": its feed-forward or null}``.  Model-wide
keys: ``vocab``, ``width``, ``norm.eps``.  Mixer kinds:

* ``attention`` - ``heads``, ``kv_heads``, ``dim`` (query/key size per head), ``vdim`` (value size per head; the values
  are the keys, so it equals ``dim``), ``scale`` (the factor on q.k), ``softcap`` (optional; scores pass through
  softcap * tanh(s / softcap)), ``rot`` = ``{"base", "dims", "scaling": {"factor", "original", "fast", "slow"} or absent}``.
* ``lightning`` - ``heads``, ``dim``, ``vdim``, ``decay`` (one number per head; a single number stands for all heads).

Feed-forward: ``{"kind": "dense", "ff": n}`` or ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts": E, "top": k},
"shared": {"ff": m} or absent}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import KeyReader

ARCHITECTURE = "Zikupel"
MIXER_KINDS = ("attention", "lightning")


def _object(raw, at: str) -> KeyReader:
    if not isinstance(raw, dict):
        raise ConfigError(f"{at}: must be an object")
    return KeyReader(raw, at)


@dataclass(frozen=True)
class RotScaling:
    factor: float
    original: int
    fast: float
    slow: float

    def to_dict(self) -> Dict[str, Any]:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class RotSpec:
    base: float
    dims: int
    scaling: Optional[RotScaling] = None

    def to_dict(self) -> Dict[str, Any]:
        d = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = self.scaling.to_dict()
        return d


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    rot: RotSpec

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
             "rot": self.rot.to_dict()}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class LightningSpec:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str                  # "dense" or "moe"
    ff: int                    # inner size (of each routed expert, for "moe")
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: object              # AttentionSpec or LightningSpec
    mlp: Optional[FeedForwardSpec]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class ZikupelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None

    architecture = ARCHITECTURE

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], where: str = "config.json") -> "ZikupelConfig":
        r = KeyReader(raw, where)
        vocab = r.integer("vocab", minimum=1)
        width = r.integer("width", minimum=1)
        eps = _object(r.any("norm"), f"{where}: norm").number("eps", positive=True)
        layers_raw = r.any("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        layers = []
        for i, item in enumerate(layers_raw):
            at = f"{where}: layers[{i}]"
            lr = _object(item, at)
            kind = lr.string("type")
            if kind == "attention":
                mixer = _read_attention(lr.any("mixer"), f"{at}.mixer")
            elif kind == "lightning":
                mixer = _read_lightning(lr.any("mixer"), f"{at}.mixer")
            else:
                raise ConfigError(f"{at}: 'type' {kind!r} is not a mixer of {ARCHITECTURE} (have {list(MIXER_KINDS)})")
            layers.append(LayerSpec(kind, mixer, _read_ff(lr.any("mlp"), f"{at}.mlp")))
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default="bfloat16")
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers), torch_dtype=dtype,
                   bos_token_id=r.integer("bos_token_id", default=None), eos_token_id=r.integer("eos_token_id", default=None))

    def to_dict(self) -> Dict[str, Any]:
        """config.json content that :meth:`from_dict` reads back to an equal object."""
        d = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": [l.to_dict() for l in self.layers]}
        for k in ("bos_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                d[k] = getattr(self, k)
        return d


def _read_attention(raw, at: str) -> AttentionSpec:
    m = _object(raw, at)
    heads, kv_heads = m.integer("heads", minimum=1), m.integer("kv_heads", minimum=1)
    dim, vdim = m.integer("dim", minimum=1), m.integer("vdim", minimum=1)
    if heads % kv_heads:
        raise ConfigError(f"{at}: 'heads' {heads} must be a multiple of 'kv_heads' {kv_heads}")
    if vdim != dim:
        raise ConfigError(f"{at}: 'vdim' {vdim} must equal 'dim' {dim}: the values of this mixer are its keys")
    rr = _object(m.any("rot"), f"{at}.rot")
    base, dims = rr.number("base", positive=True), rr.integer("dims", minimum=0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"{at}.rot: 'dims' {dims} must be even and at most 'dim' {dim}")
    scaling = None
    if rr.any("scaling") is not None:
        sr = _object(rr.any("scaling"), f"{at}.rot.scaling")
        scaling = RotScaling(sr.number("factor", positive=True), sr.integer("original", minimum=1),
                             sr.number("fast", positive=True), sr.number("slow", positive=True))
        if base == 1.0:
            raise ConfigError(f"{at}.rot: 'base' 1 has no scaling")
    return AttentionSpec(heads, kv_heads, dim, vdim, m.number("scale"), m.number("softcap", default=None, positive=True),
                         RotSpec(base, dims, scaling))


def _read_lightning(raw, at: str) -> LightningSpec:
    m = _object(raw, at)
    heads = m.integer("heads", minimum=1)
    decay = m.any("decay")
    if isinstance(decay, (int, float)) and not isinstance(decay, bool):
        decay = [decay] * heads                   # one number: the same decay for every head
    if not isinstance(decay, list) or len(decay) != heads or any(isinstance(a, bool) or not isinstance(a, (int, float))
                                                                 for a in decay):
        raise ConfigError(f"{at}: 'decay' must be a list of {heads} numbers, one per head")
    return LightningSpec(heads, m.integer("dim", minimum=1), m.integer("vdim", minimum=1), tuple(float(a) for a in decay))


def _read_ff(raw, at: str) -> Optional[FeedForwardSpec]:
    if raw is None:
        return None
    f = _object(raw, at)
    kind = f.string("kind")
    if kind == "dense":
        return FeedForwardSpec("dense", f.integer("ff", minimum=1))
    if kind == "moe":
        rr = _object(f.any("router"), f"{at}.router")
        experts, top = rr.integer("experts", minimum=1), rr.integer("top", minimum=1)
        if top > experts:
            raise ConfigError(f"{at}.router: 'top' {top} exceeds 'experts' {experts}")
        shared = None
        if f.any("shared") is not None:
            shared = _object(f.any("shared"), f"{at}.shared").integer("ff", minimum=1)
        return FeedForwardSpec("moe", _object(f.any("expert"), f"{at}.expert").integer("ff", minimum=1), experts, top, shared)
    raise ConfigError(f"{at}: 'kind' {kind!r} is not a feed-forward of {ARCHITECTURE} (have ['dense', 'moe'])")
