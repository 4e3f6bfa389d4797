"""Typed configuration of the Nizazen decoder, read from ``config.json``.

The file names the design under ``"architecture"``.  ``layers[i]`` holds ``type`` (the mixer: ``attention`` or
``latent_attention``), ``mixer`` (its sizes and constants) and ``mlp`` (a dense feed-forward, a mixture of experts,
or null).  Global: ``vocab``, ``width``, ``norm.eps``, ``streams`` (lanes of the residual stream; absent: one
lane with a plain residual sum) and ``logit_softcap`` (absent: the logits are not squashed).  Nothing else has a
default: a key the design needs and the file lacks is an error.  A key this reader does not know changes nothing it
computes; it is kept in ``unknown_keys`` and named in one warning.
"""

from __future__ import annotations

import copy
import warnings
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Union

from .qwen2 import ConfigError


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} misses {key!r}")
    return d[key]


def _only(d: Dict[str, Any], known, where: str, unknown: List[str]) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    unknown.extend(f"{where}.{k}" for k in sorted(set(d) - set(known)))


def _window(m: Dict[str, Any], where: str, unknown: List[str]) -> Optional[int]:
    mask = m.get("mask")
    if mask is None:
        return None
    _only(mask, ("size",), f"{where}.mask", unknown)
    size = int(_need(mask, "size", f"{where}.mask"))
    if size < 1:
        raise ConfigError(f"config.json: {where}.mask.size must be positive")
    return size


@dataclass
class WindowAttentionConfig:
    """``type: attention``: grouped heads, q and k normed over their whole projection, a sliding window."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]          # None: the configuration has no 'mask': every earlier key is visible

    @classmethod
    def from_dict(cls, m, where, unknown):
        _only(m, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), where, unknown)
        c = cls(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)),
                dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)),
                scale=float(_need(m, "scale", where)), window=_window(m, where, unknown))
        if min(c.heads, c.kv_heads, c.dim, c.vdim) <= 0 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        return c

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass
class LatentAttentionConfig:
    """``type: latent_attention``: keys and values of every head made from one cached vector of ``kv_rank``."""
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]

    @classmethod
    def from_dict(cls, m, where, unknown):
        _only(m, ("heads", "dim", "vdim", "kv_rank", "scale", "mask"), where, unknown)
        c = cls(heads=int(_need(m, "heads", where)), dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)),
                kv_rank=int(_need(m, "kv_rank", where)), scale=float(_need(m, "scale", where)),
                window=_window(m, where, unknown))
        if min(c.heads, c.dim, c.vdim, c.kv_rank) <= 0:
            raise ConfigError(f"config.json: {where}: sizes must be positive")
        return c

    def to_dict(self):
        d = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass
class DenseMLPConfig:
    ff: int

    @classmethod
    def from_dict(cls, m, where, unknown):
        _only(m, ("kind", "ff"), where, unknown)
        c = cls(ff=int(_need(m, "ff", where)))
        if c.ff <= 0:
            raise ConfigError(f"config.json: {where}.ff must be positive")
        return c

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


@dataclass
class ExpertsMLPConfig:
    experts: int
    top: int
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, m, where, unknown):
        _only(m, ("kind", "router", "expert"), where, unknown)
        r, e = _need(m, "router", where), _need(m, "expert", where)
        _only(r, ("experts", "top"), f"{where}.router", unknown)
        _only(e, ("ff", "limit"), f"{where}.expert", unknown)
        c = cls(experts=int(_need(r, "experts", f"{where}.router")), top=int(_need(r, "top", f"{where}.router")),
                ff=int(_need(e, "ff", f"{where}.expert")), limit=float(_need(e, "limit", f"{where}.expert")))
        if not (1 <= c.top <= c.experts) or c.ff <= 0 or not c.limit > 0:
            raise ConfigError(f"config.json: {where}: needs 1 <= top <= experts, a positive ff and a positive limit")
        return c

    def to_dict(self):
        return {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
                "router": {"experts": self.experts, "top": self.top}}


MIXERS = {"attention": WindowAttentionConfig, "latent_attention": LatentAttentionConfig}
MLPS = {"dense": DenseMLPConfig, "moe": ExpertsMLPConfig}


@dataclass
class NizazenLayer:
    type: str
    mixer: Union[WindowAttentionConfig, LatentAttentionConfig]
    mlp: Union[DenseMLPConfig, ExpertsMLPConfig, None]


@dataclass
class NizazenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[NizazenLayer]
    streams: Optional[int] = None            # None: one lane and a plain residual sum (no lane weights in the checkpoint)
    logit_softcap: Optional[float] = None
    eos_token_id: Optional[Any] = None
    architecture: str = "Nizazen"
    unknown_keys: List[str] = field(default_factory=list)

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "NizazenConfig":
        unknown: List[str] = []
        _only(cfg, ("architecture", "architectures", "layers", "norm", "vocab", "width", "streams", "logit_softcap",
                    "eos_token_id"), "the top level", unknown)
        raw = _need(cfg, "layers", "the top level")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]"
            _only(L, ("type", "mixer", "mlp"), where, unknown)
            kind = _need(L, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r}: this design's mixers are {sorted(MIXERS)}")
            mixer = MIXERS[kind].from_dict(_need(L, "mixer", where), f"{where}.mixer", unknown)
            mlp = L.get("mlp")
            if mlp is not None:
                mk = _need(mlp, "kind", f"{where}.mlp")
                if mk not in MLPS:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mk!r}: this design's feed-forwards are {sorted(MLPS)}")
                mlp = MLPS[mk].from_dict(mlp, f"{where}.mlp", unknown)
            layers.append(NizazenLayer(kind, mixer, mlp))
        streams, cap = cfg.get("streams"), cfg.get("logit_softcap")
        out = cls(vocab=int(_need(cfg, "vocab", "the top level")), width=int(_need(cfg, "width", "the top level")),
                  norm_eps=float(_need(_need(cfg, "norm", "the top level"), "eps", "norm")), layers=layers,
                  streams=None if streams is None else int(streams),
                  logit_softcap=None if cap is None else float(cap), eos_token_id=cfg.get("eos_token_id"))
        if out.vocab <= 0 or out.width <= 0 or not out.norm_eps > 0:
            raise ConfigError("config.json: vocab, width and norm.eps must be positive")
        if out.streams is not None and not (1 <= out.streams <= 8):
            raise ConfigError("config.json: streams must lie in 1..8")
        if out.logit_softcap is not None and not out.logit_softcap > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        out.unknown_keys = unknown
        if unknown:
            warnings.warn(f"config.json has keys the Nizazen design does not define (ignored): {unknown}")
        return out

    def stop_token_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        if isinstance(self.eos_token_id, (list, tuple)):
            return [int(t) for t in self.eos_token_id]
        return [int(self.eos_token_id)]

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [{"type": L.type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
                       for L in self.layers],
            "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width,
        }
        if self.streams is not None:
            d["streams"] = self.streams
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_id is not None:
            d["eos_token_id"] = copy.deepcopy(self.eos_token_id)
        return d

    def summary(self) -> str:
        kinds = ", ".join(f"{L.type}+{'none' if L.mlp is None else L.mlp.to_dict()['kind']}" for L in self.layers)
        return (f"Nizazen layers={len(self.layers)} width={self.width} vocab={self.vocab} eps={self.norm_eps} "
                f"streams={self.streams} softcap={self.logit_softcap}: {kinds}")
