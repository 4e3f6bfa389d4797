"""Typed configuration of the Lonasun decoder, read from ``config.json``.

The file names the design under ``"architecture"`` and gives every size and
constant per layer: ``layers[i]`` holds ``type`` (which mixer), ``mixer`` (its
sizes and constants) and ``mlp`` (the feed-forward, or null); ``loop`` names a
span of layers that runs several times with the same weights; ``norm.eps``,
``vocab`` and ``width`` are global.  Nothing has a default: a key the design
needs and the file lacks is an error.  A key this reader does not know changes
nothing it computes; it is kept in ``unknown_keys`` and named in one warning.
"""

from __future__ import annotations

import copy
import warnings
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .qwen2 import ConfigError


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} misses {key!r}")
    return d[key]


_UNKNOWN: List[str] = []       # filled while a configuration is read


def _only(d: Dict[str, Any], known, where: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    _UNKNOWN.extend(f"{where}.{k}" for k in sorted(set(d) - set(known)))


@dataclass
class ChunkedConvAttentionConfig:
    """Constants of the attention mixer (``layers[i].mixer``)."""
    heads: int
    kv_heads: int
    dim: int                  # per-head query/key size
    vdim: int                 # per-head value size
    conv: int                 # taps of the short convolution on q, k and v
    rot_dims: int             # leading dimensions of each head that are rotated
    rot_base: Optional[float]  # None: the configuration has no 'rot' (nothing is rotated)
    scale: float
    chunk: Optional[int]      # keys are visible inside the query's chunk of this many positions (None: all earlier keys)

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "ChunkedConvAttentionConfig":
        _only(m, ("heads", "kv_heads", "dim", "vdim", "conv", "rot", "scale", "mask"), where)
        # a mixer whose configuration has no 'rot' rotates nothing, one without 'mask' sees every earlier key
        rot, mask = m.get("rot"), m.get("mask")
        if rot is not None:
            _only(rot, ("dims", "base"), f"{where}.rot")
        if mask is not None:
            _only(mask, ("size",), f"{where}.mask")
        rot_dims = 0 if rot is None else int(_need(rot, "dims", f"{where}.rot"))
        c = cls(heads=int(_need(m, "heads", where)), kv_heads=int(_need(m, "kv_heads", where)),
                dim=int(_need(m, "dim", where)), vdim=int(_need(m, "vdim", where)), conv=int(_need(m, "conv", where)),
                rot_dims=rot_dims, rot_base=None if rot is None else float(_need(rot, "base", f"{where}.rot")),
                scale=float(_need(m, "scale", where)),
                chunk=None if mask is None else int(_need(mask, "size", f"{where}.mask")))
        if min(c.heads, c.kv_heads, c.dim, c.vdim, c.conv, 1 if c.chunk is None else c.chunk) <= 0 or c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: sizes must be positive and heads a multiple of kv_heads")
        if c.rot_dims < 0 or c.rot_dims % 2 or c.rot_dims > c.dim or (c.rot_dims and not c.rot_base > 0):
            raise ConfigError(f"config.json: {where}.rot: dims must be even and at most dim, base positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d = {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
             "scale": self.scale, "vdim": self.vdim}
        if self.rot_base is not None:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.chunk is not None:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass
class RoutedExpertsConfig:
    """Constants of the mixture-of-experts feed-forward (``layers[i].mlp``)."""
    experts: int              # experts that have weights
    identity: int             # further router outputs whose expert passes its input on
    top: int
    expert_ff: int
    shared_ff: Optional[int]  # None: no shared expert

    @classmethod
    def from_dict(cls, m: Dict[str, Any], where: str) -> "RoutedExpertsConfig":
        _only(m, ("kind", "router", "expert", "shared"), where)
        if _need(m, "kind", where) != "moe":
            raise ConfigError(f"config.json: {where}.kind {m['kind']!r}: this design's feed-forward is 'moe'")
        r, e = _need(m, "router", where), _need(m, "expert", where)
        _only(r, ("experts", "identity", "top"), f"{where}.router")
        _only(e, ("ff",), f"{where}.expert")
        shared = m.get("shared")
        if shared is not None:
            _only(shared, ("ff",), f"{where}.shared")
        c = cls(experts=int(_need(r, "experts", f"{where}.router")), identity=int(r.get("identity", 0)),
                top=int(_need(r, "top", f"{where}.router")), expert_ff=int(_need(e, "ff", f"{where}.expert")),
                shared_ff=None if shared is None else int(_need(shared, "ff", f"{where}.shared")))
        if c.experts < 0 or c.identity < 0 or c.top <= 0 or c.top > c.experts + c.identity or c.expert_ff <= 0:
            raise ConfigError(f"config.json: {where}: needs 0 < top <= experts + identity and a positive ff")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d = {"expert": {"ff": self.expert_ff}, "kind": "moe",
             "router": {"experts": self.experts, "identity": self.identity, "top": self.top}}
        if self.shared_ff is not None:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass
class LonasunLayer:
    type: str
    mixer: ChunkedConvAttentionConfig
    mlp: Optional[RoutedExpertsConfig]


@dataclass
class LonasunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[LonasunLayer]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0              # 0: no loop, every layer runs once
    eos_token_id: Optional[Any] = None
    architecture: str = "Lonasun"
    unknown_keys: List[str] = field(default_factory=list)     # keys of config.json this design does not define

    MIXERS = {"attention": ChunkedConvAttentionConfig}

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "LonasunConfig":
        _UNKNOWN.clear()
        _only(cfg, ("architecture", "architectures", "layers", "loop", "norm", "vocab", "width", "eos_token_id"),
              "the top level")
        layers = []
        raw_layers = _need(cfg, "layers", "the top level")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            _only(L, ("type", "mixer", "mlp"), where)
            kind = _need(L, "type", where)
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r}: this design's mixers are {sorted(cls.MIXERS)}")
            mixer = cls.MIXERS[kind].from_dict(_need(L, "mixer", where), f"{where}.mixer")
            mlp = L.get("mlp")
            layers.append(LonasunLayer(kind, mixer,
                                       None if mlp is None else RoutedExpertsConfig.from_dict(mlp, f"{where}.mlp")))
        loop = cfg.get("loop")
        start = stop = times = 0
        if loop is not None:
            _only(loop, ("start", "stop", "times"), "loop")
            start, stop, times = (int(_need(loop, k, "loop")) for k in ("start", "stop", "times"))
            if not (0 <= start < stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: loop {loop}: needs 0 <= start < stop <= {len(layers)} layers and times >= 1")
        out = cls(vocab=int(_need(cfg, "vocab", "the top level")), width=int(_need(cfg, "width", "the top level")),
                  norm_eps=float(_need(_need(cfg, "norm", "the top level"), "eps", "norm")), layers=layers,
                  loop_start=start, loop_stop=stop, loop_times=times, eos_token_id=cfg.get("eos_token_id"))
        if out.vocab <= 0 or out.width <= 0 or not out.norm_eps > 0:
            raise ConfigError("config.json: vocab, width and norm.eps must be positive")
        out.unknown_keys = list(_UNKNOWN)
        if out.unknown_keys:
            warnings.warn(f"config.json has keys the Lonasun design does not define (ignored): {out.unknown_keys}")
        return out

    def layer_runs(self) -> List[tuple]:
        """[(layer, starts a pass of the loop)] in the order the layers run."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, False) for i in range(n)]
        runs = [(i, False) for i in range(self.loop_start)]
        for _ in range(self.loop_times):
            runs += [(i, i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, False) for i in range(self.loop_stop, n)]

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
        if self.loop_times:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        if self.eos_token_id is not None:
            d["eos_token_id"] = copy.deepcopy(self.eos_token_id)
        return d

    def summary(self) -> str:
        runs = self.layer_runs()
        m = self.layers[0].mixer
        return (f"Lonasun layers={len(self.layers)} (runs {len(runs)}) width={self.width} vocab={self.vocab} "
                f"eps={self.norm_eps} first mixer: heads={m.heads}/{m.kv_heads} dim={m.dim}/{m.vdim} "
                f"conv={m.conv} chunk={m.chunk}")
