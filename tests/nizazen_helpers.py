"""Shared by the Nizazen tests: small configurations that differ from one another in every size and option, model
folders with random weights, the plain implementation as ground truth."""

from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List

import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.weights import load_checkpoint
from plain import nizazen_plain as P


def _att(heads, kv_heads, dim, vdim, scale, window):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def _lat(heads, dim, vdim, rank, scale, window=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "scale": scale, "vdim": vdim}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def _dense(ff):
    return {"ff": ff, "kind": "dense"}


def _moe(experts, top, ff, limit):
    return {"expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": {"experts": experts, "top": top}}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


NIZAZEN: Dict[str, dict] = {
    # three lanes; a window that is no multiple of a page, values narrower than keys; a latent narrower than the heads
    # it feeds put together; a layer without a feed-forward whose window is longer than most test sequences
    "P": {"architecture": "Nizazen", "vocab": 200, "width": 96, "norm": {"eps": 1e-6}, "streams": 3, "logit_softcap": 30.0,
          "layers": [_layer(_att(4, 2, 32, 16, 0.2, 20), _dense(160)),
                     _layer(_lat(3, 16, 24, 40, 0.25), _moe(5, 2, 40, 1.5)),
                     _layer(_att(2, 2, 48, 56, 0.15, 133), None)]},
    # one lane WITH lane weights (all of shape one), no soft cap; sizes the tensor-core kernels take: a latent of 64
    # under four heads, key and value heads of 64 with eight query heads on one key head and a window of one page, a
    # latent of 128; one choice per token; an expert limit so small that it clamps most values
    "Q": {"architecture": "Nizazen", "vocab": 160, "width": 128, "norm": {"eps": 1e-5}, "streams": 1,
          "layers": [_layer(_lat(4, 32, 32, 64, 0.18), _moe(4, 1, 64, 0.3)),
                     _layer(_att(8, 1, 64, 64, 0.125, 64), _dense(192)),
                     _layer(_lat(2, 64, 40, 128, 0.1), _dense(96))]},
    # no lanes at all in the configuration (a plain residual sum with the per-channel scale); a window of one position
    # (a query sees itself only); a latent layer WITH a window; every expert chosen; a tight soft cap
    "R": {"architecture": "Nizazen", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 2.0,
          "layers": [_layer(_att(2, 1, 16, 24, 0.3, 1), _moe(3, 3, 16, 2.0)),
                     _layer(_lat(5, 8, 16, 24, 0.35, 17), _dense(40)),
                     _layer(_att(6, 3, 8, 8, 0.35, 9), _moe(7, 3, 24, 1.0))]},
    # latent layers whose whole prompts attend over expanded keys and values (head sizes 64 and 128 for keys and values
    # alike, latents of other sizes), one of them with a window; two lanes
    "S": {"architecture": "Nizazen", "vocab": 120, "width": 64, "norm": {"eps": 1e-5}, "streams": 2, "logit_softcap": 20.0,
          "layers": [_layer(_lat(2, 64, 64, 24, 0.125), _dense(48)),
                     _layer(_lat(3, 128, 128, 192, 0.09, 50), _moe(3, 2, 16, 1.0))]},
    # head sizes and a latent that are no multiple of 8 (padded with zeros when the weights are bound), odd width
    "T": {"architecture": "Nizazen", "vocab": 77, "width": 50, "norm": {"eps": 1e-5}, "streams": 2,
          "layers": [_layer(_att(4, 2, 20, 12, 0.22, 11), _moe(3, 2, 10, 1.5)),
                     _layer(_lat(3, 10, 6, 27, 0.3), _dense(30)),
                     _layer(_lat(2, 5, 9, 12, 0.4, 13), None)]},
}


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: widths that are no power of two, one to five lanes or none, head sizes that
    are multiples of 8 only, windows from one position to longer than any test sequence, layers in any order."""
    rng = random.Random(seed)
    width = rng.choice([48, 72, 96, 128, 200])

    def mixer():
        window = rng.choice([None, 1, 2, 15, 16, 17, 64, 100, 1000])
        if rng.random() < 0.5:
            kv, g = rng.choice([1, 2, 3]), rng.choice([1, 2, 4])
            dim = rng.choice([8, 16, 24, 40, 64, 128])
            return _att(kv * g, kv, dim, rng.choice([dim, 8, 16, 48, 80]), rng.choice([0.1, 0.125, 0.3]), window)
        dim = rng.choice([4, 8, 20, 32, 64])
        return _lat(rng.choice([1, 2, 5, 8]), dim, rng.choice([dim, 4, 8, 24, 40]),
                    rng.choice([8, 24, 64, 104, 128]), rng.choice([0.1, 0.2, 0.3]), rng.choice([None, None, window]))

    def mlp():
        r = rng.random()
        if r < 0.15:
            return None
        if r < 0.55:
            return _dense(rng.choice([8, 40, 100, 192]))
        E = rng.choice([1, 2, 3, 8, 16])
        return _moe(E, rng.randint(1, min(E, 4)), rng.choice([8, 24, 40, 100]), rng.choice([0.5, 2.0, 7.0]))
    cfg = {"architecture": "Nizazen", "vocab": rng.choice([50, 333, 1000]), "width": width,
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": [_layer(mixer(), mlp()) for _ in range(rng.randint(1, 4))]}
    if rng.random() < 0.8:
        cfg["streams"] = rng.choice([1, 2, 3, 4, 5])
    if rng.random() < 0.7:
        cfg["logit_softcap"] = rng.choice([3.0, 12.0, 50.0])
    return cfg


def write_folder(tmp: Path, name: str, seed: int = 0, fixed_choice: bool = False) -> Path:
    """A model folder with random weights.  ``fixed_choice``: the biases of every router are set two apart, so they
    decide which experts are chosen (the same ones for every token of a layer).  The bfloat16 tests use such folders:
    a choice between two experts of nearly equal logits falls either way under bfloat16 rounding and changes the output
    by a whole expert, which would say nothing about the kernels.  Choices that follow the input are tested in float32
    and on the kernels."""
    folder = Path(tmp) / f"nizazen_{name}_{seed}{'_fixed' if fixed_choice else ''}"
    if not (folder / "model.safetensors").exists():
        from flashdecode_cuda_b200.weights.loader import write_model_folder
        fd.write_random_model(folder, NIZAZEN[name], seed)
        if fixed_choice:
            tensors = weights_of(folder)
            for i, layer in enumerate(NIZAZEN[name]["layers"]):
                if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
                    n = tensors[f"l{i}.mlp.router.b"].numel()
                    order = torch.randperm(n, generator=torch.Generator().manual_seed(seed + i))
                    tensors[f"l{i}.mlp.router.b"] = (2.0 * order).to(torch.bfloat16)
            write_model_folder(folder, NIZAZEN[name], tensors)
    return folder


def raw_config(folder: Path) -> dict:
    return json.loads((Path(folder) / "config.json").read_text())


def weights_of(folder: Path) -> Dict[str, torch.Tensor]:
    return {k: v.clone() for k, v in load_checkpoint(folder).items()}


_ORACLE: dict = {}


def oracle_logits(folder: Path, tokens: List[int]) -> torch.Tensor:
    """float64 logits [len, vocab] of one whole sequence from the plain implementation."""
    key = (str(folder), tuple(tokens))
    if key not in _ORACLE:
        _ORACLE[key] = P.forward(raw_config(folder), weights_of(folder), tokens)
    return _ORACLE[key]


def plain_greedy(folder: Path, prompt: List[int], n: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(oracle_logits(folder, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
