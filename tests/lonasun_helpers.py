"""Shared by the Lonasun tests: small configurations that differ from one another in every size and option, model
folders with random weights, the plain implementation as ground truth."""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List

import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.weights import load_checkpoint
from plain import lonasun_plain as P


def _mixer(heads, kv_heads, dim, vdim, conv, rot_dims, base, scale, chunk):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk},
            "rot": {"base": base, "dims": rot_dims}, "scale": scale, "vdim": vdim}


def _moe(experts, identity, top, ff, shared_ff):
    d = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}}
    if shared_ff is not None:
        d["shared"] = {"ff": shared_ff}
    return d


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


LONASUN: Dict[str, dict] = {
    # value heads wider than key heads, four taps, a looped span at the very start that runs three times, an odd chunk
    "X": {"architecture": "Lonasun", "vocab": 200, "width": 96, "norm": {"eps": 1e-6},
          "layers": [_layer(_mixer(4, 2, 32, 48, 4, 8, 10000.0, 0.2, 24), _moe(5, 2, 3, 40, 56)),
                     _layer(_mixer(4, 2, 32, 48, 4, 8, 10000.0, 0.2, 24), _moe(5, 2, 3, 40, 56)),
                     _layer(_mixer(2, 1, 48, 16, 3, 48, 500.0, 0.11, 37), _moe(3, 1, 2, 24, None))],
          "loop": {"start": 0, "stop": 2, "times": 3}},
    # head size 128 for keys and values (the widest tensor-core kernels), one query head per key head, two taps, every
    # dimension rotated, a chunk that is no multiple of a page or tile, one choice per token, no identity and no shared
    # expert, a layer without a feed-forward, no loop
    "Y": {"architecture": "Lonasun", "vocab": 160, "width": 128, "norm": {"eps": 1e-5},
          "layers": [_layer(_mixer(2, 2, 128, 128, 2, 128, 250000.0, 0.09, 100), _moe(4, 0, 1, 64, None)),
                     _layer(_mixer(2, 2, 128, 128, 2, 128, 250000.0, 0.09, 100), None)]},
    # eight query heads on one key head, one tap (no state), nothing rotated, a chunk of exactly one page, more
    # identity experts than experts, a loop of one pass over the middle layer
    "Z": {"architecture": "Lonasun", "vocab": 96, "width": 64, "norm": {"eps": 1e-5},
          "layers": [_layer(_mixer(8, 1, 64, 64, 1, 0, 10000.0, 0.125, 64), _moe(2, 3, 2, 32, 32)),
                     _layer(_mixer(8, 1, 64, 64, 1, 0, 10000.0, 0.125, 64), _moe(2, 3, 2, 32, 32)),
                     _layer(_mixer(2, 2, 64, 64, 3, 16, 10000.0, 0.125, 16), _moe(6, 0, 6, 16, 16))],
          "loop": {"start": 1, "stop": 2, "times": 1}},
}


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: widths that are no power of two, head sizes that are multiples of 8 only, value
    heads of another size than key heads, one to five taps, nothing to everything rotated, chunks from one position to
    longer than any test sequence, routers with and without identity and shared experts, layers without a feed-forward,
    layers that differ from one another, and loops anywhere in the stack."""
    import random
    rng = random.Random(seed)
    width = rng.choice([48, 72, 96, 128, 200, 256])
    n_layers = rng.randint(1, 4)

    def mixer():
        kv, g = rng.choice([1, 2, 3]), rng.choice([1, 2, 4])
        dim = rng.choice([8, 16, 24, 32, 40, 64, 128])
        vdim = rng.choice([dim, dim, 8, 16, 48, 64])
        rot = min(dim, rng.choice([0, 2, 4, 8, dim]))
        m = _mixer(kv * g, kv, dim, vdim, rng.choice([1, 2, 3, 4, 5]), rot - rot % 2, rng.choice([100.0, 10000.0, 250000.0]),
                   rng.choice([0.1, 0.125, 0.3]), rng.choice([1, 3, 16, 17, 50, 64, 100, 1000]))
        if rng.random() < 0.15:
            del m["mask"]                              # every earlier key is visible
        if rng.random() < 0.1:
            del m["rot"]                               # nothing is rotated
        return m

    def mlp():
        if rng.random() < 0.15:
            return None
        E, n_id = rng.choice([1, 2, 3, 8, 16]), rng.choice([0, 0, 1, 4])
        return _moe(E, n_id, rng.randint(1, min(E + n_id, 5)), rng.choice([8, 24, 40, 96, 100]),
                    rng.choice([None, 16, 56, 128]))
    same = rng.random() < 0.5
    m0, f0 = mixer(), mlp()
    cfg = {"architecture": "Lonasun", "vocab": rng.choice([50, 333, 1000]), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
           "layers": [_layer(m0 if same else mixer(), f0 if same else mlp()) for _ in range(n_layers)]}
    if rng.random() < 0.7:
        a = rng.randint(0, n_layers - 1)
        cfg["loop"] = {"start": a, "stop": rng.randint(a + 1, n_layers), "times": rng.randint(1, 3)}
    return cfg


def write_folder(tmp: Path, name: str, seed: int = 0, fixed_choice: bool = False) -> Path:
    """A model folder with random weights.  ``fixed_choice``: the corrections of every router are set two apart, so
    they alone decide which experts are chosen (the same ones for every token of a layer), while the weights of the
    chosen still follow the scores.  The bfloat16 tests use such folders: a choice between two experts of nearly equal
    score falls either way under bfloat16 rounding and changes the output by a whole expert, which would say nothing
    about the kernels.  Choices that follow the input are tested in float32 and, one layer at a time, on the kernels."""
    folder = Path(tmp) / f"lonasun_{name}_{seed}{'_fixed' if fixed_choice else ''}"
    if not (folder / "model.safetensors").exists():
        from flashdecode_cuda_b200.weights.loader import write_model_folder
        fd.write_random_model(folder, LONASUN[name], seed)
        if fixed_choice:
            tensors = weights_of(folder)
            for i, layer in enumerate(LONASUN[name]["layers"]):
                if layer["mlp"] is not None:
                    n = tensors[f"l{i}.mlp.correction"].numel()
                    order = torch.randperm(n, generator=torch.Generator().manual_seed(seed + i))
                    tensors[f"l{i}.mlp.correction"] = (2.0 * order).to(torch.bfloat16)
            write_model_folder(folder, LONASUN[name], tensors)
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
