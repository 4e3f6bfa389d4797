"""Nizazen without a GPU: configuration, blueprint, the cache's key-only groups, and the plain implementation's
mechanisms against closed forms."""

import copy
import math
import warnings

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.cache.paged import KVGroupSpec, PagedCache
from flashdecode_cuda_b200.config import ConfigError, NizazenConfig
from flashdecode_cuda_b200.engine.model import Model
from nizazen_helpers import NIZAZEN, random_config
from plain import nizazen_plain as P


@pytest.mark.parametrize("name", sorted(NIZAZEN))
def test_configuration_round_trip(name):
    cfg = fd.load_config(NIZAZEN[name])
    assert isinstance(cfg, NizazenConfig) and cfg.to_dict() == NIZAZEN[name]
    assert fd.load_config(cfg.to_dict()).to_dict() == NIZAZEN[name]


def test_configurations_drawn_at_random_round_trip():
    for seed in range(40):
        raw = random_config(seed)
        assert fd.load_config(raw).to_dict() == raw


def test_missing_keys_are_errors_and_unknown_keys_warn():
    for path in (("width",), ("norm", "eps"), ("layers", 0, "mixer", "scale"), ("layers", 1, "mixer", "kv_rank"),
                 ("layers", 1, "mlp", "expert", "limit"), ("layers", 0, "mlp", "ff"), ("layers", 0, "type")):
        raw = copy.deepcopy(NIZAZEN["P"])
        d = raw
        for k in path[:-1]:
            d = d[k]
        del d[path[-1]]
        with pytest.raises(ConfigError):
            fd.load_config(raw)
    raw = copy.deepcopy(NIZAZEN["P"])
    raw["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError):
        fd.load_config(raw)
    raw = copy.deepcopy(NIZAZEN["P"])
    raw["layers"][1]["mixer"]["rope"] = {"base": 10000.0}
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        cfg = fd.load_config(raw)
    assert cfg.unknown_keys == ["layers[1].mixer.rope"] and len(w) == 1


def test_blueprint_parts_lanes_and_cache_groups():
    for name, raw in NIZAZEN.items():
        cfg = fd.load_config(raw)
        m = Model.from_config(cfg, torch.float32, "cpu")
        assert m.blueprint.lanes == (raw.get("streams") or 1)
        names = {s.name for s in m.tensor_specs()}
        for i, L in enumerate(raw["layers"]):
            assert (f"l{i}.hc1.mix" in names) == ("streams" in raw)
            assert (f"l{i}.norm2" in names) == (L["mlp"] is not None) == (f"l{i}.ls2" in names)
            assert (f"l{i}.mix.dkv.norm" in names) == (L["type"] == "latent_attention")
            assert (f"l{i}.mix.q.norm" in names) == (L["type"] == "attention")
        groups = m.cache_groups()
        latent = [g for g in groups if g.keys_only]
        assert sum(g.n_layers for g in latent) == sum(L["type"] == "latent_attention" for L in raw["layers"])
        assert all(g.n_kv_heads == 1 for g in latent)
        assert sum(g.n_layers for g in groups) == len(raw["layers"])
        shapes = {s.name: s.shape for s in m.tensor_specs()}
        if "streams" in raw:
            S = raw["streams"]
            assert shapes["l0.hc1.in"] == (S,) and shapes["l0.hc1.mix"] == (S, S) and shapes["l0.hc1.out"] == (S,)


def test_a_head_size_no_kernel_takes_is_refused_when_the_model_is_built():
    raw = copy.deepcopy(NIZAZEN["R"])
    raw["layers"][1]["mixer"]["kv_rank"] = 520
    with pytest.raises(ValueError):
        Model.from_config(fd.load_config(raw), torch.float32, "cpu")


def test_key_only_group_keeps_one_pool_and_a_window_gives_blocks_back():
    groups = [KVGroupSpec(2, 1, 24, None, None, None, True), KVGroupSpec(1, 2, 16, 9, None, 8)]
    cache = PagedCache(groups, [], num_blocks=12, max_slots=2, max_blocks_per_seq=6, block_size=4,
                       dtype=torch.float32, device="cpu")
    g = cache.groups[0]
    assert g.values is g.keys and g.v_pool(1).data_ptr() == g.k_pool(1).data_ptr()
    assert g.bytes_per_token() == 2 * 24 * 4
    assert cache.groups[1].bytes_per_token() == 2 * (16 + 8) * 4
    s = cache.admit()
    cache.reserve([(s, 22)])
    cache.advance(s, 22)
    assert cache.blocks_in_use() == [6, 3]          # positions 14.. are still seen by the next query: blocks 3, 4, 5
    cache.check_invariants()
    cache.release(s)
    assert cache.blocks_in_use() == [0, 0]
    with pytest.raises(ValueError):
        PagedCache([KVGroupSpec(1, 1, 24, None, None, 8, True)], [], 4, 1, 2, 4, torch.float32, "cpu")


# ---------------------------------------------------------------- the plain implementation against closed forms
def test_plain_norm_and_activation():
    x = torch.full((3, 10), 2.0, dtype=torch.float64)
    assert torch.allclose(P.rmsnorm(x, torch.full((10,), 3.0, dtype=torch.float64), 0.0), torch.full((3, 10), 3.0, dtype=torch.float64))
    assert abs(float(P.rmsnorm(torch.zeros(1, 4, dtype=torch.float64), torch.ones(4, dtype=torch.float64), 1e-4).abs().max())) == 0.0
    z = torch.tensor([0.0, 1.0, -1.0, 3.0], dtype=torch.float64)
    want = [0.0, 0.8411919906082768, -0.15880800939172324, 2.99636]
    assert torch.allclose(P.gelu_tanh(z), torch.tensor(want, dtype=torch.float64), atol=1e-5)


def test_plain_window_visibility():
    S, d = 12, 4
    q = torch.zeros(S, 1, d, dtype=torch.float64)          # equal scores: the output is the mean of the visible values
    k = torch.randn(S, 1, d, dtype=torch.float64)
    v = torch.arange(S, dtype=torch.float64).view(S, 1, 1)
    for window in (None, 1, 3, 50):
        out = P.softmax_attention(q, k, v, 1.0, window)[:, 0, 0]
        for i in range(S):
            lo = 0 if window is None else max(0, i - window + 1)
            assert abs(float(out[i]) - (lo + i) / 2) < 1e-12


def test_plain_latent_attention_equals_attention_over_the_latents():
    """(q . U c) = (U^T q) . c and sum_j a_j V c_j = V sum_j a_j c_j: one key/value head of the latent's size."""
    torch.manual_seed(0)
    S, W, H, d, dv, r = 9, 20, 3, 4, 5, 6
    t = {"m.q": torch.randn(H * d, W), "m.dkv": torch.randn(r, W), "m.dkv.norm": torch.rand(r) + 0.5,
         "m.uk": torch.randn(H * d, r), "m.uv": torch.randn(H * dv, r), "m.o": torch.randn(W, H * dv)}
    t = {k: v.double() for k, v in t.items()}
    h = torch.randn(S, W, dtype=torch.float64)
    m = {"heads": H, "dim": d, "vdim": dv, "kv_rank": r, "scale": 0.4}
    want = P.latent_attention(h, t, "m", m, 1e-5)
    c = P.rmsnorm(h @ t["m.dkv"].T, t["m.dkv.norm"], 1e-5)
    q = (h @ t["m.q"].T).view(S, H, d)
    qc = torch.einsum("shd,hdr->shr", q, t["m.uk"].view(H, d, r))
    ac = P.softmax_attention(qc, c.view(S, 1, r), c.view(S, 1, r), 0.4, None)
    v = torch.einsum("shr,hvr->shv", ac, t["m.uv"].view(H, dv, r))
    assert torch.allclose(v.reshape(S, H * dv) @ t["m.o"].T, want, atol=1e-10)


def test_plain_lanes_reduce_to_a_residual_sum():
    torch.manual_seed(1)
    T, W = 5, 8
    x = torch.randn(1, T, W, dtype=torch.float64)
    w, ls = torch.rand(W, dtype=torch.float64) + 0.5, torch.randn(W, dtype=torch.float64)
    f = lambda z: 2.0 * z + 1.0
    one = torch.ones(1, dtype=torch.float64)
    a = P.lane_sublayer(x, f, w, 1e-6, ls, None, None, None)
    b = P.lane_sublayer(x, f, w, 1e-6, ls, one, one.view(1, 1), one)
    assert torch.allclose(a, b) and torch.allclose(a[0], x[0] + ls * f(P.rmsnorm(x[0], w, 1e-6)))
    # two lanes, the second never read or written: it passes through the mixing matrix alone
    X = torch.randn(2, T, W, dtype=torch.float64)
    M = torch.tensor([[1.0, 0.0], [0.0, 0.5]], dtype=torch.float64)
    out = P.lane_sublayer(X, f, w, 1e-6, ls, torch.tensor([1.0, 0.0], dtype=torch.float64), M,
                          torch.tensor([1.0, 0.0], dtype=torch.float64))
    assert torch.allclose(out[1], 0.5 * X[1]) and torch.allclose(out[0], X[0] + ls * f(P.rmsnorm(X[0], w, 1e-6)))


def test_plain_routing_and_clamped_expert():
    t = {"m.router": torch.eye(4, dtype=torch.float64), "m.router.b": torch.tensor([0.0, 0.0, 0.0, 2.5], dtype=torch.float64)}
    h = torch.tensor([[3.0, 1.0, 2.0, 0.0]], dtype=torch.float64)
    idx, w = P.route(h, t, "m", 2)
    assert idx.tolist() == [[0, 3]]
    e = math.exp(3.0) + math.exp(2.5)
    assert torch.allclose(w, torch.tensor([[math.exp(3.0) / e, math.exp(2.5) / e]], dtype=torch.float64))
    te = {"e.gate": torch.tensor([[1.0], [1.0]], dtype=torch.float64), "e.up": torch.tensor([[1.0], [-1.0]], dtype=torch.float64),
          "e.down": torch.eye(2, dtype=torch.float64)}
    y = P.clamped_expert(torch.tensor([[5.0]], dtype=torch.float64), te, "e", 2.0)
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(y, torch.tensor([[g * 3.0, g * -1.0]], dtype=torch.float64))


def test_plain_logits_are_capped():
    raw = NIZAZEN["R"]
    m = Model.from_config(fd.load_config(raw), torch.float32, "cpu")
    tensors = fd.random_weights(m, 3)
    tensors["head"] = tensors["head"] * 200.0
    lg = P.forward(raw, tensors, [1, 2, 3, 4])
    assert float(lg.abs().max()) <= raw["logit_softcap"] and float(lg.abs().max()) > 0.9 * raw["logit_softcap"]
