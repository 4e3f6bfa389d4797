"""Lonasun without a GPU: the configuration reader, the plain implementation's mechanisms against closed forms, the
cache's chunk groups and separate value sizes, and the blueprint."""

import copy

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200.cache.paged import KVGroupSpec, PagedCache
from flashdecode_cuda_b200.config import ConfigError, load_config
from flashdecode_cuda_b200.engine.model import Model
from lonasun_helpers import LONASUN
from plain import lonasun_plain as P


# ---------------------------------------------------------------- configuration
@pytest.mark.parametrize("name", sorted(LONASUN))
def test_config_round_trip(name):
    cfg = load_config(LONASUN[name])
    assert cfg.architecture == "Lonasun"
    assert cfg.to_dict() == LONASUN[name]
    assert load_config(cfg.to_dict()).to_dict() == cfg.to_dict()


def test_layer_runs_follow_the_loop():
    assert load_config(LONASUN["X"]).layer_runs() == [(0, True), (1, False)] * 3 + [(2, False)]
    assert load_config(LONASUN["Y"]).layer_runs() == [(0, False), (1, False)]
    assert load_config(LONASUN["Z"]).layer_runs() == [(0, False), (1, True), (2, False)]
    assert P.layer_runs(LONASUN["X"]) == load_config(LONASUN["X"]).layer_runs()


def test_config_errors_name_the_place():
    bad = copy.deepcopy(LONASUN["X"])
    del bad["layers"][1]["mixer"]["vdim"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer misses 'vdim'"):
        load_config(bad)
    odd = copy.deepcopy(LONASUN["X"])
    odd["layers"][0]["mixer"]["sink"] = 4
    with pytest.warns(UserWarning, match="does not define"):
        cfg = load_config(odd)
    assert cfg.unknown_keys == ["layers[0].mixer.sink"] and cfg.to_dict() == LONASUN["X"]
    bad = copy.deepcopy(LONASUN["X"])
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(ConfigError, match="mixers are"):
        load_config(bad)
    bad = copy.deepcopy(LONASUN["X"])
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        load_config(bad)
    bad = copy.deepcopy(LONASUN["Z"])
    bad["layers"][0]["mlp"]["router"]["top"] = 6
    with pytest.raises(ConfigError, match="top"):
        load_config(bad)


def test_a_mixer_without_mask_or_rotation_in_its_configuration():
    plain = copy.deepcopy(LONASUN["Z"])
    for layer in plain["layers"]:
        del layer["mixer"]["mask"]
    del plain["layers"][0]["mixer"]["rot"]
    cfg = load_config(plain)
    assert [L.mixer.chunk for L in cfg.layers] == [None] * 3 and cfg.layers[0].mixer.rot_dims == 0
    m = Model.from_config(cfg, torch.float32, "cpu")
    assert all(g.chunk is None for g in m.cache_groups())
    assert "mask" not in cfg.to_dict()["layers"][1]["mixer"]


def test_blueprint_declares_every_tensor_once_and_orders_the_runs():
    cfg = load_config(LONASUN["X"])
    m = Model.from_config(cfg, torch.float32, "cpu")
    names = [s.name for s in m.tensor_specs()]
    assert len(names) == len(set(names))
    assert {"embed", "loop.in", "final.norm", "head", "l0.mix.q.conv", "l2.mlp.e2.down", "l0.mlp.shared.up",
            "l1.mlp.correction"} <= set(names)
    assert "l2.mlp.shared.up" not in names and "l2.mlp.e3.up" not in names
    assert [(r.layer, r.before) for r in m.schedule] == [(0, "loop_in"), (1, None)] * 3 + [(2, None)]
    # two kinds of storage: (2 key heads of 32 with values of 48, chunk 24) six times and (1 of 48 / 16, chunk 37) once
    groups = {(g.n_kv_heads, g.head_dim, g.value_dim, g.chunk): g.n_layers for g in m.cache_groups()}
    assert groups == {(2, 32, 48, 24): 6, (1, 48, 16, 37): 1}
    # a layer without a feed-forward declares no expert, and its second norm only as an option
    y = Model.from_config(load_config(LONASUN["Y"]), torch.float32, "cpu")
    spec = {s.name: s for s in y.tensor_specs()}
    assert spec["l1.norm2"].optional and not spec["l0.norm2"].optional and "l1.mlp.router" not in spec
    assert "loop.in" not in spec


# ---------------------------------------------------------------- the plain mechanisms
def test_plain_norm_has_a_unit_offset():
    x = torch.tensor([[3.0, -4.0]], dtype=torch.float64)
    y = P.unit_offset_rmsnorm(x, torch.tensor([0.0, 1.0], dtype=torch.float64), 0.0)
    rms = (12.5) ** 0.5
    assert torch.allclose(y, torch.tensor([[3.0 / rms, -8.0 / rms]], dtype=torch.float64))


def test_plain_short_conv_is_causal_and_ordered():
    u = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=torch.float64)
    w = torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64)        # the last tap sits on the current step
    assert P.short_conv(u, w).flatten().tolist() == [1.0, 12.0, 123.0, 1230.0]


def test_plain_partial_rotation():
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    y = P.partial_rotation(x, torch.arange(5), 4, 100.0)
    assert torch.equal(y[..., 4:], x[..., 4:])                       # only the first four dimensions move
    assert torch.equal(y[0], x[0])                                   # position 0: no rotation
    assert torch.allclose(y[..., :4].norm(dim=-1), x[..., :4].norm(dim=-1))
    # pair (0, 2) turns by the position, pair (1, 3) by position / 10
    u, v = x[3, 0, 0], x[3, 0, 2]
    assert torch.allclose(y[3, 0, 0], u * torch.cos(torch.tensor(3.0)) - v * torch.sin(torch.tensor(3.0)))
    u, v = x[3, 0, 1], x[3, 0, 3]
    assert torch.allclose(y[3, 0, 3], v * torch.cos(torch.tensor(0.3)) + u * torch.sin(torch.tensor(0.3)))


def test_plain_chunks():
    assert P.chunk_visible(7, 4, 4) and not P.chunk_visible(7, 3, 4) and not P.chunk_visible(4, 5, 4)
    assert P.chunk_visible(4, 4, 4) and P.chunk_visible(3, 0, 4)
    q, k, v = (torch.randn(11, 4, 8, dtype=torch.float64), torch.randn(11, 2, 8, dtype=torch.float64),
               torch.randn(11, 2, 6, dtype=torch.float64))
    slow, fast = P.chunked_attention(q, k, v, 0.3, 4), P.chunked_attention_fast(q, k, v, 0.3, 4)
    assert torch.allclose(slow, fast)
    assert torch.allclose(slow[8], v[8].repeat_interleave(2, 0))      # the first position of a chunk sees itself only


def test_plain_routing():
    h = torch.randn(6, 10, dtype=torch.float64)
    router = torch.randn(7, 10, dtype=torch.float64)
    corr = torch.zeros(7, dtype=torch.float64)
    chosen, w = P.route(h, router, corr, 3)
    s = torch.softmax(h @ router.T, -1)
    assert torch.equal(chosen, s.topk(3).indices)
    assert torch.allclose(w.sum(-1), torch.ones(6, dtype=torch.float64))
    corr[5] = 10.0                                                   # the correction moves the choice, not the weights
    chosen2, w2 = P.route(h, router, corr, 3)
    assert (chosen2[:, 0] == 5).all()
    picked = torch.gather(s, 1, chosen2)
    assert torch.allclose(w2, picked / picked.sum(-1, keepdim=True))


def test_plain_identity_experts_pass_the_input_on():
    h = torch.randn(4, 8, dtype=torch.float64)
    W = {"l0.mlp.router": torch.randn(3, 8, dtype=torch.float64), "l0.mlp.correction": torch.zeros(3, dtype=torch.float64)}
    m = {"kind": "moe", "router": {"experts": 0, "identity": 3, "top": 2}, "expert": {"ff": 4}}
    assert torch.allclose(P.moe_feed_forward(h, W, "l0", m), h)      # the weights of the chosen sum to one


# ---------------------------------------------------------------- the cache
def test_chunk_group_gives_back_blocks_before_the_chunk():
    c = PagedCache([KVGroupSpec(1, 1, 8, None, 10, None)], [], num_blocks=16, max_slots=2, max_blocks_per_seq=16,
                   block_size=4, dtype=torch.float32, device="cpu")
    s = c.admit()
    c.reserve([(s, 9)]); c.advance(s, 9)
    assert c.blocks_in_use() == [3]                  # the next query (9) is in chunk 0..9: all kept
    c.reserve([(s, 1)]); c.advance(s, 1)
    assert c.blocks_in_use() == [1]                  # the next query (10) starts chunk 10..19: blocks 0, 1 go, block 2 holds 8..11
    assert c.slots[s].blocks[0][:3] == [-1, -1, c.slots[s].blocks[0][2]]
    c.reserve([(s, 13)]); c.advance(s, 13)           # 23 tokens: the next query sees 20..: blocks of 0..19 go
    assert c.blocks_in_use() == [1]
    assert c.kv_bytes([s]) == 3 * c.groups[0].bytes_per_token()      # position 22 saw 20, 21, 22
    c.check_invariants()
    c.release(s)
    assert c.blocks_in_use() == [0]


def test_keys_and_values_of_different_sizes_have_a_pool_each():
    c = PagedCache([KVGroupSpec(2, 3, 8, None, None, 24)], [], num_blocks=4, max_slots=1, max_blocks_per_seq=4,
                   block_size=4, dtype=torch.float32, device="cpu")
    g = c.groups[0]
    assert g.k_pool(1).shape == (4, 3, 4, 8) and g.v_pool(1).shape == (4, 3, 4, 24)
    assert g.bytes_per_token() == 2 * 3 * (8 + 24) * 4
    s = c.admit()
    c.reserve([(s, 5)]); c.advance(s, 5)
    b, off = c.slot_of(s, 4)
    g.keys[1, b, :, off] = 7.0
    g.values[1, b, :, off] = 9.0
    k, v = c.gather(s, 0, 1)
    assert k.shape == (5, 3, 8) and v.shape == (5, 3, 24) and float(k[4].min()) == 7.0 and float(v[4].min()) == 9.0
    same = PagedCache([KVGroupSpec(1, 1, 8)], [], 2, 1, 2, 4, torch.float32, "cpu").groups[0]
    assert same.k_pool(0).shape == same.v_pool(0).shape == (2, 1, 4, 8)


def test_random_model_folder_round_trip(tmp_path):
    folder = fd.write_random_model(tmp_path / "m", LONASUN["Z"], seed=3)
    cfg = load_config(folder)
    assert cfg.to_dict() == LONASUN["Z"]
    w = fd.weights.load_checkpoint(folder)
    assert w["loop.in"].shape == (64, 128) and w["l0.mix.q.conv"].shape == (512, 1) and w["l2.mlp.router"].shape == (6, 64)
    assert abs(float(w["l0.norm1"].float().mean())) < 0.1            # norm weights are offsets from one
