"""Nizazen on the GPU against the plain implementation: each mechanism's kernels alone, then whole models in float32
and bfloat16 - whole prompts, token-by-token decoding, portions down to two tokens, unequal batches against each
request alone, slots and pages used again, keys far back, at page borders and on both sides of every window's edge,
long decoding, greedy generation through the engine's entry point and scheduler, and the trace runner."""

import json
import subprocess
import sys
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200 import kernels as K
from flashdecode_cuda_b200.engine.model import Workspace
from flashdecode_cuda_b200.parts.base import Runtime
from flashdecode_cuda_b200.parts.mlp import GatedMLP
from flashdecode_cuda_b200.parts.moe import RoutedExperts
from helpers import prompts_for, rel_err
from nizazen_helpers import NIZAZEN, oracle_logits, plain_greedy, random_config, raw_config, weights_of, write_folder
from plain import nizazen_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda"
NAMES = ["P", "Q", "R", "S", "T"]
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KTOL = {"float32": 2e-5, "bfloat16": 2e-2}
# Whole models, relative to the largest logit.  float32: only the order of summation differs from the float64 ground
# truth.  bfloat16: what a wrong mask, lane or page does is told apart by the float32 runs and by the kernel tests
# with keys that stand out, not by this number.
TOL = {"float32": 1e-5, "bfloat16": 5e-2}


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def step_arrays(ctx_lens, q_lens, slots):
    tok_row, tok_pos, starts = [], [], []
    for r, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        starts.append(len(tok_row))
        tok_row += [r] * n
        tok_pos += list(range(c, c + n))
    return i32(tok_row), i32(tok_pos), i32(slots), i32(starts), i32(q_lens), i32(ctx_lens)


def fake_ctx(T, dtype):
    rt = Runtime(torch.device(DEV), dtype, torch.zeros(1, dtype=torch.int32, device=DEV), K.sm_count())
    return SimpleNamespace(T=T, ws=Workspace(torch.device(DEV)), rt=rt, upcoming=None), rt


# ---------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S,H,T", [(1, 48, 5), (2, 200, 9), (3, 96, 4), (5, 64, 3), (8, 40, 2), (4, 4096, 2)])
def test_lane_connection(dtype, S, H, T):
    """The pending update of all lanes from the old ones, then the read mixture and its norm; rows gathered; a read
    that leaves the lanes alone; float partial sums."""
    torch.manual_seed(S * 100 + H)
    dt = TD[dtype]
    X = torch.randn(S, T, H, dtype=torch.float64)
    y = torch.randn(T, H).to(dt)
    gain, w = torch.randn(H), torch.rand(H) + 0.5
    mix, back, read = torch.eye(S) + 0.3 * torch.randn(S, S), torch.randn(S), torch.randn(S)
    eps = 1e-5
    new = torch.einsum("sr,stw->rtw", mix.double(), X) + back.double()[:, None, None] * (gain.double() * y.double())[None]
    u = torch.einsum("s,stw->tw", read.double(), new)
    want = P.rmsnorm(u, w.double(), eps)
    lanes0 = X.permute(1, 0, 2).reshape(T, S * H).float().to(DEV).contiguous()
    dev = lambda t: t.to(DEV).contiguous()
    lanes = lanes0.clone()
    out = torch.zeros(T, H, dtype=dt, device=DEV)
    K.lanes_norm(dev(y), dev(gain), dev(mix), dev(back), lanes, dev(read), dev(w), eps, out, S)
    assert rel_err(out, want) < KTOL[dtype]
    assert rel_err(lanes.view(T, S, H).permute(1, 0, 2), new) < 1e-5
    # the same from three float partial sums, two rows gathered, nothing written
    if dtype == "bfloat16" or True:
        parts = torch.randn(3, T, H)
        parts[0] = y.float() - parts[1] - parts[2]
        rows = i32([T - 1, 0])
        lanes = lanes0.clone()
        out2 = torch.zeros(2, H, dtype=dt, device=DEV)
        K.lanes_norm(dev(parts), dev(gain), dev(mix), dev(back), lanes, dev(read), dev(w), eps, out2, S, rows=rows,
                     write_lanes=False)
        assert rel_err(out2, want[[T - 1, 0]]) < KTOL[dtype] and torch.equal(lanes, lanes0)
    # nothing pending, lanes added up (what the final norm does), and the sum of the lanes for traces
    out3 = torch.zeros(T, H, dtype=dt, device=DEV)
    K.lanes_norm(None, None, None, None, lanes0.clone(), None, dev(w), eps, out3, S)
    assert rel_err(out3, P.rmsnorm(X.sum(0), w.double(), eps)) < KTOL[dtype]
    total = torch.zeros(T, H, device=DEV)
    K.lanes_sum(dev(y), dev(gain), dev(mix), dev(back), lanes0, total, S)
    assert rel_err(total, new.sum(0)) < 1e-5
    filled = torch.zeros(T, S * H, device=DEV)
    K.lanes_fill(dev(X[0].float()), filled, S)
    assert torch.equal(filled.view(T, S, H)[:, S - 1], dev(X[0].float()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,d,dv,cuts", [(4, 2, 16, 8, [5, 1, 1, 6]), (3, 1, 24, 0, [2, 2, 9]), (2, 2, 64, 64, [7, 1])])
def test_norm_over_the_whole_projection_and_append(dtype, n_q, n_kv, d, dv, cuts):
    """q and k normed over all their heads at once (or passed on as they are), k and v in the pages of two sequences
    fed in portions; dv 0: keys only."""
    torch.manual_seed(d)
    dt = TD[dtype]
    nq, nk, nv = n_q * d, n_kv * d, n_kv * dv
    bs, n_cols, slots = 4, 8, [2, 0]
    total = sum(cuts)
    proj = [torch.randn(total, nq + nk + nv + 8).to(dt) for _ in range(2)]          # a few columns that belong to nobody
    qw, kw = torch.rand(nq) + 0.5, torch.rand(nk) + 0.5
    k_pool = torch.zeros(2 * n_cols, n_kv, bs, d, dtype=dt, device=DEV)
    v_pool = torch.zeros(2 * n_cols, n_kv, bs, dv, dtype=dt, device=DEV) if dv else None
    table = torch.full((3, n_cols), -1, dtype=torch.int32, device=DEV)
    perm = torch.randperm(2 * n_cols).to(torch.int32).to(DEV)
    table[2], table[0] = perm[:n_cols], perm[n_cols:]
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for normed in (True, False):
        q_got = [[], []]
        at = 0
        for n in cuts:
            tok_row, tok_pos, row_slot, *_ = step_arrays([at, at], [n, n], slots)
            x = torch.cat([proj[0][at:at + n], proj[1][at:at + n]]).to(DEV).contiguous()
            q = torch.zeros(2 * n, nq, dtype=dt, device=DEV)
            K.norm_append(x, q, qw.to(DEV) if normed else None, kw.to(DEV) if normed else None, 1e-5, tok_row, tok_pos,
                          row_slot, k_pool, v_pool, table, n_kv, True, status)
            q_got[0].append(q[:n].float().cpu())
            q_got[1].append(q[n:].float().cpu())
            at += n
        assert int(status.item()) == 0
        for r in range(2):
            x = proj[r].double()
            q_want = P.rmsnorm(x[:, :nq], qw.double(), 1e-5) if normed else x[:, :nq]
            k_want = P.rmsnorm(x[:, nq:nq + nk], kw.double(), 1e-5) if normed else x[:, nq:nq + nk]
            assert rel_err(torch.cat(q_got[r]), q_want) < KTOL[dtype]
            blocks = table[slots[r]].tolist()
            k_got = torch.stack([k_pool[blocks[p // bs], :, p % bs] for p in range(total)]).reshape(total, nk)
            assert rel_err(k_got, k_want) < KTOL[dtype]
            if dv:
                v_got = torch.stack([v_pool[blocks[p // bs], :, p % bs] for p in range(total)]).reshape(total, nv)
                assert torch.equal(v_got.cpu(), proj[r][:, nq + nk:nq + nk + nv])


def _window_case(dtype, d, dv, G, n_kv, window, bs, S, portions, seed, shared=False):
    """Every seventh key stands out: it is the first key inside the window of one query and the first outside the
    window of the next, so a visibility that is one position off changes a result by the size of a value.  ``shared``:
    one pool serves as keys and as values (attention over cached latents)."""
    torch.manual_seed(seed)
    dt = TD[dtype]
    n_q = G * n_kv
    q = torch.randn(S, n_q, d) * 0.3
    k = torch.randn(S, n_kv, d) * 0.3
    e = torch.zeros(d)
    e[3] = 1.0
    k[::7] += 6.0 * e
    q += 2.0 * e
    v = k.clone() if shared else torch.randn(S, n_kv, dv)
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = 0.7
    want = P.softmax_attention(q.double(), k.double(), v.double(), scale, window).reshape(S, n_q * dv)
    n_cols = -(-S // bs)
    k_pool = torch.zeros(n_cols + 3, n_kv, bs, d, dtype=dt, device=DEV)
    v_pool = k_pool if shared else torch.zeros(n_cols + 3, n_kv, bs, dv, dtype=dt, device=DEV)
    perm = torch.randperm(n_cols + 3)[:n_cols]
    table = torch.full((2, n_cols), -1, dtype=torch.int32, device=DEV)
    table[1] = perm.to(torch.int32).to(DEV)
    for p in range(S):
        k_pool[perm[p // bs], :, p % bs] = k[p].to(DEV)
        if not shared:
            v_pool[perm[p // bs], :, p % bs] = v[p].to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    got = torch.zeros(S, n_q * dv)
    at = 0
    for n in portions:
        n = min(n, S - at)
        if n <= 0:
            break
        tok_row, _, row_slot, q_start, q_len, ctx_len = step_arrays([at], [n], [1])
        out = torch.full((n, n_q * dv), float("nan"), dtype=dt, device=DEV)
        n_splits, split_len, scratch = 1, 0, None
        if n == 1 and at + 1 > 64:
            split_len = 64
            n_splits = -(-(at + 1) // split_len)
            scratch = torch.zeros(K.attention_scratch_floats(1, n_q, dv, n_splits), device=DEV)
        K.attention(q[at:at + n].reshape(n, n_q * d).to(DEV).contiguous(), k_pool, v_pool, out, table, tok_row, row_slot,
                    q_start, q_len, ctx_len, 1, n, n_q, n_kv, d, scale, window or 0, n_splits, split_len, scratch, status)
        got[at:at + n] = out.float().cpu()
        at += n
    assert at == S and int(status.item()) == 0
    err = (got.double() - want).abs().max(dim=1).values / want.abs().max()
    assert float(err.max()) < KTOL[dtype], f"first wrong position {int((err >= KTOL[dtype]).nonzero()[0])} (window {window})"


WINDOW_CASES = [  # d, dv, G, n_kv, window, block size, length
    (32, 16, 2, 2, 20, 8, 150),        # values narrower than keys: the CUDA-core kernel; edges inside pages
    (64, 64, 8, 1, 64, 64, 260),       # tensor-core kernels of head size 64; a window of exactly a page
    (64, 64, 2, 2, 16, 16, 100),       # every window edge on a page border
    (128, 128, 1, 2, 100, 64, 330),    # head size 128: the widest prompt kernel
    (48, 56, 1, 2, 133, 4, 300),
    (16, 24, 2, 1, 1, 8, 40),          # a query sees itself only
    (8, 8, 2, 3, 9, 16, 90),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", WINDOW_CASES)
def test_window_edges_in_whole_prompts(dtype, case):
    d, dv, G, n_kv, window, bs, S = case
    _window_case(dtype, d, dv, G, n_kv, window, bs, S, [S], seed=1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", WINDOW_CASES)
def test_window_edges_in_portions_and_token_by_token(dtype, case):
    d, dv, G, n_kv, window, bs, S = case
    _window_case(dtype, d, dv, G, n_kv, window, bs, S, [window + 3, 2, window, 3, 129, 2] + [1] * S, seed=2)
    _window_case(dtype, d, dv, G, n_kv, window, bs, min(S, 2 * window + 20), [1] * S, seed=3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("r,G,window,bs,S", [(40, 3, None, 8, 300), (64, 4, None, 16, 700), (128, 2, None, 64, 400),
                                             (88, 7, None, 64, 1100), (24, 5, 17, 8, 120),
                                             # more query heads than the tensor-core decode kernel takes in one group:
                                             # cut into groups of 8, of 5, and (a prime) left to the CUDA-core kernel
                                             (64, 32, None, 16, 300), (128, 20, None, 64, 330), (64, 17, None, 8, 200),
                                             (128, 40, 50, 16, 200),
                                             # latents wider than 128: prompts on the mma.sync kernel's wide forms
                                             (256, 8, None, 64, 500), (192, 3, 40, 16, 300),
                                             # wider than any tensor-core kernel takes: the CUDA-core kernel's narrow tiles
                                             (384, 4, None, 16, 200), (512, 8, 70, 64, 260), (320, 32, None, 8, 90)])
def test_attention_over_cached_latents_far_keys(dtype, r, G, window, bs, S):
    """One pool read as keys and as values by all query heads; keys that stand out lie hundreds of positions back."""
    _window_case(dtype, r, r, G, 1, window, bs, S, [S], seed=4, shared=True)
    _window_case(dtype, r, r, G, 1, window, bs, S, [S - 40, 3] + [1] * 40, seed=5, shared=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,heads,N,Kd", [(1, 3, 40, 16), (9, 8, 96, 32), (70, 2, 24, 100), (33, 5, 130, 8)])
def test_per_head_products(dtype, T, heads, N, Kd):
    torch.manual_seed(T)
    dt = TD[dtype]
    a, w = torch.randn(T, heads, Kd).to(dt), (torch.randn(heads, N, Kd) / Kd ** 0.5).to(dt)
    out = torch.zeros(T, heads * N, dtype=dt, device=DEV)
    K.head_gemm(a.view(T, heads * Kd).to(DEV), w.to(DEV), out)
    assert rel_err(out.view(T, heads, N), torch.einsum("thk,hnk->thn", a.double(), w.double())) < KTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,H,ff,T,limit", [(5, 2, 96, 40, 37, 1.5), (4, 1, 64, 24, 9, 0.3), (3, 3, 32, 16, 70, 2.0),
                                                (9, 4, 40, 8, 33, 7.0), (3, 2, 64, 48, 300, 1.0), (4, 2, 72, 20, 19, 2.0),
                                                (3, 2, 256, 192, 400, 2.0)])      # the last: products on tcgen05 in bfloat16
def test_routing_by_biased_logits_and_clamped_gated_experts(dtype, E, top, H, ff, T, limit):
    torch.manual_seed(E * 10 + top)
    dt = TD[dtype]
    h = torch.randn(T, H).to(dt)
    W = {"m.router": (torch.randn(E, H) * 0.3).to(dt), "m.router.b": torch.randn(E).to(dt)}
    for e in range(E):
        W[f"m.e{e}.gate"] = (2 * torch.randn(ff, H) / H ** 0.5).to(dt)       # large enough for the limit to clamp
        W[f"m.e{e}.up"] = (2 * torch.randn(ff, H) / H ** 0.5).to(dt)
        W[f"m.e{e}.down"] = (torch.randn(H, ff) / ff ** 0.5).to(dt)
    cfg = {"kind": "moe", "router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}}
    W64 = {k: v.double() for k, v in W.items()}
    want = P.expert_mixture(h.double(), W64, "m", cfg)
    idx_want, w_want = P.route(h.double(), W64, "m", top)
    x = h.to(DEV)
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, top, device=DEV)
    K.moe_route(x, W["m.router"].to(DEV), None, ids, wts, bias=W["m.router.b"].float().to(DEV))
    assert torch.equal(ids.cpu().long(), idx_want)                 # margins of random logits are far above rounding
    assert rel_err(wts, w_want) < 1e-5
    ctx, rt = fake_ctx(T, dt)
    part = RoutedExperts("m", H, E, top, ff, correction=False, expert_act="clamped_swish", limit=limit, router_bias=True)
    part.bind({k: v.to(DEV) for k, v in W.items()}, rt)
    got = part.forward(ctx, x)
    assert int(rt.status.item()) == 0
    assert rel_err(got, want) < KTOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,I,T", [(48, 40, 1), (96, 160, 7), (128, 192, 40), (256, 512, 300)])
def test_gated_feed_forward_with_biases(dtype, H, I, T):
    torch.manual_seed(I)
    dt = TD[dtype]
    W = {"f.gate": (2 * torch.randn(I, H) / H ** 0.5), "f.up": torch.randn(I, H) / H ** 0.5, "f.down": torch.randn(H, I) / I ** 0.5,
         "f.gate.b": torch.randn(I), "f.up.b": torch.randn(I), "f.down.b": torch.randn(H)}
    W = {k: v.to(dt) for k, v in W.items()}
    h = torch.randn(T, H).to(dt)
    want = P.dense_ff(h.double(), {k: v.double() for k, v in W.items()}, "f")
    ctx, rt = fake_ctx(T, dt)
    part = GatedMLP("f", H, I, "gelu_tanh", True)
    part.bind({k: v.to(DEV) for k, v in W.items()}, rt)
    assert rel_err(part.forward(ctx, h.to(DEV)), want) < KTOL[dtype]


def test_soft_cap():
    x = torch.randn(7, 333, device=DEV) * 40
    want = 11.0 * torch.tanh(x.double() / 11.0)
    K.softcap(x, 11.0)
    assert rel_err(x, want) < 1e-6


# ---------------------------------------------------------------- whole models
class Folders(dict):
    def __missing__(self, key):
        return self[(key, "float32")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("nizazen")
    return Folders({(n, d): write_folder(tmp, n, seed=21, fixed_choice=d == "bfloat16") for n in NAMES for d in DTYPES})


@pytest.fixture(scope="module")
def engines(folders):
    return {(n, d): fd.load(folders[(n, d)], device="cuda", dtype=d) for n in NAMES for d in DTYPES}


def _vocab(name):
    return NIZAZEN[name]["vocab"]


def _lengths(name):
    return {"P": [1, 2, 19, 20, 21, 75, 140], "Q": [3, 64, 65, 260], "R": [1, 9, 10, 17, 18, 129],
            "S": [1, 2, 50, 51, 130, 200], "T": [1, 11, 12, 14, 90]}[name]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("block_size", [8, 64])
def test_whole_prompts(engines, folders, name, dtype, block_size):
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=320, block_size=block_size)
    for p in prompts_for(_vocab(name), _lengths(name), seed=1):
        slot = cache.admit()
        got = eng.model.step(cache, [slot], [p], "all")
        assert rel_err(got, oracle_logits(folders[(name, dtype)], p)) < TOL[dtype], f"prompt of {len(p)} tokens"
        cache.release(slot)
    eng.model.check_status()
    cache.check_invariants()


def test_every_layer_in_float32(engines, folders):
    """The lanes added up after every layer against the plain ones."""
    for name in NAMES:
        eng = engines[(name, "float32")]
        (p,) = prompts_for(_vocab(name), [45], seed=2)
        states = []
        P.forward(raw_config(folders[name]), weights_of(folders[name]), p, layer_states=states)
        cache = eng.model.new_cache(max_tokens=64)
        slot = cache.admit()
        eng.model.trace = {}
        eng.model.step(cache, [slot], [p], None)
        got, eng.model.trace = eng.model.trace, None
        assert len(states) == len(eng.model.schedule)
        for i, want in enumerate(states):
            assert rel_err(got[f"layer.{i}"], want) < 1e-5, f"{name}: layer {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token_across_window_edges(engines, folders, name, dtype):
    """A prompt, then so many single tokens that every window of the model passes over decoded tokens only."""
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=256, block_size=16)
    n_decode = {"P": 150, "Q": 80, "R": 40, "S": 70, "T": 40}[name]
    for head in (1, 30):
        (p,) = prompts_for(_vocab(name), [head + n_decode], seed=3 + head)
        want = oracle_logits(folders[(name, dtype)], p)
        slot = cache.admit()
        got = eng.model.step(cache, [slot], [p[:head]], "last")
        assert rel_err(got[0], want[head - 1]) < TOL[dtype]
        for i in range(head, len(p)):
            got = eng.model.step(cache, [slot], [[p[i]]], "last")
            assert rel_err(got[0], want[i]) < TOL[dtype], f"position {i} of a request decoded from {head}"
        cache.release(slot)
    eng.model.check_status()
    cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_several_sizes(engines, folders, name, dtype):
    """A prompt cut into portions of 2, 3, 1, 7, 33, ... tokens gives the logits of the whole prompt; in float32 to
    the last bits, since no sum's order depends on the cut."""
    eng = engines[(name, dtype)]
    (p,) = prompts_for(_vocab(name), [150], seed=5)
    want = oracle_logits(folders[(name, dtype)], p)
    cache = eng.model.new_cache(max_tokens=256, block_size=8)
    slot = cache.admit()
    whole = eng.model.step(cache, [slot], [p], "all").clone()
    cache.release(slot)
    for sizes in ([2] * 75, [3, 1, 7, 33, 2, 64, 5, 1, 1, 30, 3], [149, 1], [1, 149]):
        slot = cache.admit()
        at, rows = 0, []
        for n in sizes:
            rows.append(eng.model.step(cache, [slot], [p[at:at + n]], "all").clone())
            at += n
        assert at == len(p)
        got = torch.cat(rows)
        cache.release(slot)
        assert rel_err(got, want) < TOL[dtype]
        assert rel_err(got, whole) < (2e-6 if dtype == "float32" else TOL[dtype]), f"portions {sizes[:4]}..."
    eng.model.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batch_equals_each_request_alone_and_slots_are_used_again(engines, folders, name, dtype):
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=64 * 8, block_size=8, max_slots=4)
    for batch_no, lengths in enumerate([[9, 80, 1, 44], [130, 3, 26], [5, 5, 62, 25]]):
        reqs = prompts_for(_vocab(name), lengths, seed=30 + batch_no)
        decode = [min(k, len(p) - 1) for k, p in zip([6, 40, 0, 9], reqs)]
        heads = [len(p) - k for p, k in zip(reqs, decode)]
        slots = [cache.admit() for _ in reqs]                 # the second and third batch get used slots and pages
        got = eng.model.step(cache, slots, [p[:h] for p, h in zip(reqs, heads)], "last")
        for i, (p, h) in enumerate(zip(reqs, heads)):
            assert rel_err(got[i], oracle_logits(folders[(name, dtype)], p)[h - 1]) < TOL[dtype]
        live = [i for i in range(len(reqs)) if heads[i] < len(reqs[i])]
        for i in set(range(len(reqs))) - set(live):
            cache.release(slots[i])
        step = 0
        while live:
            got = eng.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + step]] for i in live], "last")
            for j, i in enumerate(live):
                want = oracle_logits(folders[(name, dtype)], reqs[i])[heads[i] + step]
                assert rel_err(got[j], want) < TOL[dtype], f"batch {batch_no}, request {i}, decoded token {step}"
            step += 1
            for i in [i for i in live if heads[i] + step >= len(reqs[i])]:
                cache.release(slots[i])
                live.remove(i)
        cache.check_invariants()
        assert cache.blocks_in_use() == [0] * len(cache.groups)
    eng.model.check_status()


def test_batch_neighbours_change_no_bit_in_float32(engines):
    for name in NAMES:
        eng = engines[(name, "float32")]
        reqs = prompts_for(_vocab(name), [70, 3, 131], seed=40)
        cache = eng.model.new_cache(max_tokens=512, block_size=8, max_slots=4)
        alone = []
        for p in reqs:
            s = cache.admit()
            a = eng.model.step(cache, [s], [p[:-2]], "last").clone()
            b = eng.model.step(cache, [s], [[p[-2]]], "last").clone()
            alone.append((a, b))
            cache.release(s)
        slots = [cache.admit() for _ in reqs]
        a = eng.model.step(cache, slots, [p[:-2] for p in reqs], "last").clone()
        b = eng.model.step(cache, slots, [[p[-2]] for p in reqs], "last").clone()
        for i in range(len(reqs)):
            assert torch.equal(a[i], alone[i][0][0]) and torch.equal(b[i], alone[i][1][0]), f"{name}: request {i}"


@pytest.mark.parametrize("seed", range(200, 212))
def test_configurations_drawn_at_random_in_float32(tmp_path, seed):
    """Sizes nobody chose: a whole prompt, then a batch of unequal prompts decoded together, against the plain model."""
    cfg = random_config(seed)
    folder = fd.write_random_model(tmp_path / "m", cfg, seed)
    W = weights_of(folder)
    reqs = prompts_for(cfg["vocab"], [1, 37, 131], seed=seed)
    want = [P.forward(cfg, W, r) for r in reqs]
    eng = fd.load(folder, device="cuda", dtype="float32")
    cache = eng.model.new_cache(max_tokens=256, max_slots=4, slack_blocks=4, block_size=16)
    s = cache.admit()
    assert rel_err(eng.model.step(cache, [s], [reqs[2]], "all"), want[2]) < 5e-5, cfg
    cache.release(s)
    slots = [cache.admit() for _ in reqs]
    heads = [1, 30, 120]
    got = eng.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], "last")
    for i in range(3):
        assert rel_err(got[i], want[i][heads[i] - 1]) < 5e-5, cfg
    cache.release(slots[0])
    for step in range(7):
        live = [i for i in (1, 2) if heads[i] + step < len(reqs[i])]
        got = eng.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + step]] for i in live], "last")
        for j, i in enumerate(live):
            assert rel_err(got[j], want[i][heads[i] + step]) < 5e-5, (cfg, i, step)
    eng.model.check_status()
    cache.check_invariants()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(folders, name):
    """``Engine.generate``: the scheduler admits five requests three at a time, decode steps replay captured graphs."""
    eng = fd.load(folders[name], device="cuda", dtype="float32")
    prompts = prompts_for(_vocab(name), [3, 30, 1, 70, 9], seed=50)
    got = eng.generate(prompts, 40, max_batch=3)
    for p, r in zip(prompts, got):
        assert r.tokens == plain_greedy(folders[name], p, 40)
    eng.model.check_status()


@pytest.mark.parametrize("name", ["P", "Q", "S"])
def test_greedy_generation_in_bfloat16_picks_a_best_token(folders, name):
    folder = folders[(name, "bfloat16")]
    eng = fd.load(folder, device="cuda", dtype="bfloat16")
    prompts = prompts_for(_vocab(name), [5, 50, 2], seed=51)
    got = eng.generate(prompts, 30)
    for p, r in zip(prompts, got):
        full = p + r.tokens
        ref = oracle_logits(folder, full[:-1])
        scale = float(ref.abs().max())
        for i, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 2 * TOL["bfloat16"] * scale, f"token {i}"
    eng.model.check_status()


def test_command_line_generates(folders):
    p = prompts_for(_vocab("R"), [12], seed=52)[0]
    cmd = [sys.executable, "-m", "flashdecode_cuda_b200", "generate", "--model", str(folders["R"]), "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, p)), "--max-new-tokens", "8"]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["tokens"] == plain_greedy(folders["R"], p, 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_replays_a_schedule(folders, tmp_path, dtype):
    """Prompts of unequal lengths in one step, then one token each, the shorter request ending earlier; the same
    request again afterwards in the freed slot."""
    name = "P"
    a, b = prompts_for(_vocab(name), [40, 9], seed=53)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 19, 20, 29]},
                                     {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[30]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[31]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]}]
    steps += [{"step": 3 + i, "entries": [{"id": "a", "tokens": [a[32 + i]], "want": [0]}], "end": ["a"] if i == 7 else []}
              for i in range(8)]
    steps.append({"step": 11, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})
    out = tmp_path / "out"
    r = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folders[(name, dtype)]), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", cwd=ROOT,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(12)]
    V = _vocab(name)
    wa, wb = oracle_logits(folders[(name, dtype)], a), oracle_logits(folders[(name, dtype)], b)

    def read(i):
        return torch.frombuffer(bytearray((out / f"{i}.f32").read_bytes()), dtype=torch.float32).view(-1, V)
    assert rel_err(read(0), torch.stack([wa[0], wa[19], wa[20], wa[29], wb[6]])) < TOL[dtype]
    assert rel_err(read(1), wa[30:31]) < TOL[dtype]
    assert rel_err(read(2), torch.stack([wa[31], wb[8]])) < TOL[dtype]
    for i in range(8):
        assert rel_err(read(3 + i), wa[32 + i:33 + i]) < TOL[dtype]
    assert rel_err(read(11), wb[8:9]) < TOL[dtype]
