"""Lonasun on the GPU against the plain implementation: each mechanism's kernels alone, then whole models in float32
and bfloat16 - whole prompts, token-by-token decoding, portions down to two tokens, unequal batches against each
request alone, slots and pages used again, keys at chunk edges and page borders, long decoding, greedy generation
through the engine's entry point and scheduler, and the trace runner."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import flashdecode_cuda_b200 as fd
from flashdecode_cuda_b200 import kernels as K
from helpers import prompts_for, rel_err
from lonasun_helpers import LONASUN, oracle_logits, plain_greedy, random_config, raw_config, weights_of, write_folder
from plain import lonasun_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda"
NAMES = ["X", "Y", "Z"]
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KTOL = {"float32": 2e-5, "bfloat16": 2e-2}
# Whole models, relative to the largest logit.  float32: only the order of summation differs from the float64 ground
# truth.  bfloat16: the worst measured over these tests is 3.1e-2 (model X: seven layer runs, each with squared
# activations, which double a relative error, and logits whose largest is about 0.4); what a wrong mask, state or page
# does is told apart by the float32 runs and by the kernel tests with keys that stand out, not by this number.
TOL = {"float32": 1e-5, "bfloat16": 5e-2}


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def step_arrays(ctx_lens, q_lens, slots):
    """Index arrays of a step whose rows bring q_lens[i] tokens after ctx_lens[i] cached ones."""
    tok_row, tok_pos, starts = [], [], []
    for r, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        starts.append(len(tok_row))
        tok_row += [r] * n
        tok_pos += list(range(c, c + n))
    return i32(tok_row), i32(tok_pos), i32(slots), i32(starts), i32(q_lens), i32(ctx_lens)


def make_pools(n_blocks, n_kv, bs, d, dv, dtype):
    return (torch.zeros(n_blocks, n_kv, bs, d, dtype=dtype, device=DEV),
            torch.zeros(n_blocks, n_kv, bs, dv, dtype=dtype, device=DEV))


# ---------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,rot,d,dv,cuts", [(3, 8, 16, 32, [5, 1, 1, 6]), (4, 16, 16, 16, [2, 2, 9]),
                                                (1, 0, 32, 16, [7, 1]), (2, 32, 32, 48, [1, 1, 1, 10]),
                                                (9, 4, 8, 8, [3, 1, 1, 10, 1])])     # more taps than the kernel unrolls
def test_convolution_rotation_and_append(dtype, taps, rot, d, dv, cuts):
    """Two sequences fed in portions (some of one token, some shorter than the taps): q, the cached keys and values
    and the carried state equal the plain convolution and rotation of the whole sequences."""
    torch.manual_seed(taps * 100 + rot)
    dt = TD[dtype]
    n_q, n_kv, bs = 3, 1, 4
    C = (n_q + n_kv) * d + n_kv * dv
    S = sum(cuts)
    lens = [S, S - 3]
    u = [torch.randn(n, C + 6).to(dt) for n in lens]                 # six more columns that the kernel must leave alone
    w = torch.randn(C, taps) * 0.5
    base = 100.0
    k_pool, v_pool = make_pools(16, n_kv, bs, d, dv, dt)
    table = torch.full((4, 8), -1, dtype=torch.int32, device=DEV)
    slots = [2, 0]
    table[2, :4] = i32([5, 1, 7, 3])
    table[0, :4] = i32([0, 9, 2, 11])
    state = torch.zeros(4, max(taps - 1, 1), C, device=DEV) if taps > 1 else None
    half = rot // 2
    pos = torch.arange(64).float()
    inv = base ** (-torch.arange(half).float() * 2 / rot) if rot else torch.zeros(0)
    cos, sin = torch.outer(pos, inv).cos().to(DEV), torch.outer(pos, inv).sin().to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q_got = [torch.zeros(n, n_q * d) for n in lens]
    done = [0, 0]
    for cut in cuts:
        rows = [r for r in range(2) if done[r] < lens[r]]
        q_lens = [min(cut, lens[r] - done[r]) for r in rows]
        proj = torch.cat([u[r][done[r]:done[r] + n] for r, n in zip(rows, q_lens)]).to(DEV).contiguous()
        tok_row, tok_pos, row_slot, q_start, q_len, _ = step_arrays([done[r] for r in rows], q_lens, [slots[r] for r in rows])
        q_out = torch.zeros(proj.shape[0], n_q * d, dtype=dt, device=DEV)
        single = max(q_lens) == 1
        K.conv_rope_append(proj, w.to(DEV), state, q_out, cos if rot else None, sin if rot else None, rot, tok_row,
                           tok_pos, row_slot, q_start, q_len, k_pool, v_pool, table, n_q, n_kv, d, dv, True, single, status)
        if state is not None and not single:
            K.conv_state_update(proj, state, row_slot, q_start, q_len, len(rows))
        at = 0
        for r, n in zip(rows, q_lens):
            q_got[r][done[r]:done[r] + n] = q_out[at:at + n].float().cpu()
            at += n
            done[r] += n
    assert int(status.item()) == 0
    for r in range(2):
        x = u[r][:, :C].double()
        y = P.short_conv(x, w.double())
        n = lens[r]
        q_want = P.partial_rotation(y[:, :n_q * d].reshape(n, n_q, d), torch.arange(n), rot, base) if rot else y[:, :n_q * d].reshape(n, n_q, d)
        k_want = y[:, n_q * d:(n_q + n_kv) * d].reshape(n, n_kv, d)
        if rot:
            k_want = P.partial_rotation(k_want, torch.arange(n), rot, base)
        v_want = y[:, (n_q + n_kv) * d:].reshape(n, n_kv, dv)
        assert rel_err(q_got[r], q_want.reshape(n, -1)) < KTOL[dtype]
        blocks = table[slots[r]].tolist()
        k_got = torch.stack([k_pool[blocks[p // bs], :, p % bs] for p in range(n)]).float().cpu()
        v_got = torch.stack([v_pool[blocks[p // bs], :, p % bs] for p in range(n)]).float().cpu()
        assert rel_err(k_got, k_want) < KTOL[dtype] and rel_err(v_got, v_want) < KTOL[dtype]
        if state is not None:
            assert torch.equal(state[slots[r]].cpu(), u[r][n - (taps - 1):, :C].float())      # the last projected values, exactly


def _attention_case(dtype, d, dv, G, n_kv, chunk, bs, S, portions, seed):
    """Keys that stand out sit on the last position of every chunk and on the first of the next: a visibility that is
    one position off changes the result by the size of a value."""
    torch.manual_seed(seed)
    dt = TD[dtype]
    n_q = G * n_kv
    q = torch.randn(S, n_q, d) * 0.3
    k = torch.randn(S, n_kv, d) * 0.3
    v = torch.randn(S, n_kv, dv)
    e = torch.zeros(d)
    e[3] = 1.0
    for p in range(S):
        if p % chunk in (0, chunk - 1):
            k[p] += 6.0 * e
    q += 2.0 * e
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    scale = 0.7
    want = P.chunked_attention_fast(q.double(), k.double(), v.double(), scale, chunk).reshape(S, n_q * dv)
    n_cols = -(-S // bs)
    k_pool, v_pool = make_pools(n_cols + 3, n_kv, bs, d, dv, dt)
    perm = torch.randperm(n_cols + 3)[:n_cols]
    table = torch.full((2, n_cols), -1, dtype=torch.int32, device=DEV)
    table[1] = perm.to(torch.int32).to(DEV)
    for p in range(S):
        k_pool[perm[p // bs], :, p % bs] = k[p].to(DEV)
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
                    q_start, q_len, ctx_len, 1, n, n_q, n_kv, d, scale, 0, n_splits, split_len, scratch, status, chunk=chunk)
        got[at:at + n] = out.float().cpu()
        at += n
    assert at == S and int(status.item()) == 0
    err = (got.double() - want).abs().max(dim=1).values / want.abs().max()
    assert float(err.max()) < KTOL[dtype], f"first wrong position {int((err >= KTOL[dtype]).nonzero()[0])} (chunk {chunk})"


ATTN_CASES = [  # d, dv, G, n_kv, chunk, block size, length
    (64, 64, 2, 2, 24, 16, 150),       # tensor-core kernels of head size 64; chunk edges inside pages
    (64, 64, 4, 1, 64, 64, 200),       # a chunk is exactly a page
    (128, 128, 1, 2, 100, 64, 330),    # head size 128: the widest prompt kernel; a chunk that is no multiple of anything
    (32, 48, 2, 2, 24, 8, 100),        # values wider than keys: the CUDA-core kernel
    (48, 16, 3, 1, 37, 4, 120),
    (24, 40, 2, 2, 30, 16, 100),       # head sizes that are multiples of 8 only
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTN_CASES)
def test_chunked_attention_whole_prompt(dtype, case):
    d, dv, G, n_kv, chunk, bs, S = case
    _attention_case(dtype, d, dv, G, n_kv, chunk, bs, S, [S], seed=1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTN_CASES)
def test_chunked_attention_in_portions_and_token_by_token(dtype, case):
    d, dv, G, n_kv, chunk, bs, S = case
    # a long first portion, then portions that start and end on, before and after chunk edges, then single tokens
    first = chunk * 2 - 1
    _attention_case(dtype, d, dv, G, n_kv, chunk, bs, S, [first, 2, chunk, 3, 129, 2] + [1] * S, seed=2)
    _attention_case(dtype, d, dv, G, n_kv, chunk, bs, min(S, 3 * chunk + 2), [1] * S, seed=3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,n_id,top,H,ff,T", [(5, 2, 3, 96, 40, 37), (4, 0, 1, 64, 24, 9), (2, 5, 4, 32, 16, 70),
                                               (0, 3, 2, 32, 8, 5), (9, 0, 9, 40, 8, 33),
                                               (3, 1, 2, 64, 48, 300),      # many rows per expert: tiles of 128 rows in bfloat16
                                               (4, 0, 2, 72, 20, 19)])      # an inner size that is no multiple of 8
def test_routed_experts(dtype, E, n_id, top, H, ff, T):
    """Router, grouping, both grouped products and the combine against the plain feed-forward."""
    torch.manual_seed(E * 10 + top)
    dt = TD[dtype]
    h = torch.randn(T, H).to(dt)
    W = {"m.mlp.router": (torch.randn(E + n_id, H) * 0.3).to(dt), "m.mlp.correction": torch.randn(E + n_id) * 0.05}
    for e in range(E):
        W[f"m.mlp.e{e}.up"] = (torch.randn(ff, H) / H ** 0.5).to(dt)
        W[f"m.mlp.e{e}.down"] = (torch.randn(H, ff) / ff ** 0.5).to(dt)
    cfg = {"kind": "moe", "router": {"experts": E, "identity": n_id, "top": top}, "expert": {"ff": ff}}
    want = P.moe_feed_forward(h.double(), {k: v.double() for k, v in W.items()}, "m", cfg)
    chosen_want, w_want = P.route(h.double(), W["m.mlp.router"].double(), W["m.mlp.correction"].double(), top)
    x = h.to(DEV)
    ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    wts = torch.zeros(T, top, device=DEV)
    K.moe_route(x, W["m.mlp.router"].to(DEV), W["m.mlp.correction"].to(DEV), ids, wts)
    assert torch.equal(ids.cpu().long(), chosen_want)                 # margins of random scores are far above rounding
    assert rel_err(wts, w_want) < 1e-5
    pair_pos = torch.zeros(T * top, dtype=torch.int32, device=DEV)
    y = None
    if E:
        mt = K.moe_tile_rows(dt, T * top, E, (H, ff))
        assert mt == (128 if dtype == "bfloat16" and ff % 8 == 0 and T * top // E >= 96 else 32)
        cap = K.moe_grouped_rows(T * top, E, mt)
        sorted_pair = torch.full((cap,), -7, dtype=torch.int32, device=DEV)
        tile_expert = torch.zeros(cap // mt, dtype=torch.int32, device=DEV)
        n_tiles = torch.zeros(1, dtype=torch.int32, device=DEV)
        K.moe_align(ids, E, pair_pos, sorted_pair, tile_expert, n_tiles, mt)
        sp, pp = sorted_pair.cpu(), pair_pos.cpu()
        used = int(n_tiles.item()) * mt
        real = sp[:used][sp[:used] >= 0]
        assert sorted(real.tolist()) == [p for p in range(T * top) if int(ids.view(-1)[p]) < E]     # every pair once
        assert all(int(sp[pp[p]]) == p for p in real.tolist())
        w_up = torch.stack([W[f"m.mlp.e{e}.up"] for e in range(E)]).to(DEV)
        w_down = torch.stack([W[f"m.mlp.e{e}.down"] for e in range(E)]).to(DEV)
        act = torch.zeros(cap, ff, dtype=dt, device=DEV)
        K.moe_gemm(x, w_up, act, False, sorted_pair, tile_expert, n_tiles, top, mt)
        y = torch.zeros(cap, H, dtype=dt, device=DEV)
        K.moe_gemm(act, w_down, y, True, sorted_pair, tile_expert, n_tiles, top, mt)
    out = torch.zeros(T, H, dtype=dt, device=DEV)
    K.moe_combine(y, x, None, ids, wts, pair_pos, out, E)
    assert rel_err(out, want) < KTOL[dtype]


@pytest.mark.parametrize("E,H,ff,T,top", [(3, 256, 384, 300, 2), (5, 320, 256, 700, 3), (2, 512, 768, 150, 2)])
def test_grouped_products_on_tcgen05_equal_the_plain_experts(E, H, ff, T, top):
    """Prompts in bfloat16: the grouped rows gathered into one matrix, then both products by the TMA + tcgen05 kernel
    with the tile's expert looked up on the device; against the plain experts row by row, and with row tiles that do
    not exist left alone."""
    torch.manual_seed(E + T)
    dt = torch.bfloat16
    x = torch.randn(T, H).to(dt)
    w_up = (torch.randn(E, ff, H) / H ** 0.5).to(dt)
    w_down = (torch.randn(E, H, ff) / ff ** 0.5).to(dt)
    ids = torch.stack([torch.randperm(E + 1)[:top] for _ in range(T)]).to(torch.int32)      # output E: an identity expert
    mt = K.moe_tile_rows(dt, T * top, E, (H, ff))
    assert mt == 128
    cap = K.moe_grouped_rows(T * top, E, mt)
    pair_pos = torch.zeros(T * top, dtype=torch.int32, device=DEV)
    sorted_pair = torch.zeros(cap, dtype=torch.int32, device=DEV)
    tile_expert = torch.zeros(cap // mt, dtype=torch.int32, device=DEV)
    n_tiles = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.moe_align(ids.to(DEV), E, pair_pos, sorted_pair, tile_expert, n_tiles, mt)
    xs = torch.full((cap, H), 7.0, dtype=dt, device=DEV)
    act = torch.full((cap, ff), 7.0, dtype=dt, device=DEV)
    y = torch.full((cap, H), 7.0, dtype=dt, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    K.moe_gather(x.to(DEV), xs, sorted_pair, n_tiles, top, mt)
    K.gemm_tc_grouped(xs, w_up.to(DEV), act, True, tile_expert, n_tiles, status)
    K.gemm_tc_grouped(act, w_down.to(DEV), y, False, tile_expert, n_tiles, status)
    assert int(status.item()) == 0
    used = int(n_tiles.item()) * mt
    assert used < cap and bool((y[used:] == 7.0).all()) and bool((xs[used:] == 7.0).all())
    pp, yc = pair_pos.cpu(), y.cpu().double()
    worst = 0.0
    scale = 0.0
    for p in range(0, T * top, 7):
        e = int(ids.view(-1)[p])
        if e >= E:
            assert int(pp[p]) == -1
            continue
        want = P.relu2_expert(x[p // top].double(), w_up[e].double(), w_down[e].double())
        worst = max(worst, float((yc[int(pp[p])] - want).abs().max()))
        scale = max(scale, float(want.abs().max()))
    assert worst / scale < KTOL["bfloat16"]


# ---------------------------------------------------------------- whole models
class Folders(dict):
    """Model folders by (name, dtype): in bfloat16 the routers' choice is fixed by their corrections (see
    ``write_folder``); ``folders[name]`` is the float32 one."""

    def __missing__(self, name):
        return self[(name, "float32")]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("lonasun")
    return Folders({(n, d): write_folder(tmp, n, seed=21, fixed_choice=d == "bfloat16") for n in NAMES for d in DTYPES})


@pytest.fixture(scope="module")
def engines(folders):
    return {(n, d): fd.load(folders[(n, d)], device="cuda", dtype=d) for n in NAMES for d in DTYPES}


def _vocab(name):
    return LONASUN[name]["vocab"]


def _lengths(name):
    return {"X": [1, 2, 23, 24, 25, 75, 140], "Y": [3, 100, 101, 260], "Z": [1, 16, 64, 65, 129, 200]}[name]


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


def test_every_layer_run_in_float32(engines, folders):
    """The residual stream after every layer run (a looped layer counts each time) against the plain one."""
    for name in NAMES:
        eng = engines[(name, "float32")]
        (p,) = prompts_for(_vocab(name), [45], seed=2)
        trace = []
        P.forward(raw_config(folders[name]), weights_of(folders[name]), p, trace=trace)
        cache = eng.model.new_cache(max_tokens=64)
        slot = cache.admit()
        eng.model.trace = {}
        eng.model.step(cache, [slot], [p], None)
        got, eng.model.trace = eng.model.trace, None
        assert len(trace) == len(eng.model.schedule)
        for i, want in enumerate(trace):
            assert rel_err(got[f"layer.{i}"], want) < 1e-5, f"{name}: layer run {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token_across_chunk_edges(engines, folders, name, dtype):
    """A prompt, then so many single tokens that every chunk size of the model passes an edge while decoding."""
    eng = engines[(name, dtype)]
    cache = eng.model.new_cache(max_tokens=256, block_size=16)
    n_decode = {"X": 60, "Y": 110, "Z": 70}[name]
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


@pytest.mark.parametrize("seed", range(100, 110))
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


@pytest.mark.parametrize("name", ["X", "Z"])
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
    p = prompts_for(_vocab("Z"), [12], seed=52)[0]
    cmd = [sys.executable, "-m", "flashdecode_cuda_b200", "generate", "--model", str(folders["Z"]), "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, p)), "--max-new-tokens", "8"]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert json.loads(r.stdout.strip().splitlines()[-1])["tokens"] == plain_greedy(folders["Z"], p, 8)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_replays_a_schedule(folders, tmp_path, dtype):
    """Prompts of unequal lengths in one step, then one token each, the shorter request ending earlier; the same
    request again afterwards in the freed slot."""
    name = "X"
    a, b = prompts_for(_vocab(name), [40, 9], seed=53)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 23, 24, 29]},
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
    assert rel_err(read(0), torch.stack([wa[0], wa[23], wa[24], wa[29], wb[6]])) < TOL[dtype]
    assert rel_err(read(1), wa[30:31]) < TOL[dtype]
    assert rel_err(read(2), torch.stack([wa[31], wb[8]])) < TOL[dtype]
    for i in range(8):
        assert rel_err(read(3 + i), wa[32 + i:33 + i]) < TOL[dtype]
    assert rel_err(read(11), wb[8:9]) < TOL[dtype]
