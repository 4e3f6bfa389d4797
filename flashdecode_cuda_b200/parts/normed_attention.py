"""Attention mixers without a rotation: grouped-query attention whose q and k are normed over their whole
projection, with a sliding window; and latent attention, which keeps one low-rank vector per position and makes
every head's keys and values from it."""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.spec import TensorSpec
from .attention import FP32_SPLIT_LEN, plan_splits
from .base import KVRequest, LayerCache, Mixer, Runtime
from .linear import matmul


def decode_splits(ctx, n_q: int, n_kv: int, v_dim: int, dtype: torch.dtype, rt: Runtime, head_dim: int = 0):
    """(n_splits, split_len, scratch) of a step's attention: a step of single tokens cuts every sequence's keys into
    splits (float32: of a fixed length, so that where a sequence's partial sums are cut depends on its own length only;
    bfloat16: by the batch's size); any other step does not."""
    if ctx.max_q_len != 1:
        return 1, 0, None
    if dtype == torch.float32:
        split_len = FP32_SPLIT_LEN
        n_splits = max(1, -(-ctx.kv_len_bound // split_len))
    else:
        # (the tensor-core kernel cuts a large group of query heads into several, each with CTAs of its own)
        heads = K.attention_decode_heads(n_q, n_kv, head_dim, v_dim) if head_dim else n_kv
        n_splits, split_len = plan_splits(ctx.n_rows, heads, ctx.kv_len_bound, rt.sm_count)
    scratch = None
    if n_splits > 1:
        scratch = ctx.ws.get("attn_scratch", (K.attention_scratch_floats(ctx.T, n_q, v_dim, n_splits),), torch.float32)
    return n_splits, split_len, scratch


def _up8(n: int) -> int:
    return -(-n // 8) * 8


def _head_sizes_ok(prefix: str, **sizes: int) -> None:
    """The attention kernels take head sizes that are multiples of 8 up to 512; other sizes are padded with zeros to
    the next multiple when the weights are bound (zero rows of the projections, zero norm weights), which changes no
    score and no output."""
    for what, n in sizes.items():
        if n < 1 or _up8(n) > 512:
            raise ValueError(f"{prefix}: {what.replace('_', ' ')} {n} is not taken: the attention kernels take sizes "
                             f"from 1 to 512")


def _pad_heads(w: torch.Tensor, n_heads: int, size: int, padded: int) -> torch.Tensor:
    """w [n_heads * size, ...] -> [n_heads * padded, ...]: zero rows after every head's own."""
    if size == padded:
        return w
    out = w.new_zeros((n_heads, padded) + tuple(w.shape[1:]))
    out[:, :size] = w.view((n_heads, size) + tuple(w.shape[1:]))
    return out.view((n_heads * padded,) + tuple(w.shape[1:]))


@register_part("mixer", "qk_normed_attention")
class QKNormedAttention(Mixer):
    """For the mixer's input h [T, hidden]:

        q, k, v = W_q h, W_k h, W_v h                           (no biases)
        q       = q / sqrt(mean(q^2) + eps) * w_q               over ALL of q's n_heads * head_dim values at once,
        k       = k / sqrt(mean(k^2) + eps) * w_k               likewise; then both are split into heads
        a       = softmax over the visible keys of (q . k) * scale; query head h reads key/value head
                  h // (n_heads / n_kv_heads); value heads have ``v_head_dim`` dimensions
        out     = W_o a

    Nothing is rotated: positions enter through visibility alone.  Visible keys of the query at position i: j <= i,
    and with a ``window`` only i - j < window.  ``qk_norm`` False: q and k are used as projected.  One packed
    product gives q, k and v.  Tensors ``<prefix>.q`` / ``.k`` / ``.v`` / ``.o`` (stored [out, in]), ``.q.norm``,
    ``.k.norm``.  The norms are float32 in both dtypes.
    """

    def __init__(self, prefix: str, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int,
                 scale: float, eps: float, window: Optional[int] = None, qk_norm: bool = True):
        _head_sizes_ok(prefix, head_size=head_dim, value_head_size=v_head_dim)
        if n_kv_heads < 1 or n_heads % n_kv_heads != 0 or n_heads // n_kv_heads > 64:
            raise ValueError(f"{prefix}: {n_heads} query heads for {n_kv_heads} key/value heads: the kernels take whole "
                             f"groups of up to 64 query heads per key/value head")
        if window is not None and window < 1:
            raise ValueError(f"{prefix}: a window of {window} positions")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.n_q, self.n_kv, self.d, self.dv = n_heads, n_kv_heads, head_dim, v_head_dim
        self.dp, self.dvp = _up8(head_dim), _up8(v_head_dim)         # head sizes as the kernels see them
        self.scale, self.eps, self.window, self.qk_norm = float(scale), float(eps), window, qk_norm

    def _sizes(self):
        return (("q", self.n_q * self.d), ("k", self.n_kv * self.d), ("v", self.n_kv * self.dv))

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        specs = [TensorSpec(f"{p}.{n}", (c, H), init="unit") for n, c in self._sizes()]
        if self.qk_norm:
            specs += [TensorSpec(f"{p}.q.norm", (self.n_q * self.d,), "vector", init="norm"),
                      TensorSpec(f"{p}.k.norm", (self.n_kv * self.d,), "vector", init="norm")]
        specs.append(TensorSpec(f"{p}.o", (H, self.n_q * self.dv), init="unit"))
        return specs

    def kv_request(self) -> KVRequest:
        return KVRequest(self.n_kv, self.dp, self.window, None, self.dvp)

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        heads = {"q": (self.n_q, self.d, self.dp), "k": (self.n_kv, self.d, self.dp), "v": (self.n_kv, self.dv, self.dvp)}
        self.w_in = torch.cat([_pad_heads(tensors.pop(f"{p}.{n}"), *heads[n]) for n, _ in self._sizes()], dim=0).contiguous()
        self.q_norm = self.k_norm = None
        if self.qk_norm:
            self.q_norm = _pad_heads(tensors[f"{p}.q.norm"].float(), *heads["q"]).contiguous()
            self.k_norm = _pad_heads(tensors[f"{p}.k.norm"].float(), *heads["k"]).contiguous()
        w_o = tensors[f"{p}.o"]
        if self.dvp != self.dv:             # zero columns where the padded value dimensions arrive
            w_o = _pad_heads(w_o.t().contiguous(), self.n_q, self.dv, self.dvp).t().contiguous()
            tensors[f"{p}.o"] = w_o
        self.w_o = w_o

    def weight_bytes(self) -> int:
        return self.w_in.numel() * self.w_in.element_size() + self.w_o.numel() * self.w_o.element_size()

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_in

    def forward(self, ctx, x: torch.Tensor, lc: LayerCache) -> torch.Tensor:
        T, ws, rt = ctx.T, ctx.ws, self.rt
        proj = ws.get("nat_proj", (T, self.w_in.shape[0]), x.dtype)
        matmul(x, self.w_in, None, proj, status=rt.status)
        q = ws.get("nat_q", (T, self.n_q * self.dp), x.dtype)
        K.norm_append(proj, q, self.q_norm, self.k_norm, self.eps, ctx.tok_row, ctx.tok_pos, ctx.row_slot, lc.k_pool,
                      lc.v_pool, lc.group.table, self.n_kv, lc.writes, rt.status, q_count=self.n_q * self.d,
                      k_count=self.n_kv * self.d)
        attn = ws.get("nat_attn", (T, self.n_q * self.dvp), x.dtype)
        n_splits, split_len, scratch = decode_splits(ctx, self.n_q, self.n_kv, self.dvp, x.dtype, rt, self.dp)
        K.attention(q, lc.k_pool, lc.v_pool, attn, lc.group.table, ctx.tok_row, ctx.row_slot, ctx.row_q_start,
                    ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, ctx.max_q_len, self.n_q, self.n_kv, self.dp, self.scale,
                    self.window or 0, n_splits, split_len, scratch, rt.status)
        out = ws.get("mixer_out", (T, self.hidden_size), x.dtype)
        return matmul(attn, self.w_o, None, out, target_ctas=4 * rt.sm_count, status=rt.status)


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """For the mixer's input h [T, hidden], with ``n_heads`` heads, ``head_dim`` query/key and ``v_head_dim`` value
    dimensions per head and a latent of ``kv_rank`` dimensions:

        q   = W_q h                                        (no rotated part)
        c   = (W_dkv h) / sqrt(mean((W_dkv h)^2) + eps) * w_c           the latent: all that is cached
        k_h = U_h c,  v_h = V_h c                          (U = ``.uk`` [heads * head_dim, kv_rank], V = ``.uv``, head by head)
        a_h = softmax over the visible keys j of (q_h . k_h[j]) * scale
        out = W_o [a_1 V-values ... ]

    computed without ever expanding the cached positions: (q_h . U_h c) = (U_h^T q_h) . c, so the queries are taken
    into the latent's basis (one small product per head), attention runs over the cached latents as ONE key/value head
    of size ``kv_rank`` that all query heads share and that serves as key and as value, and V_h is applied to each
    head's attended latent afterwards.  Visible keys: j <= i, and with a ``window`` only i - j < window.

    Whole prompts in bfloat16 (a step whose sequences all start at their first token) take the other order where that
    reaches a faster attention kernel: k_h and v_h of the step's own tokens are expanded by one product into pages of the
    workspace, and attention runs over them with a key/value head per query head (``expands``); the cache still
    receives the latents only.  Tensors ``<prefix>.q``, ``.dkv``, ``.dkv.norm``, ``.uk``, ``.uv``, ``.o``.
    """

    def __init__(self, prefix: str, hidden_size: int, n_heads: int, head_dim: int, v_head_dim: int, kv_rank: int,
                 scale: float, eps: float, window: Optional[int] = None):
        _head_sizes_ok(prefix, latent_size=kv_rank)
        if n_heads < 1 or n_heads > (64 if _up8(kv_rank) <= 256 else 32) or head_dim < 1 or v_head_dim < 1:
            raise ValueError(f"{prefix}: {n_heads} heads of {head_dim} / {v_head_dim}: the attention kernel takes up to 64 "
                             f"query heads on the one latent (32 on a latent wider than 256)")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.n_q, self.d, self.dv, self.r_true = n_heads, head_dim, v_head_dim, kv_rank
        self.r = _up8(kv_rank)                     # the latent as the kernels see it: zero-padded to a multiple of 8
        self.scale, self.eps, self.window = float(scale), float(eps), window

    def tensor_specs(self) -> List[TensorSpec]:
        p, H = self.prefix, self.hidden_size
        r = self.r_true
        return [TensorSpec(f"{p}.q", (self.n_q * self.d, H), init="unit"),
                TensorSpec(f"{p}.dkv", (r, H), init="unit"),
                TensorSpec(f"{p}.dkv.norm", (r,), "vector", init="norm"),
                TensorSpec(f"{p}.uk", (self.n_q * self.d, r), init="unit"),
                TensorSpec(f"{p}.uv", (self.n_q * self.dv, r), init="unit"),
                TensorSpec(f"{p}.o", (H, self.n_q * self.dv), init="unit")]

    def kv_request(self) -> KVRequest:
        return KVRequest(1, self.r, self.window, None, None, keys_only=True)

    def bind(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        p = self.prefix
        pad = lambda w: _pad_heads(w, 1, self.r_true, self.r)            # zero rows up to the padded latent size
        self.w_in = torch.cat([tensors.pop(f"{p}.q"), pad(tensors.pop(f"{p}.dkv"))], dim=0).contiguous()     # [q | latent]
        self.c_norm = pad(tensors[f"{p}.dkv.norm"].float()).contiguous()
        # per head: U_h^T [kv_rank, head_dim] takes a query into the latent's basis; V_h [v_head_dim, kv_rank]
        uk, uv = tensors.pop(f"{p}.uk"), tensors.pop(f"{p}.uv")
        if self.r != self.r_true:
            uk, uv = pad(uk.t().contiguous()).t().contiguous(), pad(uv.t().contiguous()).t().contiguous()
        self.w_qc = uk.view(self.n_q, self.d, self.r).transpose(1, 2).contiguous()
        self.w_cv = uv.view(self.n_q, self.dv, self.r).contiguous()
        self.w_o = tensors[f"{p}.o"]
        # which attention kernel each order reaches (3 tcgen05, 2 mma.sync, 1 mma.sync at wide heads, 0 CUDA cores)
        rank = lambda size: {128: 3, 64: 2, 192: 1, 256: 1}.get(size, 0)
        latent, expanded = rank(self.r), (rank(self.d) if self.d == self.dv else 0)
        self.expands = rt.dtype == torch.bfloat16 and (expanded > latent or (expanded == latent and expanded > 1
                                                                              and 2 * self.r > self.d + self.dv))
        self.w_kv = torch.cat([uk, uv], dim=0).contiguous() if self.expands else None      # [heads (d + dv), kv_rank]

    def weight_bytes(self) -> int:
        # (the expansion matrix is a second copy of .uk and .uv in another order: a step reads one of the two)
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_qc, self.w_cv, self.w_o))

    def first_weights(self) -> Optional[torch.Tensor]:
        return self.w_in

    def forward(self, ctx, x: torch.Tensor, lc: LayerCache) -> torch.Tensor:
        T, ws, rt = ctx.T, ctx.ws, self.rt
        proj = ws.get("lat_proj", (T, self.w_in.shape[0]), x.dtype)
        matmul(x, self.w_in, None, proj, status=rt.status)
        q = ws.get("lat_q", (T, self.n_q * self.d), x.dtype)
        out = ws.get("mixer_out", (T, self.hidden_size), x.dtype)
        if self.expands and ctx.max_q_len > 1 and not any(ctx.h_ctx_len):
            # whole prompts: expand the step's own keys and values and attend over them
            c = ws.get("lat_c", (T, self.r), x.dtype)
            K.norm_append(proj, q, None, self.c_norm, self.eps, ctx.tok_row, ctx.tok_pos, ctx.row_slot, lc.k_pool, None,
                          lc.group.table, 1, lc.writes, rt.status, k_rows=c, k_count=self.r_true)
            kv = ws.get("lat_kv", (T, self.w_kv.shape[0]), x.dtype)
            matmul(c, self.w_kv, None, kv, status=rt.status)
            bs = lc.group.block_size
            per_row = -(-ctx.max_q_len // bs)
            n_blocks = ctx.n_rows * per_row
            k_tmp = ws.get("lat_k_pages", (n_blocks, self.n_q, bs, self.d), x.dtype)
            v_tmp = ws.get("lat_v_pages", (n_blocks, self.n_q, bs, self.dv), x.dtype)
            table = ws.get("lat_page_table", (ctx.n_rows, per_row), torch.int32)       # row i owns pages i * per_row ...
            torch.arange(n_blocks, out=table.view(-1))
            rows = ws.get("lat_page_rows", (ctx.n_rows,), torch.int32)
            torch.arange(ctx.n_rows, out=rows)
            K.norm_append(kv, None, None, None, self.eps, ctx.tok_row, ctx.tok_pos, rows, k_tmp, v_tmp, table, self.n_q,
                          True, rt.status)
            av = ws.get("lat_v", (T, self.n_q * self.dv), x.dtype)
            K.attention(q, k_tmp, v_tmp, av, table, ctx.tok_row, rows, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx_len,
                        ctx.n_rows, ctx.max_q_len, self.n_q, self.n_q, self.d, self.scale, self.window or 0, 1, 0, None,
                        rt.status)
            return matmul(av, self.w_o, None, out, target_ctas=4 * rt.sm_count, status=rt.status)
        K.norm_append(proj, q, None, self.c_norm, self.eps, ctx.tok_row, ctx.tok_pos, ctx.row_slot, lc.k_pool, None,
                      lc.group.table, 1, lc.writes, rt.status, k_count=self.r_true)
        qc = ws.get("lat_qc", (T, self.n_q * self.r), x.dtype)
        K.head_gemm(q, self.w_qc, qc)
        ac = ws.get("lat_ac", (T, self.n_q * self.r), x.dtype)
        n_splits, split_len, scratch = decode_splits(ctx, self.n_q, 1, self.r, x.dtype, rt, self.r)
        K.attention(qc, lc.k_pool, lc.k_pool, ac, lc.group.table, ctx.tok_row, ctx.row_slot, ctx.row_q_start,
                    ctx.row_q_len, ctx.row_ctx_len, ctx.n_rows, ctx.max_q_len, self.n_q, 1, self.r, self.scale,
                    self.window or 0, n_splits, split_len, scratch, rt.status)
        v = ws.get("lat_v", (T, self.n_q * self.dv), x.dtype)
        K.head_gemm(ac, self.w_cv, v)
        return matmul(v, self.w_o, None, out, target_ctas=4 * rt.sm_count, status=rt.status)
