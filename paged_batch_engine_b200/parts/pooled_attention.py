"""Softmax attention over a sliding window of tokens and mean-pooled blocks of older tokens."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import ParamSpec
from .base import CacheTensor, CompositeNeed, Mixer, PagedNeed, register_part


class PooledWindowAttention(Mixer):
    """Grouped-query softmax attention in which a row at position p sees the tokens p - window
    + 1 .. p and, for everything older, one key and value per block of ``pool`` tokens (the
    means of the block's cached keys and values), once the whole block lies before the window:
    block b is seen when b*pool + pool - 1 <= p - window.  Tokens and blocks share one softmax.

    Options, all constants of the part: ``qk_norm`` (an RMS norm over the whole query projection
    and over the whole key projection, before the split into heads, with gains ``q.norm`` and
    ``k.norm``), ``rotary`` (dict(base, dims, factor): neighbouring pairs (2i, 2i+1) of the first
    ``dims`` dimensions of every head turn by p * base^(-2i/dims) / factor; None: no rotation),
    ``scale`` of the scores, ``talking_heads`` (the heads' probabilities are mixed by the matrix
    ``talk`` [H, H] after the softmax: w'_h = sum_g talk[h, g] w_g; head h applies w'_h to the
    values of its own key/value head).

    It keeps the tokens' keys and values in pages that are given back once both the window and
    the token's unfinished block have passed them, and the pooled ones in pages of one entry per
    ``pool`` tokens that are kept.  Checkpoint tensors under the prefix: q [H*D, hidden], k [G*D,
    hidden], v [G*E, hidden], o [hidden, H*E], q.norm [H*D], k.norm [G*D], talk [H, H]."""
    TENSOR_NAMES = dict(q="q_proj", k="k_proj", v="v_proj", o="o_proj", q_norm="q_norm", k_norm="k_norm",
                        talk="talk")
    decode_capturable = True      # decoded tokens are stepped from the step's device arrays alone

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, window: int, eps: float, dtype, device, pool: Optional[int] = None,
                 rotary: Optional[dict] = None, qk_norm: bool = True, talking_heads: bool = True,
                 tensor_names: Optional[dict] = None, weight_suffix: str = ".weight"):
        unknown = set(tensor_names or {}) - set(self.TENSOR_NAMES)
        if unknown:
            raise ValueError(f"tensor_names knows {sorted(self.TENSOR_NAMES)}; got {sorted(unknown)}")
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if key_dim % 2:
            raise ValueError("the key width per head must be even")
        if window < 1 or (pool is not None and pool < 1):
            raise ValueError("window and pool are at least 1")
        self.names = dict(self.TENSOR_NAMES, **(tensor_names or {}))
        self.suffix = weight_suffix
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.key_dim, self.value_dim = key_dim, value_dim
        self.scale, self.window, self.pool, self.eps = float(scale), int(window), int(pool or 0), float(eps)
        self.qk_norm, self.talking_heads = bool(qk_norm), bool(talking_heads)
        self.dtype, self.device = dtype, device
        self.rotary_dim, self.inv_freq = 0, None
        if rotary is not None:
            dims, base, factor = int(rotary["dims"]), float(rotary["base"]), float(rotary.get("factor", 1.0))
            if dims % 2 or not 0 < dims <= key_dim:
                raise ValueError(f"rotary dims must be even and in (0, key_dim], got {dims}")
            i = torch.arange(dims // 2, dtype=torch.float64)
            self.inv_freq = (torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims) / factor) \
                .to(torch.float32).to(device)
            self.rotary_dim = dims
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = self.talk = None
        self._tile_rows = None

    # ---- what it keeps
    def cache_need(self):
        G = self.num_kv_heads
        pair = (CacheTensor("k", G, self.key_dim), CacheTensor("v", G, self.value_dim))
        # a token's key is read by rows up to window - 1 later, and by the pooling of its block,
        # which happens when the block's last token arrives, up to pool - 1 later
        tokens = PagedNeed(pair, window=max(self.window, self.pool))
        if not self.pool:
            return CompositeNeed.of(tokens=tokens)
        return CompositeNeed.of(tokens=tokens, pooled=PagedNeed(pair, window=None, stride=self.pool))

    def kernel_libraries(self, dtype):
        return [("pooled_attention", {"PBE_PA_F32": 1 if dtype == torch.float32 else 0})] + ops.gemm_libraries(dtype)

    # ---- tensors
    def param_specs(self, prefix):
        n, s = self.names, self.suffix
        H, G, D, E, w = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim, self.hidden_size
        specs = [ParamSpec(prefix + n["q"] + s, (H * D, w)), ParamSpec(prefix + n["k"] + s, (G * D, w)),
                 ParamSpec(prefix + n["v"] + s, (G * E, w)), ParamSpec(prefix + n["o"] + s, (w, H * E))]
        if self.qk_norm:
            specs += [ParamSpec(prefix + n["q_norm"], (H * D,)), ParamSpec(prefix + n["k_norm"], (G * D,))]
        if self.talking_heads:
            specs.append(ParamSpec(prefix + n["talk"], (H, H)))
        return specs

    def load(self, tensors, prefix):
        n, s = self.names, self.suffix
        ws = [tensors.pop(prefix + n[x] + s) for x in "qkv"]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_o = tensors.pop(prefix + n["o"] + s).contiguous()
        if self.qk_norm:
            self.q_gain = tensors.pop(prefix + n["q_norm"]).to(torch.float32).contiguous()
            self.k_gain = tensors.pop(prefix + n["k_norm"]).to(torch.float32).contiguous()
        if self.talking_heads:
            self.talk = tensors.pop(prefix + n["talk"]).to(torch.float32).contiguous()

    # ---- compute
    def forward(self, x, ctx, cache):
        H, G, D, E = self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        proj = ops.linear(x, self.w_qkv, None, out_dtype=self.dtype, kind=1)
        tok = cache.sub["tokens"]
        gt = ctx.group(tok.group)
        writes = cache.writes
        q = ops.qk_prepare(proj[:, :H * D], proj[:, H * D:(H + G) * D], proj[:, (H + G) * D:], self.q_gain,
                           self.k_gain, self.inv_freq, self.rotary_dim, ctx.positions, gt.slots,
                           tok.k if writes else None, tok.v if writes else None, H, G, self.eps, ctx.page_tokens)
        k_pool = v_pool = bt_pool = None
        if self.pool:
            pl = cache.sub["pooled"]
            gp = ctx.group(pl.group)
            k_pool, v_pool, bt_pool = pl.k, pl.v, gp.block_table
            if writes:
                ops.pool_blocks(tok.k, tok.v, k_pool, v_pool, ctx.positions, ctx.request_of_row, gt.block_table,
                                bt_pool, self.pool, ctx.page_tokens)
        if self._tile_rows is None:
            self._tile_rows = ops.pooled_attention_tile_rows(H, E, 16, self.dtype)
        # decoded tokens only (always so in a captured step): a row a tile
        single = getattr(ctx, "captured", False) or int(ctx.q_len_host.max(initial=1)) == 1
        rows = 1 if single else self._tile_rows
        tiles, n_tiles = ctx.row_tiles(rows)
        # few row tiles (decoded tokens, short portions): the keys are split over more blocks; a
        # captured step is sized for the longest context its block tables can hold
        if getattr(ctx, "captured", False):
            longest = gt.block_table.shape[1] * ctx.page_tokens
        else:
            longest = int(ctx.seq_len_host.max(initial=1))
        most_keys = min(longest, self.window + rows - 1) + (longest // self.pool if self.pool else 0)
        splits, split_tiles = ops.pooled_attention_splits(n_tiles, rows, most_keys, H, G, D, E, self.dtype)
        out = ops.pooled_attention(q, tok.k, tok.v, k_pool, v_pool, self.talk, tiles, n_tiles, rows, ctx.q_start,
                                   ctx.q_len, ctx.seq_len, gt.block_table, bt_pool, H, G, self.scale, self.window,
                                   self.pool, ctx.page_tokens, splits, split_tiles)
        return ops.linear(out, self.w_o, None, out_dtype=self.dtype, kind=2)


register_part("mixer", "pooled_window_attention", PooledWindowAttention, replace=True)
