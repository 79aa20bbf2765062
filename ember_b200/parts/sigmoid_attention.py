"""Grouped-query causal attention without softmax over a paged key/value cache.

A visible key's weight is sigmoid(scale * q . k + pb[head]); weights are not normalised over keys, so the read-out
is a plain sum in ascending key order (fp32) and needs no maxima or denominators.  Keys have ``head_dim`` elements,
values ``value_dim``; the first ``rotary_dim`` elements of query and key heads are rotated (rotate-half pairs).
Tensors under the prefix: q, k, v, o, pb.
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..config.spec import ConfigError
from .base import CacheNeed, Mixer, Runtime, WeightDecl
from .linear import Linear
from .registry import build_part, register_part


class SigmoidAttention(Mixer):
    graph_safe = True
    can_store = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ConfigError(f"{s.num_heads} heads do not divide into {s.num_kv_heads} key/value heads")
        if s.head_dim <= 0 or not 0 < s.value_dim <= 512:
            raise ConfigError(f"sigmoid attention: heads of {s.head_dim} / {s.value_dim} (values up to 512)")
        self.position = build_part("position", s.position)
        self.q_dim, self.k_dim, self.v_dim = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.value_dim

    def weight_decls(self) -> List[WeightDecl]:
        s, p = self.spec, self.prefix
        return [WeightDecl(p + "q", (self.q_dim, s.hidden_size)), WeightDecl(p + "k", (self.k_dim, s.hidden_size)),
                WeightDecl(p + "v", (self.v_dim, s.hidden_size)),
                WeightDecl(p + "pb", (s.num_heads,), init="uniform", lo=-4.0, hi=-2.0),
                WeightDecl(p + "o", (s.hidden_size, s.num_heads * s.value_dim))]

    def load(self, store, rt: Runtime) -> None:
        p = self.prefix
        self.rt = rt
        got = {d.name: store.take(d.name, d.shape) for d in self.weight_decls()}
        if any(v is None for v in got.values()):
            return
        wd = rt.weight_dtype(got[p + "q"].dtype)
        self.qkv = Linear(torch.cat([rt.to_device(got[p + n], wd) for n in "qkv"], dim=0).contiguous())
        self.o = Linear.from_host(got[p + "o"], rt)
        self.head_bias = rt.to_device(got[p + "pb"], torch.float32)
        self.inv_freq, self.rotary = self.position.rotary_table(rt)

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(kind="full", num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, value_dim=s.value_dim)

    def tile_requests(self):
        return [(ops.sigmoid_attention_tile_queries(self.spec.num_heads // self.spec.num_kv_heads), "all")]

    def forward(self, ctx, x, out, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        s, rt, T, mt = self.spec, self.rt, ctx.T, ctx.max_tokens
        H, G, D, V = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        qkv = ctx.buf("sigmoid_attention.qkv", (mt, self.q_dim + self.k_dim + self.v_dim), torch.float32)
        q = ctx.buf("sigmoid_attention.q", (mt, self.q_dim), rt.dtype)
        att = ctx.buf("sigmoid_attention.out", (mt, H * V), rt.dtype)
        table = ctx.block_table(cache.group)
        self.qkv(ctx, x, qkv, T, ops.EPI_STORE_F32)
        ops.rotate_store(qkv, T, H, G, D, V, self.inv_freq, self.rotary, ctx.positions, ctx.seq_of, table, cache.page_tokens,
                         cache.k, cache.v, q, write_kv=owns_cache, err=ctx.err, stream=ctx.stream)
        tiles, n = ctx.attention_tiles(ops.sigmoid_attention_tile_queries(H // G), "all")
        ops.sigmoid_attention(q, cache.k, cache.v, att, H, G, D, V, tiles, n, table, cache.page_tokens, s.scale,
                              self.head_bias, err=ctx.err, stream=ctx.stream)
        self.o(ctx, att, out, T, ops.EPI_ADD_F32 if accumulate else ops.EPI_STORE_F32)


register_part("mixer", "sigmoid_attention", SigmoidAttention)
