"""Grouped-query attention whose keys are also its values, over a cache that holds one vector per token and kv head:

    qk = x Wqk^T                     Wqk = rows(q) over rows(k), no bias; there is no value projection: v_j = k_j
    k written to this step's slots of the cache pages [kv_head, slot, head_dim]
    s_ij = scale * q_i . k_j         over the visible j: j <= i and (i - j < window or j < keep_first); window 0: all j <= i
    att_i = softmax_j(s_ij) k_j      scores, softmax and the weighted sum in float
    y = att Wo^T

No rotation: positions enter only through the mask.  The first ``keep_first`` positions stay visible after the window has
passed them; the cache manager keeps their pages and gives the others back as the window passes.  All sizes and the
scale are parameters.  Prompt portions and decoded tokens run through the same kernels: every token attends to its
request's pages, which already hold the step's own keys.  bf16 with head sizes that are multiples of 16 (up to 128) runs
on the tensor cores (csrc/attention_keys.cu: one tile of keys in shared memory feeds both products); float32 and other
shapes take the general kernel (csrc/attention_general.cu).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import CacheSpec, Mixer, WeightSpec, register_part


@register_part("mixer", "keys_attention")
class KeysAttention(Mixer):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: Optional[float] = None, window: int = 0, keep_first: int = 0, q_name: str = "q", k_name: str = "k",
                 o_name: str = "o", force_general: bool = False):
        super().__init__(runtime, prefix, names)
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} key/value heads")
        if window < 0 or keep_first < 0:
            raise ValueError("window and keep_first cannot be negative")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = map(int, (hidden_size, num_heads, num_kv_heads, head_dim))
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(window)
        self.keep_first = int(keep_first) if self.window > 0 else 0       # without a window every position is visible anyway
        self.q_name, self.k_name, self.o_name = q_name, k_name, o_name
        self.force_general = bool(force_general) or runtime.plain_kernels
        self.w_qk = self.w_o = None

    def cache_spec(self) -> CacheSpec:
        return CacheSpec.keys_only(self.num_kv_heads, self.head_dim, self.window, self.keep_first)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, KV, hd = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        return {
            self.full_name(self.q_name): WeightSpec((H * hd, D)),
            self.full_name(self.k_name): WeightSpec((KV * hd, D)),
            self.full_name(self.o_name): WeightSpec((D, H * hd)),
        }

    def bind(self, tensors) -> None:
        q, k = tensors[self.full_name(self.q_name)], tensors[self.full_name(self.k_name)]
        if q.dtype != k.dtype:
            q, k = q.float(), k.float()
        self.w_qk = torch.cat([q, k], dim=0).contiguous()
        self.w_o = tensors[self.full_name(self.o_name)]

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_qk, self.w_o))

    def _project(self, x, w, out, rows):
        return ops.linear(x, w, out=out) if self.rt.plain_kernels else ops.project_rows(x, w, out, rows)

    def forward(self, x, ctx, cache, state):
        T = x.shape[0]
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        ws = self.rt.workspace
        g = ctx.groups[cache.group]
        qk = self._project(x, self.w_qk, ws.rows("attn_qk", T, (H + KV) * hd, x.dtype), T)
        if cache.writes:
            ops.write_rows(cache.pages, qk, g.slot_mapping, H * hd, KV, hd, g.page_size)
        att = ws.rows("attn_out", T, H * hd, x.dtype)
        self.attend(att, qk, ctx, cache, g)
        return self._project(att, self.w_o, ws.rows("attn_proj", T, self.hidden_size, x.dtype), T)

    def attend(self, att, qk, ctx, cache, g):
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        if not self.force_general and ops.attn_keys_supported(qk.dtype, H, KV, hd, qk.shape[1]):
            q_lens = ctx.q_lens if ctx.q_lens is not None else [1] * ctx.num_seqs
            single = ctx.all_decode and ctx.num_tokens == ctx.num_seqs
            splits, scratch = 1, None
            if single:
                visible = min(ctx.max_kv_len, self.window + self.keep_first) if self.window > 0 else ctx.max_kv_len
                splits = ops.attn_keys_decode_splits(ctx.num_seqs, KV, visible)
                if splits > 1:
                    most = ops.attn_keys_scratch_floats(self.rt.workspace.max_seqs, KV, hd, 8)
                    scratch = self.rt.workspace.flat(f"attn_keys_parts_{KV}_{hd}", most, torch.float32)
            ops.attn_keys_bf16(att, qk, cache.pages, g.block_tables, ctx.cu_seqlens, ctx.positions, ctx.num_seqs,
                               ops.attn_keys_tiles(q_lens, H, KV), H, KV, hd, g.page_size, self.scale, window=self.window,
                               keep_first=self.keep_first, all_single=single, splits=splits, scratch=scratch)
            return
        ops.paged_attention_general(att, qk, cache.pages, g.block_tables, ctx.seq_of_token, ctx.positions, self.num_heads,
                                    self.num_kv_heads, self.head_dim, g.page_size, self.scale, window=self.window,
                                    num_tokens=ctx.num_tokens, keep_first=self.keep_first, keys_are_values=True)
