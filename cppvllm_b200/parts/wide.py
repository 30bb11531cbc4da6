"""Parts that work on a residual stream kept in float32 under activations of any element type
(``ModelSpec.residual_dtype = "float32"``): the stream is summed in 32-bit and rounded to the activations' type only
where a norm hands it to a matrix product.

* embedding ``scaled_positions``: h = table[token] * scale + pos_table[position] (a learned vector per position; the
  position table is optional, the scale defaults to 1).
* norm ``rmsnorm_wide``: y = T(x / sqrt(mean(x^2) + eps) * w), one rounding, at the store.  ``add_forward`` takes one
  delta or a tuple of two, adds them to the stream in float (h + (d1 + d2)) and norms the sum, one kernel.
* block ``parallel``: x = norm(h);  h <- h + (mixer(x) + ffn(x)).  One norm; both sublayers read its output; a layer may
  have no feed-forward.  The two outputs leave the block as pending deltas, so that the next block's norm (or the final
  norm) adds them: a layer costs one elementwise kernel.
* input ``pass_input``: in front of pass number t of a repeated run of layers, h <- (h + embedded) + step[t] (the
  embedding output only from the second pass on); pending deltas are folded in by the same kernel.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Block, Norm, Part, StreamInput, WeightSpec, register_part


def _as_tuple(pending):
    if pending is None:
        return ()
    return tuple(pending) if isinstance(pending, (tuple, list)) else (pending,)


@register_part("embedding", "scaled_positions")
class ScaledPositionEmbedding(Part):
    category = "embedding"

    def __init__(self, runtime, prefix="", names=None, *, vocab_size: int, hidden_size: int, scale: float = 1.0,
                 max_positions: int = 0):
        super().__init__(runtime, prefix, names)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale, self.max_positions = float(scale), int(max_positions)
        self.table = self.pos_table = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {self.full_name("embed"): WeightSpec((self.vocab_size, self.hidden_size))}
        if self.max_positions > 0:
            specs[self.full_name("pos")] = WeightSpec((self.max_positions, self.hidden_size))
        return specs

    def bind(self, tensors) -> None:
        self.table = tensors[self.full_name("embed")]
        if self.max_positions > 0:
            self.pos_table = tensors[self.full_name("pos")]
            if self.pos_table.dtype != self.table.dtype:
                self.table, self.pos_table = self.table.float(), self.pos_table.float()

    def forward_step(self, ctx, keep: bool = False):
        """Returns (residual stream, embedding output).  With `keep` the two are different buffers, so that the
        embedding output survives the layers."""
        T = ctx.num_tokens
        ws = self.rt.workspace
        out = ws.rows("residual", T, self.hidden_size, torch.float32)
        kept = ws.rows("embedded", T, self.hidden_size, torch.float32) if keep else None
        ops.embed_positions(out, self.table, ctx.tokens[:T], ctx.positions[:T], self.scale, self.pos_table, kept)
        return out, (kept if keep else out)


@register_part("norm", "rmsnorm_wide")
class WideRMSNorm(Norm):
    def __init__(self, runtime, prefix="", names=None, *, size: int, eps: float, buffer: str = "normed",
                 weight_name: str = "weight"):
        super().__init__(runtime, prefix, names)
        self.size, self.eps, self.buffer, self.weight_name = int(size), float(eps), buffer, weight_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name(self.weight_name): WeightSpec((self.size,), role="vector", init="norm")}

    def bind(self, tensors) -> None:
        self.weight = tensors[self.full_name(self.weight_name)]

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def _out(self, x, out):
        return out if out is not None else self.rt.workspace.rows(self.buffer, x.shape[0], self.size, self.rt.dtype)

    def forward(self, x, out=None):
        return ops.resid_update(x, (), norm_weight=self.weight, eps=self.eps, out=self._out(x, out))

    def add_forward(self, residual, delta, out=None):
        return ops.resid_update(residual, _as_tuple(delta), norm_weight=self.weight, eps=self.eps, out=self._out(residual, out))


@register_part("block", "parallel")
class ParallelBlock(Block):
    def __init__(self, runtime, prefix="", names=None, *, mixer, ffn, mixer_norm, ffn_norm=None):
        super().__init__(runtime, prefix, names)
        if ffn_norm is not None:
            raise ValueError("a parallel block has one norm; its sublayers share it")
        self.mixer, self.ffn, self.norm = mixer, ffn, mixer_norm

    def parts(self):
        return tuple(p for p in (self.norm, self.mixer, self.ffn) if p is not None)

    def forward(self, h, pending, ctx, cache, state):
        x = self.norm.forward(h) if pending is None else self.norm.add_forward(h, pending)
        a = self.mixer.forward(x, ctx, cache, state)
        if self.ffn is None:
            return h, a
        return h, (a, self.ffn.forward(x, ctx))


@register_part("input", "pass_input")
class PassInput(StreamInput):
    def __init__(self, runtime, prefix="", names=None, *, hidden_size: int, times: int, weight_name: str = "step",
                 embedding_from: int = 1):
        super().__init__(runtime, prefix, names)
        self.hidden_size, self.times, self.weight_name = int(hidden_size), int(times), weight_name
        self.embedding_from = int(embedding_from)         # the embedding output is added from this pass on
        self.steps: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.full_name(self.weight_name): WeightSpec((self.times, self.hidden_size), role="vector")}

    def bind(self, tensors) -> None:
        self.steps = tensors[self.full_name(self.weight_name)]

    def weight_bytes(self) -> int:
        return self.hidden_size * self.steps.element_size()

    def forward(self, h, pending, embedded, index: int):
        if not (0 <= index < self.times):
            raise ValueError(f"pass {index} of {self.times}")
        rows = embedded if index >= self.embedding_from else None
        if rows is not None and rows.data_ptr() == h.data_ptr():
            raise ValueError("the embedding output was not kept apart from the residual stream")
        ops.resid_update(h, _as_tuple(pending), rows=rows, vector=self.steps[index])
        return h, None
