"""Dugulorn as data: the typed configuration becomes a ``ModelSpec``.

A decoder-only model with a residual stream summed in 32-bit whose norms stand *behind* the sublayers: the embedding row is
normed; a layer adds the normed output of its mixer to the stream and then, if it has one, the normed output of its
feed-forward; the sublayers read the stream itself.  All these norms are RMS norms whose weights are stored around zero
(1 + w is used).  Layers come in any order with one of three mixers: attention over a cached latent (optionally reading
the cache of an earlier layer), a decaying linear-attention matrix per head, or a gated delta rule with short
convolutions.  The feed-forward is dense with biases and a squared-relu activation.  The output head is the embedding
table.  Tensor names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.{up,up.b,down,down.b}``,
``final.norm``.
"""
from __future__ import annotations

from ..config.dugulorn_config import DugulornConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def build_dugulorn_spec(cfg: DugulornConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    layers, positions, order = [], {}, []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        entry = RunEntry(i)
        if layer.type == "latent_attention":
            r = m.rot
            key = f"rot_{r.dims}_{r.base!r}_{r.factor!r}_{r.original!r}_{r.fast!r}_{r.slow!r}"
            positions.setdefault(key, PartSpec("rotary_blended", dict(
                rotary_dim=r.dims, theta=r.base, max_positions=cfg.max_positions, factor=r.factor, original=r.original,
                fast=r.fast, slow=r.slow, pairing="interleaved")))
            mixer = PartSpec("latent_attention", dict(
                hidden_size=D, num_heads=m.heads, nope_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=m.q_rank,
                kv_rank=m.kv_rank, scale=m.scale, eps=eps, position=key, rot=r.dims,
                reads_other_cache=m.kv_from is not None), prefix=p + "mix.")
            # cache units are numbered by the layer that writes them
            entry = RunEntry(i, cache=i if m.kv_from is None else m.kv_from, writes_cache=m.kv_from is None)
        elif layer.type == "lightning":
            mixer = PartSpec("lightning", dict(hidden_size=D, num_heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay), eps=eps),
                             prefix=p + "mix.")
        else:
            mixer = PartSpec("channel_delta", dict(hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                                                   taps=m.conv, eps=eps, decay_rank=m.a_rank, gate_rank=m.g_rank), prefix=p + "mix.")
        ffn = ffn_norm = None
        if layer.ff:
            ffn = PartSpec("act_mlp", dict(hidden_size=D, intermediate_size=layer.ff, activation="relu2", bias=True), prefix=p + "mlp.")
            ffn_norm = PartSpec("rmsnorm_wide", dict(size=D, eps=eps, weight_name="norm2", offset=1.0), prefix=p)
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, mixer_norm=PartSpec("rmsnorm_wide", dict(size=D, eps=eps, weight_name="norm1", offset=1.0), prefix=p),
                                ffn_norm=ffn_norm, block="outnorm"))
        order.append(entry)
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=D,
        vocab_size=cfg.vocab,
        embedding=PartSpec("normed_tokens", dict(vocab_size=cfg.vocab, hidden_size=D, eps=eps, offset=1.0)),
        layers=layers,
        final_norm=PartSpec("rmsnorm_wide", dict(size=D, eps=eps, buffer="head_normed", weight_name="norm", offset=1.0), prefix="final."),
        lm_head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=D), names={"weight": "embed"}),
        positions=positions,
        run_order=order,
        max_positions=cfg.max_positions,
        eos_token_ids=tuple(cfg.eos_token_ids),
        residual_dtype="float32",
    )


register_architecture("Dugulorn", DugulornConfig.from_dict, build_dugulorn_spec, model_types=("dugulorn",), replace=True,
                      builtin=True)
