"""Givirax as data: the typed configuration becomes a ``ModelSpec``.

A decoder-only model with a residual stream summed in 32-bit: a token embedding scaled by a constant plus a learned
position vector; layers that are *parallel* blocks (one RMSNorm, whose output the mixer and the feed-forward both read;
the stream receives the sum of their outputs); a final RMSNorm and an untied output head.  The mixer is grouped-query
attention without rotation and without a value projection (the keys are the values), with a scale from the
configuration, behind a sliding window that keeps the sequence's first tokens visible.  The feed-forward is dense
(tanh-GELU, no gate), a mixture of gated SiLU experts behind a biased float32 router (top-k, weights renormalised over the k winners),
or absent.  Layers ``loop.start .. loop.stop-1`` run ``loop.times`` times in a row with the same weights and a cache of
their own per pass; each pass begins with a learned vector added to the stream, and every pass after the first also
with the embedding output added again.  Tensor names: ``embed``, ``pos``, ``loop.step``, ``l<i>.norm1``,
``l<i>.mix.{q,k,o}``, ``l<i>.mlp.{up,down}`` or ``l<i>.mlp.{router,router.b,e<j>.{gate,up,down}}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.givirax_config import GiviraxConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def build_givirax_spec(cfg: GiviraxConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = PartSpec("keys_attention", dict(hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                                scale=m.scale, window=m.window, keep_first=m.keep_first), prefix=p + "mix.")
        ffn = None
        if layer.mlp is not None and layer.mlp.kind == "dense":
            ffn = PartSpec("act_mlp", dict(hidden_size=D, intermediate_size=layer.mlp.ff, activation="gelu_tanh"), prefix=p + "mlp.")
        elif layer.mlp is not None:
            ffn = PartSpec("routed_glu", dict(hidden_size=D, intermediate_size=layer.mlp.ff, num_experts=layer.mlp.experts,
                                              top=layer.mlp.top), prefix=p + "mlp.")
        layers.append(LayerSpec(mixer=mixer, ffn=ffn,
                                mixer_norm=PartSpec("rmsnorm_wide", dict(size=D, eps=eps, weight_name="norm1"), prefix=p),
                                ffn_norm=None, block="parallel"))
    order, inputs = None, {}
    if cfg.has_loop:
        inputs["loop"] = PartSpec("pass_input", dict(hidden_size=D, times=cfg.loop_times, weight_name="step"), prefix="loop.")
        order = [RunEntry(i) for i in range(cfg.loop_start)]
        for t in range(cfg.loop_times):
            for i in range(cfg.loop_start, cfg.loop_stop):
                first = i == cfg.loop_start
                order.append(RunEntry(i, input="loop" if first else None, input_index=t if first else 0))
        order += [RunEntry(i) for i in range(cfg.loop_stop, len(cfg.layers))]
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=D,
        vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_positions", dict(vocab_size=cfg.vocab, hidden_size=D, scale=cfg.embedding_scale,
                                                    max_positions=cfg.max_positions)),
        layers=layers,
        final_norm=PartSpec("rmsnorm_wide", dict(size=D, eps=eps, buffer="head_normed", weight_name="norm"), prefix="final."),
        lm_head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=D), names={"weight": "head"}),
        run_order=order,
        max_positions=cfg.max_positions,
        eos_token_ids=tuple(cfg.eos_token_ids),
        inputs=inputs,
        residual_dtype="float32",
    )


register_architecture("Givirax", GiviraxConfig.from_dict, build_givirax_spec, model_types=("givirax",), replace=True,
                      builtin=True)
