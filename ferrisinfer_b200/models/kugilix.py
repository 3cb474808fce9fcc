"""The Kugilix decoder as a plan.

A scaled token embedding plus a sinusoidal position vector; layers of the parallel kind (both branches read the
same residual stream through an RMS norm in groups each); in front of every mixer a short causal convolution over
time; two kinds of mixer, a decayed linear attention ("lightning") and a grouped-query attention over a sliding
window whose queries and keys are unit-normed per head, whose queries grow with a temperature of the position and
whose scores lose a slope times the distance; a plain feed-forward with the xIELU activation; a span of layers
that runs several times with the same weights (every run a cache and state of its own), the embedding output
added again before each repeat; the grouped norm and an untied head at the end.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.canon1``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.kugilix import KugilixConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, RunStep

POSITION_BASE = 10000.0  # of the sinusoidal position vector
SLOPE_SPAN = 8.0  # head h of H loses 2^(-SLOPE_SPAN (h + 1) / H) per position of distance
MAX_POSITIONS = 1 << 20  # the design sets no limit; the step function wants one


def plan_kugilix(cfg: KugilixConfig) -> ModelPlan:
    cfg.validate()
    W = cfg.width
    norm = PartSpec("grouped_rmsnorm", {"hidden_size": W, "eps": cfg.norm_eps, "groups": cfg.norm_groups,
                                        "weight_name": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if m.type == "attention":
            mixer = PartSpec("gqa_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "window": m.window, "scale": m.scale,
                "position": PartSpec("distance_slopes", {"span": SLOPE_SPAN}),
                "qk_unit_norm_eps": cfg.norm_eps,
                "query_temperature": (m.temp_coef, m.temp_every) if m.temp_every else None,
                "tensor_names": {"q": "q", "k": "k", "v": "v", "o": "o"},
            })
        else:
            mixer = PartSpec("decayed_linear_attention", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "decay": m.decay,
                "norm_eps": cfg.norm_eps, "activation": "silu",
            })
        block = {"mixer_prefix": "mix"}
        if cfg.canon_taps is not None:
            # the convolution's tensor lies beside the mixer's folder, so the wrapping mixer is named by the layer itself
            mixer = PartSpec("short_conv_input", {"hidden_size": W, "taps": cfg.canon_taps, "inner": mixer,
                                                  "weight_name": "canon1", "inner_prefix": "mix"})
            block = {"mixer_prefix": ""}
        ff = None if layer.ff is None else PartSpec("dense_activation", {
            "hidden_size": W, "intermediate_size": layer.ff, "activation": "xielu"})
        layers.append(LayerPlan(prefix=f"l{i}", mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm,
                                block=PartSpec("parallel_residual", block)))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_sinusoidal_embedding", {"vocab_size": cfg.vocab, "hidden_size": W,
                                                            "scale": cfg.embedding_scale, "base": POSITION_BASE,
                                                            "weight_name": ""}),
        embedding_prefix="embed",
        layers=tuple(layers),
        run_order=tuple(RunStep(i, add_embedding=again) for i, again in cfg.run_order()),
        final_norm=norm,
        final_norm_prefix="final.norm",
        output=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied_to": None, "weight_name": ""}),
        output_prefix="head",
        max_positions=MAX_POSITIONS,
    )


register_architecture("Kugilix", KugilixConfig, plan_kugilix, replace=True)
