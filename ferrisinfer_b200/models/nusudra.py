"""The Nusudra decoder as a plan.

A scaled token embedding; pre-norm layers over several residual streams (hyper-connections: every sublayer reads a
learned mix of the streams through its RMS norm and its result is written back into all of them); every mixer reads
its input shifted towards the token before by a learned amount per channel; three kinds of mixer, chosen per layer by
the configuration: attention over a latent that the heads share (with a rotated part and an output gate per head), a
gated delta rule, and two mixers side by side (attention with a logarithmic distance penalty and a sink, beside a
state-space layer) whose normed results are averaged; a plain feed-forward with a squared ReLU; an RMS norm and an
untied head at the end.  Without ``streams`` in the configuration the layers are plain pre-norm residual ones.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.shift``, ``l<i>.hc1.*``, ``l<i>.hc2.*``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.nusudra import NusudraConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerPlan, ModelPlan, PartSpec, RunStep

UNIT_NORM_EPS = 1e-6  # of the delta rule's unit-length queries and keys
MAX_POSITIONS = 1 << 20  # the design sets no limit; the step function wants one


def _mixer(kind: str, m, width: int, eps: float) -> PartSpec:
    if kind == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": m.heads, "head_dim": m.dim, "rotary_head_dim": m.rot_dim,
            "v_head_dim": m.vdim, "latent_rank": m.kv_rank, "scale": m.scale, "rotary_base": m.rot_base,
            "rotary_dims": m.rot_dims, "norm_eps": eps})
    if kind == "delta":
        return PartSpec("gated_delta_rule", {
            "hidden_size": width, "num_heads": m.heads, "num_qk_heads": m.kv_heads, "head_dim": m.dim,
            "v_head_dim": m.vdim, "conv_taps": m.conv, "norm_eps": eps, "unit_norm_eps": UNIT_NORM_EPS})
    if kind == "parallel":
        left, right = m.left, m.right
        attention = PartSpec("gqa_attention", {
            "hidden_size": width, "num_heads": left.heads, "num_kv_heads": left.kv_heads, "head_dim": left.dim,
            "v_head_dim": left.vdim, "scale": left.scale,
            "position": PartSpec("log_distance_penalty", {"num_heads": left.heads}),
            "tensor_names": {"q": "q", "k": "k", "v": "v", "o": "o"},
            "bias_names": {"q": "q.b", "k": "k.b", "v": "v.b"}, "sink_name": "sink"})
        state_space = PartSpec("state_space_duality", {
            "hidden_size": width, "num_heads": right.heads, "v_head_dim": right.vdim, "state_size": right.state,
            "groups": right.groups, "norm_groups": right.norm_groups, "conv_taps": right.conv, "norm_eps": eps})
        return PartSpec("parallel_mixers", {"hidden_size": width, "norm_eps": eps,
                                            "branches": {"left": attention, "right": state_space}})
    raise ValueError(kind)


def plan_nusudra(cfg: NusudraConfig) -> ModelPlan:
    cfg.validate()
    W = cfg.width
    norm = PartSpec("grouped_rmsnorm", {"hidden_size": W, "eps": cfg.norm_eps, "groups": 1, "weight_name": ""})
    layers = []
    for i, layer in enumerate(cfg.layers):
        # the shift's tensor lies beside the mixer's folder, so the wrapping mixer is named by the layer itself
        mixer = PartSpec("token_shift_input", {"hidden_size": W, "inner": _mixer(layer.type, layer.mixer, W, cfg.norm_eps),
                                               "weight_name": "shift", "inner_prefix": "mix"})
        ff = None if layer.ff is None else PartSpec("dense_activation", {
            "hidden_size": W, "intermediate_size": layer.ff, "activation": "relu2"})
        # without streams: one stream with in = mix = out = 1, the plain pre-norm residual layer
        block = PartSpec("residual_streams", {"streams": cfg.streams or 1, "mixer_prefix": "",
                                              "learned": cfg.streams is not None})
        layers.append(LayerPlan(prefix=f"l{i}", mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm,
                                block=block))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale,
                                                "weight_name": ""}),
        embedding_prefix="embed",
        layers=tuple(layers),
        run_order=tuple(RunStep(i) for i in range(len(layers))),
        final_norm=norm,
        final_norm_prefix="final.norm",
        output=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied_to": None, "weight_name": ""}),
        output_prefix="head",
        max_positions=MAX_POSITIONS,
        residual_streams=cfg.streams or 1,
    )


register_architecture("Nusudra", NusudraConfig, plan_nusudra, replace=True)
