"""Buvuzen as a plan of parts.

Input: the token's row times a multiplier.  Every layer is a post-norm block (the sublayers read the stream itself;
each sublayer's OUTPUT is normed, its multiplier one plus the stored tensor, and added) around softmax attention and a routed
feed-forward, or no feed-forward, layer by layer as config.json lists them.  The attention runs over a paged cache
without rotation (positions do not enter the scores): grouped key/value heads, q and k normed per head with plain
weights shared by the heads, values of a size of their own, a sliding window, a learned sink per head in the
softmax's denominator and a sigmoid gate per head on the output.  The feed-forward scores all the router's outputs
with one softmax, chooses by score + correction inside the best groups of neighbouring outputs, weights by the
scores times a multiplier; the router's last outputs are identity experts, and a shared expert with a sigmoid gate
per token runs for every token.  A layer with `weights_of` runs with another layer's tensors and a cache of its
own: the plan's running order names that layer again.  Output: norm, head, logits times a multiplier.
Tensor names: `l<i>.` plus `norm1 | norm2 | mix.{q,k,v,o,g,sink,q.norm,k.norm} | mlp.{router,correction,e<j>.{gate,up,down},
shared.{gate,up,down,sg}}`, `embed`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import BuvuzenConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec


def _mixer(cfg: BuvuzenConfig, m: dict, p: str) -> PartSpec:
    return PartSpec("paged_attention", p, dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
        bias=False, qk_norm=True, eps=cfg.norm_eps, window=int((m.get("mask") or {}).get("size", 0)), scale=float(m["scale"]),
        position=None, names=("q", "k", "v", "o"), norm_names=("q.norm", "k.norm"), sink=True, output_gate=True,
        sink_name="sink", gate_name="g"))


def _feed_forward(cfg: BuvuzenConfig, mlp, p: str):
    if mlp is None:
        return None
    router, groups = mlp["router"], mlp["router"].get("groups") or {}
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("gated_mlp", p + "shared.", dict(hidden_size=cfg.width, intermediate_size=mlp["shared"]["ff"],
                                                           activation="silu", names=("gate", "up", "down")))
    return PartSpec("routed_experts", p, dict(
        hidden_size=cfg.width, experts=router["experts"], top=router["top"], intermediate_size=mlp["expert"]["ff"],
        activation="silu", router_bias=False, shared=shared, scores="softmax_all", correction_name="correction",
        groups=int(groups.get("count", 1)), keep_groups=int(groups.get("keep", 1)), route_scale=float(router.get("scale", 1.0)),
        identity=int(router.get("identity") or 0), shared_gate_name="shared.sg" if shared is not None else None))


def buvuzen_plan(cfg: BuvuzenConfig) -> ModelPlan:
    norm = lambda name: PartSpec("rms_norm", name, dict(size=cfg.width, eps=cfg.norm_eps, weight_name="", one_plus=True))
    layers, place_of, unused = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.get("weights_of") is not None:
            continue
        p = "l%d." % i
        ff = _feed_forward(cfg, layer.get("mlp"), p + "mlp.")
        norms = {"mixer_out": norm(p + "norm1")}
        if ff is not None:
            norms["feed_forward_out"] = norm(p + "norm2")
        else:   # (a layer without a feed-forward has no use for its norm, should a checkpoint carry it)
            unused.append(p + "norm2")
        place_of[i] = len(layers)
        layers.append(LayerSpec(mixer=_mixer(cfg, layer["mixer"], p + "mix."), feed_forward=ff, norms=norms, block="post_norm"))
    return ModelPlan(
        vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", "", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, scale=cfg.embedding_scale,
                                                       weight_name="embed", leaves_rounded=True)),
        layers=layers, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", "head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, weight_name="",
                                                  logit_scale=cfg.logit_scale)),
        # a layer that runs with another's tensors is that layer run again, at a place (and with a cache) of its own
        order=[place_of[cfg.weights_layer(i)] for i in range(len(cfg.layers))], ignored_tensors=unused)


register_architecture(BuvuzenConfig.architecture, BuvuzenConfig.model_type, BuvuzenConfig, buvuzen_plan)
