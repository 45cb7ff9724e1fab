"""Dobepel as a plan of parts.

Input: token row plus a row picked by the pair (previous token, token).  Every layer is a sandwich-norm
block (a norm before and after each sublayer, both branches times `residual_mult`) around a mixer of two
members side by side, and a feed-forward that is dense (gelu), routed (experts with a router bias and a
shared expert) or absent, layer by layer as config.json lists them.  The left member is softmax attention
over a paged cache without rotation: positions enter as a per-head bias by distance, through a sliding
window that keeps the first tokens; its values have another size than its keys.  The right member is
linear attention with a fixed decay per head and a float32 state per request.  Tensor names: `l<i>.` plus
`norm1 | norm1b | norm2 | norm2b | mix.left.{q,k,v,o,out} | mix.right.{q,k,v,g,o,norm,out} | mlp.*`,
`embed`, `bigram`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import DobepelConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec

# the per-head slopes of the distance bias are 2^(-8 (head + 1) / heads): fixed by the design
DISTANCE_BIAS_EXPONENT = 8.0


def _mixer(cfg: DobepelConfig, layer: dict, p: str) -> PartSpec:
    left, right = layer["mixer"]["left"], layer["mixer"]["right"]
    mask = left.get("mask") or {}
    window = int(mask.get("size", 0))
    members = [
        PartSpec("paged_attention", p + "left.", dict(
            hidden_size=cfg.width, num_heads=left["heads"], num_kv_heads=left["kv_heads"], head_dim=left["dim"],
            v_head_dim=left["vdim"], bias=False, qk_norm=False, eps=cfg.norm_eps, window=window,
            keep_first=int(mask.get("keep_first", 0)) if window else 0, scale=float(left["scale"]),
            distance_bias_exponent=DISTANCE_BIAS_EXPONENT, position=None, names=("q", "k", "v", "o"))),
        PartSpec("decayed_linear_attention", p + "right.", dict(
            hidden_size=cfg.width, num_heads=right["heads"], head_dim=right["dim"], v_head_dim=right["vdim"],
            decay=list(right["decay"]), eps=cfg.norm_eps, activation="silu")),
    ]
    return PartSpec("parallel", p, dict(hidden_size=cfg.width, members=members, out_norm_names=("left.out", "right.out"),
                                        eps=cfg.norm_eps))


def _feed_forward(cfg: DobepelConfig, mlp, p: str):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("dense_mlp", p, dict(hidden_size=cfg.width, intermediate_size=mlp["ff"], activation="gelu",
                                             names=("up", "down")))
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("gated_mlp", p + "shared.", dict(hidden_size=cfg.width, intermediate_size=mlp["shared"]["ff"],
                                                           activation="silu", names=("gate", "up", "down")))
    return PartSpec("routed_experts", p, dict(
        hidden_size=cfg.width, experts=mlp["router"]["experts"], top=mlp["router"]["top"],
        intermediate_size=mlp["expert"]["ff"], activation="silu", router_bias=True, shared=shared))


def dobepel_plan(cfg: DobepelConfig) -> ModelPlan:
    norm = lambda name: PartSpec("rms_norm", name, dict(size=cfg.width, eps=cfg.norm_eps, weight_name=""))
    layers, unused = [], []
    for i, layer in enumerate(cfg.layers):
        p = "l%d." % i
        ff = _feed_forward(cfg, layer.get("mlp"), p + "mlp.")
        norms = {"mixer": norm(p + "norm1"), "mixer_out": norm(p + "norm1b")}
        if ff is not None:
            norms.update({"feed_forward": norm(p + "norm2"), "feed_forward_out": norm(p + "norm2b")})
        else:   # (a layer without a feed-forward has no use for its norms, should a checkpoint carry them)
            unused += [p + "norm2", p + "norm2b"]
        layers.append(LayerSpec(mixer=_mixer(cfg, layer, p + "mix."), feed_forward=ff, norms=norms, block="sandwich_norm",
                                block_params=dict(residual_mult=cfg.residual_mult)))
    return ModelPlan(
        vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("pair_hash_embedding", "", dict(
            vocab_size=cfg.vocab, hidden_size=cfg.width, buckets=cfg.bigram_buckets, mul_prev=cfg.bigram_mul_prev,
            mul_cur=cfg.bigram_mul_cur, table_name="embed", pair_table_name="bigram")),
        layers=layers, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", "head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, weight_name="")),
        order=list(range(len(layers))), ignored_tensors=unused)


register_architecture(DobepelConfig.architecture, DobepelConfig.model_type, DobepelConfig, dobepel_plan)
