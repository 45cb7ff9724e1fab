"""Small Buvuzen configurations and lively random weights for the tests.

The weights are not the package's random-model weights (N(0, 0.02) everywhere would leave every softmax flat,
every gate at one half and every router undecided): matrices are N(0, gain / sqrt(inputs)), sinks spread over
a few units, corrections are of the size of a score, so that a wrong key, a window that is one token off, a
sink that is left out or a wrong expert moves the logits by far more than rounding does.  Everything is rounded
to bfloat16 before it is written, so that the engine in either precision and the plain implementation read
the same numbers.
"""
import json
import os

import numpy as np
import torch

import plain_buvuzen as B


def mixer(heads, kv_heads, dim, vdim, scale, size=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
    return m


def moe(ff, experts, top, identity=None, groups=None, scale=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    return {"kind": "moe", "expert": {"ff": ff}, "router": router, "shared": None if shared is None else {"ff": shared}}


def layer(mix, mlp, weights_of=None):
    out = {"type": "attention", "mixer": mix, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(vocab, width, layers, eps=1e-5, embedding_scale=None, logit_scale=None):
    cfg = {"architecture": "Buvuzen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if embedding_scale is not None:
        cfg["embedding"] = {"scale": embedding_scale}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


# sizes no fast kernel takes (a width that is no multiple of 8, heads of 24, 27 and 16 elements with values of 20, 27 and
# 24); grouped and ungrouped heads, one kv head for all; a window shorter than a page, one longer than any test sequence,
# and none; a layer that runs with another's tensors; a layer without a feed-forward; three groups of which two are kept;
# one identity expert; a router without groups, identity experts, multiplier or shared expert that chooses ALL its
# experts; an expert size that is no multiple of 8; no multiplier of the logits
_ODD0 = layer(mixer(4, 2, 24, 20, 0.3, 9), moe(12, 5, 3, identity=1, groups=(3, 2), scale=1.5, shared=20))
ODD = config(97, 140, [
    _ODD0,
    layer(mixer(3, 3, 27, 27, 0.2, 400), None),
    layer(_ODD0["mixer"], _ODD0["mlp"], weights_of=0),
    layer(mixer(6, 1, 16, 24, 0.25), moe(16, 4, 4)),
], embedding_scale=0.7)

# sizes the tensor-core kernels take (heads of 64 and 128, values of 32 to 128, pages of 16), windows that pass over
# page borders; eight outputs in four groups, two of them identity experts; a layer run three times
_EVEN0 = layer(mixer(4, 2, 64, 64, 0.12, 40), moe(32, 6, 3, identity=2, groups=(4, 2), scale=2.5, shared=32))
_EVEN2 = layer(mixer(8, 2, 64, 128, 0.12, 70), moe(64, 8, 2, groups=(2, 1)))
EVEN = config(160, 128, [
    _EVEN0,
    layer(mixer(2, 1, 128, 32, 0.09, 23), None),
    _EVEN2,
    layer(_EVEN0["mixer"], _EVEN0["mlp"], weights_of=0),
    layer(_EVEN0["mixer"], _EVEN0["mlp"], weights_of=3),
], logit_scale=0.5)

# the same attention with routers that have nothing to decide (every output is chosen, identity experts among them; the
# weights are the scores): rounding cannot flip a choice here, so bfloat16 results of long sequences can be judged row by
# row (a flipped expert at one position reaches every later one through the keys)
_ALL0 = layer(_EVEN0["mixer"], moe(32, 2, 3, identity=1, scale=2.0, shared=32))
ALL = config(160, 128, [
    _ALL0,
    layer(EVEN["layers"][1]["mixer"], None),
    layer(_EVEN2["mixer"], moe(64, 2, 2)),
    layer(_ALL0["mixer"], _ALL0["mlp"], weights_of=0),
    layer(mixer(2, 2, 128, 128, 0.09, 45), None),    # (heads of 128 with values of 128: portions of 32 tokens or more on tcgen05)
], embedding_scale=1.5, logit_scale=0.5)

# heads of 48, 96 and 32 elements (sizes that lie in shared memory padded to a power of two), a width that is a multiple of 8
# and not of 16, routers that choose every output
MID = config(120, 104, [
    layer(mixer(6, 3, 48, 48, 0.15, 50), moe(24, 3, 4, identity=1, scale=1.25, shared=40)),
    layer(mixer(2, 1, 96, 96, 0.1, 17), None),
    layer(mixer(4, 4, 32, 32, 0.18), moe(16, 2, 2)),
    layer(mixer(6, 3, 48, 48, 0.15, 50), moe(24, 3, 4, identity=1, scale=1.25, shared=40), weights_of=0),
], embedding_scale=2.0, logit_scale=0.3)

CONFIGS = {"odd": ODD, "even": EVEN, "all": ALL, "mid": MID}


def tensor_shapes(cfg):
    E, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], E)
    for i, lay in enumerate(cfg["layers"]):
        if lay.get("weights_of") is not None:
            continue
        p = "l%d." % i
        a = lay["mixer"]
        out.update({p + "norm1": (E,), p + "mix.q": (a["heads"] * a["dim"], E), p + "mix.k": (a["kv_heads"] * a["dim"], E),
                    p + "mix.v": (a["kv_heads"] * a["vdim"], E), p + "mix.o": (E, a["heads"] * a["vdim"]),
                    p + "mix.q.norm": (a["dim"],), p + "mix.k.norm": (a["dim"],), p + "mix.sink": (a["heads"],),
                    p + "mix.g": (a["heads"], E)})
        m = lay["mlp"]
        if m is None:
            continue
        outputs = m["router"]["experts"] + int(m["router"].get("identity", 0))
        out.update({p + "norm2": (E,), p + "mlp.router": (outputs, E), p + "mlp.correction": (outputs,)})
        names = ["e%d" % e for e in range(m["router"]["experts"])]
        sizes = [m["expert"]["ff"]] * len(names)
        if m.get("shared"):
            names.append("shared")
            sizes.append(m["shared"]["ff"])
            out[p + "mlp.shared.sg"] = (1, E)
        for n, f in zip(names, sizes):
            out.update({p + "mlp.%s.gate" % n: (f, E), p + "mlp.%s.up" % n: (f, E), p + "mlp.%s.down" % n: (E, f)})
    out["final.norm"] = (E,)
    out["head"] = (cfg["vocab"], E)
    return out


def lively_weights(cfg, seed):
    """{name: float64 array of bfloat16-representable values}."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "sink":
            x = rng.normal(0.0, 1.5, shape)
        elif last == "correction":
            x = rng.normal(0.0, 0.08, shape)
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            x = 1.0 + 0.2 * rng.normal(size=shape)        # plain weights
        elif len(shape) == 1:
            x = 0.1 * rng.normal(size=shape)              # an offset: the multiplier is 1 + x
        elif name == "embed":
            x = rng.normal(0.0, 1.0, shape)
        else:
            gain = 2.0 if last in ("q", "k", "router", "g", "sg") else 1.0
            x = rng.normal(0.0, gain / np.sqrt(shape[1]), shape)
        w[name] = B.store_bfloat16(x)
    return w


def write_model(folder, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: torch.from_numpy(np.ascontiguousarray(v)).to(torch.bfloat16) for k, v in w.items()},
              os.path.join(folder, "model.safetensors"))
    return folder


CLOSE_CALL = 0.004   # choice scores lie between 0 and 1 (plus a correction); rounding the input to bfloat16 moves them by 1e-3 at most


class Oracle:
    """Exact logits [T, V] of one whole sequence and, per row, what rounding every stored activation to
    bfloat16 costs (root-mean-square distance from the exact row).  `decided[t]` is False where some router's
    choice for token t hangs on less than CLOSE_CALL: there rounding may pick another expert, in the engine as
    in the rounded plain run, and the row says nothing about either; bfloat16 comparisons leave such rows out
    (32-bit comparisons keep them)."""

    def __init__(self, cfg, w, tokens):
        margins = []
        self.exact = B.forward(cfg, w, tokens, margins_out=margins)
        self.decided = np.all(np.stack(margins) > CLOSE_CALL, axis=0) if margins else np.ones(len(tokens), bool)
        rounded = B.forward(cfg, w, tokens, store=B.store_bfloat16)
        self.cost = np.sqrt(np.mean(np.square(rounded - self.exact), axis=1))
        self.cost[~self.decided] = 0.0   # (a row whose rounded run chose other experts has no rounding cost to speak of)

    def __getitem__(self, row):
        return self.exact[row]


def compare(got, oracles_rows, dtype, what, judge):
    """`oracles_rows`: [(oracle, first row, one past the last)] in the order of `got`'s rows."""
    from helpers import assert_close
    want = np.concatenate([o.exact[a:b] for o, a, b in oracles_rows])
    cost = np.concatenate([o.cost[a:b] for o, a, b in oracles_rows])
    keep = np.ones(len(want), bool) if dtype == "float32" else np.concatenate([o.decided[a:b] for o, a, b in oracles_rows])
    assert got.shape == want.shape and np.isfinite(got).all(), what
    if keep.any():
        assert_close(got[keep], want[keep], dtype, what, cost=cost[keep], judge=judge)


def decided_tokens(cfg, w, n, seed, tries=300):
    """Random tokens whose routers all decide clearly (see `Oracle.decided`), and their oracle."""
    for k in range(tries):
        toks = [int(t) for t in np.random.default_rng(seed + 1000 * k).integers(0, cfg["vocab"], n)]
        margins = []
        B.forward(cfg, w, toks, margins_out=margins)
        if not margins or np.all(np.stack(margins) > CLOSE_CALL):
            return toks, Oracle(cfg, w, toks)
    raise AssertionError("no sequence of %d tokens without a close call among %d tries" % (n, tries))
