"""Small Dobepel configurations and lively random weights for the tests.

The weights are not the package's random-model weights (N(0, 0.02) everywhere would leave every softmax
flat and every router undecided): matrices are N(0, gain / sqrt(inputs)), so that scores, gates and router
logits spread over several units and a wrong key, a window that is one token off or a lost state moves the
logits by far more than rounding does.  Everything is rounded to bfloat16 before it is written, so that the
engine in either precision and the plain implementation read the same numbers.
"""
import json
import os

import numpy as np
import torch

import plain_dobepel as D


def layer(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def left(heads, kv_heads, dim, vdim, scale, size, keep_first):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": size, "keep_first": keep_first}}


def right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def moe(ff, experts, top, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": None if shared is None else {"ff": shared}}


def config(vocab, width, layers, residual_mult=0.5, eps=1e-5, buckets=53, mul_prev=31, mul_cur=7):
    return {"architecture": "Dobepel", "vocab": vocab, "width": width, "residual_mult": residual_mult,
            "norm": {"eps": eps}, "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
            "layers": layers}


# odd sizes everywhere (one layer's heads of 27, 11 and 7 elements): nothing a fast kernel takes; every kind of feed-forward; values of the size of keys in
# one layer; one key/value head per query head in one layer; a window longer than any test sequence; an expert
# size that is no multiple of 8; as many chosen experts as there are; no shared expert; a decay of exactly 1
ODD = config(97, 140, [
    layer(left(4, 2, 16, 8, 0.3, 9, 2), right(2, 8, 16, [0.9, 0.5]), moe(12, 3, 1)),
    layer(left(2, 2, 27, 27, 0.2, 5, 0), right(3, 11, 7, [1.0, 0.8, 0.25]), None),
    layer(left(6, 1, 16, 24, 0.25, 17, 3), right(1, 20, 40, [0.97]), {"kind": "dense", "ff": 40}),
    layer(left(4, 4, 8, 12, 0.5, 400, 1), right(2, 16, 16, [0.6, 0.99]), moe(16, 4, 4, shared=24)),
])

# sizes the tensor-core kernels take (heads of 64 and 128, pages of 16), windows that pass over page borders
EVEN = config(160, 128, [
    layer(left(4, 2, 64, 64, 0.12, 40, 4), right(2, 64, 32, [0.95, 0.7]), moe(32, 4, 2, shared=32)),
    layer(left(2, 1, 128, 64, 0.09, 23, 1), right(4, 32, 32, [0.99, 0.9, 0.8, 0.5]), {"kind": "dense", "ff": 96}),
    layer(left(8, 2, 64, 128, 0.12, 70, 17), right(1, 128, 128, [0.98]), moe(64, 8, 3)),
], residual_mult=0.4, buckets=211, mul_prev=1009, mul_cur=13)

# the same without routers: rounding cannot flip a choice here, so bfloat16 results of long sequences can be
# judged row by row (a flipped expert at one position reaches every later one through the keys and the state)
DENSE = config(160, 128, [
    layer(EVEN["layers"][0]["mixer"]["left"], EVEN["layers"][0]["mixer"]["right"], {"kind": "dense", "ff": 64}),
    layer(EVEN["layers"][1]["mixer"]["left"], EVEN["layers"][1]["mixer"]["right"], None),
    layer(EVEN["layers"][2]["mixer"]["left"], EVEN["layers"][2]["mixer"]["right"], {"kind": "dense", "ff": 160}),
], residual_mult=0.4, buckets=211, mul_prev=1009, mul_cur=13)

CONFIGS = {"odd": ODD, "even": EVEN, "dense": DENSE}


def tensor_shapes(cfg):
    E, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], E)
    out["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, E)
    for i, lay in enumerate(cfg["layers"]):
        p = "l%d." % i
        a, b = lay["mixer"]["left"], lay["mixer"]["right"]
        out.update({p + "norm1": (E,), p + "norm1b": (E,),
                    p + "mix.left.q": (a["heads"] * a["dim"], E), p + "mix.left.k": (a["kv_heads"] * a["dim"], E),
                    p + "mix.left.v": (a["kv_heads"] * a["vdim"], E), p + "mix.left.o": (E, a["heads"] * a["vdim"]),
                    p + "mix.left.out": (E,), p + "mix.right.out": (E,),
                    p + "mix.right.q": (b["heads"] * b["dim"], E), p + "mix.right.k": (b["heads"] * b["dim"], E),
                    p + "mix.right.v": (b["heads"] * b["vdim"], E), p + "mix.right.g": (b["heads"] * b["vdim"], E),
                    p + "mix.right.o": (E, b["heads"] * b["vdim"]), p + "mix.right.norm": (b["heads"] * b["vdim"],)})
        m = lay["mlp"]
        if m is None:
            continue
        out.update({p + "norm2": (E,), p + "norm2b": (E,)})
        if m["kind"] == "dense":
            out.update({p + "mlp.up": (m["ff"], E), p + "mlp.down": (E, m["ff"])})
            continue
        out.update({p + "mlp.router": (m["router"]["experts"], E), p + "mlp.router.b": (m["router"]["experts"],)})
        names = ["e%d" % e for e in range(m["router"]["experts"])]
        sizes = [m["expert"]["ff"]] * len(names)
        if m.get("shared"):
            names.append("shared")
            sizes.append(m["shared"]["ff"])
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
        if len(shape) == 1:
            x = rng.normal(0.0, 0.5, shape) if last == "b" else 1.0 + 0.1 * rng.normal(size=shape)
        elif name in ("embed", "bigram"):
            x = rng.normal(0.0, 1.0 if name == "embed" else 0.5, shape)
        else:
            gain = 2.0 if last in ("q", "k", "router") else 1.0
            x = rng.normal(0.0, gain / np.sqrt(shape[1]), shape)
        w[name] = D.store_bfloat16(x)
    return w


def write_model(folder, cfg, w):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: torch.from_numpy(np.ascontiguousarray(v)).to(torch.bfloat16) for k, v in w.items()},
              os.path.join(folder, "model.safetensors"))
    return folder


CLOSE_CALL = 0.1   # router logits spread over several units; rounding to bfloat16 moves them by a few hundredths


class Oracle:
    """Exact logits [T, V] of one whole sequence and, per row, what rounding every stored activation to
    bfloat16 costs (root-mean-square distance from the exact row).  `decided[t]` is False where some router's
    choice for token t hangs on less than CLOSE_CALL: there rounding may pick another expert, in the engine as
    in the rounded plain run, and the row says nothing about either; bfloat16 comparisons leave such rows out
    (32-bit comparisons keep them)."""

    def __init__(self, cfg, w, tokens):
        margins = []
        self.exact = D.forward(cfg, w, tokens, margins_out=margins)
        self.decided = np.all(np.stack(margins) > CLOSE_CALL, axis=0) if margins else np.ones(len(tokens), bool)
        rounded = D.forward(cfg, w, tokens, store=D.store_bfloat16)
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

    def __getitem__(self, row):
        return self.exact[row]


def decided_tokens(cfg, w, n, seed, tries=200):
    """Random tokens whose routers all decide clearly (see `Oracle.decided`), and their oracle."""
    for k in range(tries):
        toks = [int(t) for t in np.random.default_rng(seed + 1000 * k).integers(0, cfg["vocab"], n)]
        margins = []
        D.forward(cfg, w, toks, margins_out=margins)
        if not margins or np.all(np.stack(margins) > CLOSE_CALL):
            return toks, Oracle(cfg, w, toks)
    raise AssertionError("no sequence of %d tokens without a close call among %d tries" % (n, tries))
