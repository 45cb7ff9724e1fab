"""Plain, slow Buvuzen decoder in numpy: the oracle of its tests.

Whole sequences, no cache, no pages, no batches; one function per mechanism; float64
unless a `store` function rounds what a 16-bit engine would store.  It shares no code
with the product path: it takes config.json as a dict and weights as a dict of numpy arrays.

Notation: T tokens, E model width, positions p = 0 .. T-1.
  rms(x)   = x / sqrt(mean(x^2) + eps)
  norm(x)  = rms(x) * (1 + w)                      (the file holds w, an offset from one)
  input:   x = embed[token] * c_in
  layer:   x += norm_1(mix(x)) ;  x += norm_2(ff(x))     (the sublayers read x itself; no feed-forward: one line)
  mixer:   q, k, v = W h per head; q, k <- rms(.) * w_q, w_k over the head (plain weights, shared by the heads);
           s[i, j] = scale * q_i . k_j for 0 <= i - j < size;
           a[i, j] = exp(s[i, j]) / (exp(sink_h) + sum_j' exp(s[i, j']))     (the sink has no value)
           o_i = sigmoid(W_g h_i)_head * sum_j a[i, j] v_j;  y = W_o [o of all heads]
  feed-forward: z = W_r h over R = experts + identity outputs; s = softmax(z) over all R;
           choice c = s + correction; R outputs in `count` equal groups of neighbours, a group's score its largest c,
           the best `keep` groups stay; among them the `top` largest c are chosen; weights s * c_r (no renormalising);
           output e < experts: W_down (silu(W_gate h) * W_up h); output e >= experts: h itself;
           plus sigmoid(w_sg . h) * shared(h)
  output:  logits = W_head norm_f(x) * c_out
"""
from __future__ import annotations

import numpy as np


def keep(x):
    return x


def store_bfloat16(x):
    """x rounded to bfloat16 (nearest even) and widened again."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def one_plus_norm(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def scaled_embedding(ids, table, scale):
    return table[np.asarray(ids, dtype=np.int64)] * scale


def window_visible(T, size):
    """[T, T] True where query i sees key j: 0 <= i - j < size (size 0: every earlier key)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) if size > 0 else True)


def sink_softmax(scores, visible, sink):
    """Rows of weights over the visible keys whose denominator also holds exp(sink): they sum to less than 1."""
    s = np.where(visible, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def sink_window_attention(q, k, v, scale, size, sinks):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; query head h reads kv head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    vis = window_visible(T, size)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        a = sink_softmax(scale * (q[:, h] @ k[:, g].T), vis, float(sinks[h]))
        out[:, h] = a @ v[:, g]
    return out


def attention_mixer(h, w, p, c, eps, store=keep):
    """The mixer of one layer: p is the tensors' prefix ('l0.mix.'), c the layer's `mixer` entry."""
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    hs = store(h)
    q = store(hs @ w[p + "q"].T).reshape(T, H, D)
    k = store(hs @ w[p + "k"].T).reshape(T, G, D)
    v = store(hs @ w[p + "v"].T).reshape(T, G, Dv)
    gate = sigmoid(store(hs @ w[p + "g"].T))                     # [T, H]
    q = store(rms(q, eps) * w[p + "q.norm"])
    k = store(rms(k, eps) * w[p + "k.norm"])
    size = int((c.get("mask") or {}).get("size", 0))
    o = sink_window_attention(q, k, v, float(c["scale"]), size, w[p + "sink"]) * gate[:, :, None]
    return store(store(o.reshape(T, H * Dv)) @ w[p + "o"].T)


def gated_expert(h, w, p, store=keep):
    a = store(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T))
    return a @ w[p + "down"].T


def group_limited_choice(choice, count, keep_groups, top):
    """Per row of `choice` [T, R]: the indices of the `top` largest among the outputs of the `keep_groups` groups
    (of R / count neighbours) whose largest entry is largest.  Equal values: the lower index first."""
    T, R = choice.shape
    size = R // count
    chosen = np.zeros((T, top), dtype=np.int64)
    for t in range(T):
        c = choice[t]
        best = np.asarray([c[g * size:(g + 1) * size].max() for g in range(count)])
        kept = np.argsort(-best, kind="stable")[:keep_groups]
        masked = np.full(R, -np.inf)
        for g in kept:
            masked[g * size:(g + 1) * size] = c[g * size:(g + 1) * size]
        chosen[t] = np.argsort(-masked, kind="stable")[:top]
    return chosen


def route(h, w_router, correction, r):
    """(chosen [T, top], weights [T, top], scores s [T, R], choice scores [T, R])."""
    z = h @ w_router.T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    choice = s + correction
    groups = r.get("groups") or {}
    chosen = group_limited_choice(choice, int(groups.get("count", 1)), int(groups.get("keep", 1)), int(r["top"]))
    weights = np.take_along_axis(s, chosen, axis=1) * float(r.get("scale", 1.0))
    return chosen, weights, s, choice


def route_margin(h, w_router, correction, r):
    """Per row the smallest gap that decides the choice: between the last kept and the first dropped group's score,
    and between the last chosen and the first not chosen output among the kept groups."""
    chosen, _, _, choice = route(h, w_router, correction, r)
    groups = r.get("groups") or {}
    count, keep_groups, top = int(groups.get("count", 1)), int(groups.get("keep", 1)), int(r["top"])
    T, R = choice.shape
    size = R // count
    out = np.full(T, np.inf)
    for t in range(T):
        best = np.sort(np.asarray([choice[t, g * size:(g + 1) * size].max() for g in range(count)]))[::-1]
        if keep_groups < count:
            out[t] = min(out[t], best[keep_groups - 1] - best[keep_groups])
        kept = np.argsort(-np.asarray([choice[t, g * size:(g + 1) * size].max() for g in range(count)]), kind="stable")[:keep_groups]
        vals = np.sort(np.concatenate([choice[t, g * size:(g + 1) * size] for g in kept]))[::-1]
        if top < len(vals):
            out[t] = min(out[t], vals[top - 1] - vals[top])
    return out


def routed_ff(h, w, p, c, store=keep, margins_out=None):
    """The feed-forward of one layer: p = 'l0.mlp.', c the layer's `mlp` entry."""
    r = c["router"]
    E, identity = int(r["experts"]), int(r.get("identity", 0))
    hs = store(h)
    chosen, weights, _, _ = route(hs, w[p + "router"], w[p + "correction"] if p + "correction" in w else 0.0, r)
    if margins_out is not None:
        margins_out.append(route_margin(hs, w[p + "router"], w[p + "correction"] if p + "correction" in w else 0.0, r))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            y = hs[t] if e >= E else gated_expert(hs[t:t + 1], w, p + "e%d." % e, store)[0]
            out[t] += wt * y
    if c.get("shared") is not None:
        out = out + sigmoid(hs @ w[p + "shared.sg"].T) * gated_expert(hs, w, p + "shared.", store)
    return store(out)


def layer_sources(cfg):
    """Per layer the layer whose tensors it uses: itself, or the one its `weights_of` leads to."""
    out = []
    for i in range(len(cfg["layers"])):
        while cfg["layers"][i].get("weights_of") is not None:
            i = int(cfg["layers"][i]["weights_of"])
        out.append(i)
    return out


def forward(cfg, w, ids, store=keep, layers_out=None, margins_out=None):
    """Logits [T, vocab] of the whole sequence `ids`."""
    eps = float(cfg["norm"]["eps"])
    x = scaled_embedding(ids, w["embed"], float((cfg.get("embedding") or {}).get("scale", 1.0)))
    for i, src in enumerate(layer_sources(cfg)):
        layer, p = cfg["layers"][src], "l%d." % src
        x = x + one_plus_norm(attention_mixer(x, w, p + "mix.", layer["mixer"], eps, store), w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + one_plus_norm(routed_ff(x, w, p + "mlp.", layer["mlp"], store, margins_out), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    h = store(one_plus_norm(x, w["final.norm"], eps))
    return (h @ w["head"].T) * float(cfg.get("logit_scale", 1.0))


def greedy_generate(cfg, w, prompt, new_tokens):
    ids = [int(t) for t in prompt]
    for _ in range(new_tokens):
        ids.append(int(np.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
