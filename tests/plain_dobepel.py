"""Plain, slow Dobepel decoder in numpy: the oracle of its tests.

Whole sequences, no cache, no pages, no batches; one function per mechanism; float64
unless a `store` function rounds what a 16-bit engine would store.  It shares no code
with the product path: it reads config.json with `json` and takes weights as a dict
of numpy arrays.

Notation: T tokens, E model width, positions p = 0 .. T-1.
  rms(x) = x / sqrt(mean(x^2) + eps)
  layer:  x += m * rms(mix(rms(x) w1)) w1b ;  x += m * rms(ff(rms(x) w2)) w2b
  mixer "parallel" = ( rms(A(h)) a + rms(L(h)) l ) / 2 with
    A: softmax attention, score[i, j] = scale * q_i.k_j - 2^(-8 (head+1) / H) * (i - j), keys j <= i with
       i - j < size or j < keep_first; grouped key/value heads; no rotation
    L: per head S_p = d S_(p-1) + k_p v_p^T, o_p = S_p^T q_p, with q, k, v = silu(W h); heads joined, rms-normed
       with a weight, times sigmoid(W_g h), projected
  feed-forward: dense = W_down gelu(W_up h); routed = sum over the `top` largest router logits z_e of
       softmax_chosen(z)_e * expert_e(h), plus a shared expert; expert = W_down (silu(W_gate h) * W_up h)
  input: embed[token] + bigram[(prev * a + token * b) mod buckets], the table's last row for p = 0
"""
from __future__ import annotations

import math

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


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_erf(z):
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return 0.5 * z * (1.0 + erf(z / math.sqrt(2.0)))


def bigram_rows(ids, buckets, mul_prev, mul_cur):
    ids = [int(t) for t in ids]
    return np.asarray([buckets if p == 0 else (ids[p - 1] * mul_prev + ids[p] * mul_cur) % buckets
                       for p in range(len(ids))], dtype=np.int64)


def embed(ids, table, bigram, buckets, mul_prev, mul_cur):
    return table[np.asarray(ids, dtype=np.int64)] + bigram[bigram_rows(ids, buckets, mul_prev, mul_cur)]


def distance_slopes(heads):
    return np.asarray([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])


def visible(T, size, keep_first):
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def biased_window_attention(q, k, v, scale, size, keep_first):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    slopes = distance_slopes(H)
    dist = (np.arange(T)[:, None] - np.arange(T)[None, :]).astype(np.float64)
    mask = visible(T, size, keep_first)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale - slopes[h] * dist
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def decayed_linear_attention(q, k, v, decay, state=None):
    """q, k [T, H, D], v [T, H, Dv], decay [H] -> ([T, H, Dv], final state [H, D, Dv]); token by token."""
    T, H, D = q.shape
    S = np.zeros((H, D, v.shape[2])) if state is None else state.copy()
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + np.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out, S


def left_mixer(h, w, p, c, store=keep):
    T = h.shape[0]
    H, G, D, Dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = store(h @ w[p + "q"].T).reshape(T, H, D)
    k = store(h @ w[p + "k"].T).reshape(T, G, D)
    v = store(h @ w[p + "v"].T).reshape(T, G, Dv)
    a = biased_window_attention(q, k, v, c["scale"], c["mask"]["size"], c["mask"]["keep_first"])
    return store(store(a.reshape(T, H * Dv)) @ w[p + "o"].T)


def right_mixer(h, w, p, c, eps, store=keep):
    T = h.shape[0]
    H, D, Dv = c["heads"], c["dim"], c["vdim"]
    q = store(silu(h @ w[p + "q"].T)).reshape(T, H, D)
    k = store(silu(h @ w[p + "k"].T)).reshape(T, H, D)
    v = store(silu(h @ w[p + "v"].T)).reshape(T, H, Dv)
    o, _ = decayed_linear_attention(q, k, v, np.asarray(c["decay"], dtype=np.float64))
    o = rms_norm(o.reshape(T, H * Dv), w[p + "norm"], eps) * sigmoid(h @ w[p + "g"].T)
    return store(store(o) @ w[p + "o"].T)


def parallel_mixer(h, w, p, c, eps, store=keep):
    a = rms_norm(left_mixer(h, w, p + "left.", c["left"], store), w[p + "left.out"], eps)
    b = rms_norm(right_mixer(h, w, p + "right.", c["right"], eps, store), w[p + "right.out"], eps)
    return 0.5 * (a + b)


def dense_ff(h, w, p, store=keep):
    return store(store(gelu_erf(h @ w[p + "up"].T)) @ w[p + "down"].T)


def gated_expert(h, w, p, store=keep):
    return store(store(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T)


def route(h, w_router, bias, top):
    """(chosen experts [T, top], their weights [T, top])."""
    z = h @ w_router.T + bias
    chosen = np.argsort(-z, axis=1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, chosen, axis=1)
    e = np.exp(zc - zc.max(axis=1, keepdims=True))
    return chosen, e / e.sum(axis=1, keepdims=True)


def route_margin(h, w_router, bias, top):
    """Per token the gap between the last chosen logit and the first one left out (inf if none is left out)."""
    z = -np.sort(-(h @ w_router.T + bias), axis=1)
    return z[:, top - 1] - z[:, top] if top < z.shape[1] else np.full(h.shape[0], np.inf)


def routed_ff(h, w, p, c, store=keep, margins_out=None):
    chosen, weight = route(h, w[p + "router"], w[p + "router.b"], c["router"]["top"])
    if margins_out is not None:
        margins_out.append(route_margin(h, w[p + "router"], w[p + "router.b"], c["router"]["top"]))
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]))
    for e in range(c["router"]["experts"]):
        rows, col = np.nonzero(chosen == e)
        if len(rows):
            out[rows] += weight[rows, col][:, None] * gated_expert(h[rows], w, p + "e%d." % e, store)
    if c.get("shared"):
        out += gated_expert(h, w, p + "shared.", store)
    return store(out)


def forward(cfg, w, ids, store=keep, layers_out=None, margins_out=None):
    """Logits [T, vocab] of a whole sequence; `layers_out` (a list) gets the residual after every layer,
    `margins_out` (a list) every routed layer's `route_margin`."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    b = cfg["embedding"]["bigram"]
    x = embed(ids, w["embed"], w["bigram"], b["buckets"], b["mul_prev"], b["mul_cur"])
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        assert layer["type"] == "parallel"
        h = store(rms_norm(x, w[p + "norm1"], eps))
        x = x + m * rms_norm(parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, store), w[p + "norm1b"], eps)
        if layer.get("mlp"):
            h = store(rms_norm(x, w[p + "norm2"], eps))
            f = dense_ff(h, w, p + "mlp.", store) if layer["mlp"]["kind"] == "dense" else \
                routed_ff(h, w, p + "mlp.", layer["mlp"], store, margins_out)
            x = x + m * rms_norm(f, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return store(rms_norm(x, w["final.norm"], eps)) @ w["head"].T


def greedy_generate(cfg, w, prompt, new_tokens):
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(np.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]
