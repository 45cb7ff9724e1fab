"""The kernels behind Dobepel's mechanisms, each alone against its plain function (`plain_dobepel.py`):
pair embedding with the carried previous token, the merged norms and residual update, the gated norm, the
decayed linear attention with its carried state, attention with a bias by distance under a window that
keeps the first tokens (far keys, page borders, the window's and the kept tokens' edges, in prompts and
for single tokens), the router, the grouped products and the combination."""
import numpy as np
import pytest
import torch

import plain_dobepel as D

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def bf(x):
    return D.store_bfloat16(x)


def close(got, want, tol):
    got = got.float().cpu().numpy().astype(np.float64)
    scale = max(1.0, float(np.abs(want).max()))
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol * scale, "largest error %g of scale %g" % (np.abs(got - want).max(), scale)


TOL = {torch.float32: 2e-5, torch.bfloat16: 8e-3}   # (a bfloat16 result is rounded once: 2^-8 of its size)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_embedding_carries_the_previous_token_in_the_slot(dtype):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(0)
    V, E, buckets, a, b = 50, 24, 19, 1000003, 17
    table, pair = bf(rng.normal(size=(V, E))), bf(rng.normal(size=(buckets + 1, E)))
    seqs = {3: [int(t) for t in rng.integers(0, V, 9)], 0: [int(t) for t in rng.integers(0, V, 6)]}
    want = {s: D.embed(t, table, pair, buckets, a, b) for s, t in seqs.items()}
    last = torch.full((4,), -7, dtype=torch.int32, device=DEV)   # (garbage: a first token must not read it)
    # step 1: slot 3 brings 4 tokens, slot 0 brings 1; step 2: slot 0 brings 5, slot 3 brings 5
    for cut3, cut0 in (((0, 4), (0, 1)), ((4, 9), (1, 6))):
        ids = seqs[3][cut3[0]:cut3[1]] + seqs[0][cut0[0]:cut0[1]]
        n3, n0 = cut3[1] - cut3[0], cut0[1] - cut0[0]
        pos = list(range(cut3[0], cut3[1])) + list(range(cut0[0], cut0[1]))
        got = ops.embedding_pair(ints(ids), ints(pos), ints([0] * n3 + [1] * n0), ints([0, n3, n3 + n0]), ints([3, 0]),
                                 last, dev(table, dtype), dev(pair, dtype), buckets, a, b)
        close(got, np.concatenate([want[3][cut3[0]:cut3[1]], want[0][cut0[0]:cut0[1]]]), 1e-6)
    assert last.tolist()[3] == seqs[3][-1] and last.tolist()[0] == seqs[0][-1]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 256, 1030])
def test_merged_norms_and_residual_update(dtype, width):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(width)
    T, eps, m = 5, 1e-5, 0.3
    res = rng.normal(size=(T, width))
    y0, y1 = bf(rng.normal(size=(T, width)) * 3), bf(rng.normal(size=(T, width)) * 0.1)
    w0, w1, wp, wn = (bf(1 + 0.2 * rng.normal(size=width)) for _ in range(4))
    u = 0.5 * (D.rms_norm(y0, w0, eps) + D.rms_norm(y1, w1, eps))
    r_want = res + m * D.rms_norm(u, wp, eps)
    r = dev(res.astype(np.float32))
    h = ops.merge_norm_add_norm(r, dev(y0, dtype), dev(wp), m, eps, dev(w0), 0.5, dev(y1, dtype), dev(w1), 0.5, w_next=dev(wn))
    close(r, r_want.astype(np.float32).astype(np.float64), 1e-5)
    close(h, D.rms_norm(r_want, wn, eps), TOL[dtype])
    close(ops.merge_norms(dev(y0, dtype), dev(w0), 0.5, dev(y1, dtype), dev(w1), 0.5, eps), u, TOL[dtype])
    # one branch, no norm of its own, nothing after
    r2 = dev(res.astype(np.float32))
    assert ops.merge_norm_add_norm(r2, dev(y0, dtype), dev(wp), m, eps) is None
    close(r2, res + m * D.rms_norm(y0, wp, eps), 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_norm_and_activation(dtype):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(2)
    o, g, w = rng.normal(size=(7, 72)) * 4, bf(rng.normal(size=(7, 100)) * 2), bf(1 + 0.1 * rng.normal(size=72))
    packed = dev(g, dtype)
    got = ops.gated_rmsnorm(dev(o.astype(np.float32)), packed[:, 28:], dev(w), 1e-6)
    close(got, D.rms_norm(o.astype(np.float32).astype(np.float64), w, 1e-6) * D.sigmoid(g[:, 28:]), TOL[dtype])
    x = bf(rng.normal(size=(9, 33)) * 2)
    close(ops.act(dev(x, dtype), "gelu"), D.gelu_erf(x), TOL[dtype])
    close(ops.act(dev(x), "gelu", out_dtype=dtype), D.gelu_erf(x), TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Dk,Dv", [(3, 10, 40), (2, 64, 32), (1, 128, 128), (2, 7, 5), (3, 32, 96), (2, 32, 64), (2, 64, 192)])
def test_decayed_linear_attention_carries_its_state(dtype, H, Dk, Dv):
    """Three requests of 337, 1 and 570 tokens in portions (some of them single tokens) against the whole sequences;
    a far token's contribution survives hundreds of steps under a decay of 1 and dies under a small one.  In bfloat16
    the steps with a portion of 32 tokens or more run in the chunked kernel (sizes it takes), those with one of 256 or
    more with their chunks side by side, the others in the recurrent kernel: all must carry the same state."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(Dk)
    lens = [337, 1, 570]
    decay = np.asarray(([1.0, 0.9, 0.3] * H)[:H])
    W = 2 * H * Dk + H * Dv + 3   # (three columns of something else at the end of the packed rows)
    xs = [bf(rng.normal(size=(n, W))) for n in lens]
    want = []
    for x in xs:
        n = x.shape[0]
        store = bf if dtype == torch.bfloat16 else D.keep   # (a bfloat16 engine stores the activated projections rounded)
        q, k = store(D.silu(x[:, :H * Dk])).reshape(n, H, Dk), store(D.silu(x[:, H * Dk:2 * H * Dk])).reshape(n, H, Dk)
        v = store(D.silu(x[:, 2 * H * Dk:2 * H * Dk + H * Dv])).reshape(n, H, Dv)
        want.append(D.decayed_linear_attention(q, k, v, decay)[0].reshape(n, H * Dv))
    state = torch.full((5, H, Dk, Dv), float("nan"), device=DEV)
    slots = [4, 1, 2]
    for s in slots:
        state[s].zero_()
    cuts = [[20, 1, 1, 315], [1], [2, 433, 1, 134]]
    at, got = [0, 0, 0], [[], [], []]
    for step in range(4):
        rows, cu, sl, who = [], [0], [], []
        for r in range(3):
            if step < len(cuts[r]):
                rows.append(xs[r][at[r]:at[r] + cuts[r][step]])
                cu.append(cu[-1] + cuts[r][step])
                sl.append(slots[r])
                who.append(r)
        x = dev(np.concatenate(rows), dtype)
        o = ops.linear_attention(x, 0, H * Dk, 2 * H * Dk, dev(decay), state, ints(cu), ints(sl), len(who),
                                 max(b - a for a, b in zip(cu, cu[1:])), H, Dk, Dv, silu=True).cpu().numpy()
        for i, r in enumerate(who):
            got[r].append(o[cu[i]:cu[i + 1]])
            at[r] += cuts[r][step]
    for r in range(3):
        g = np.concatenate(got[r])
        scale = np.abs(want[r]).max()
        # (bfloat16: the device's silu differs from the host's by an ulp now and then, and rounding then goes the other way)
        tol = 1e-4 if dtype == torch.float32 else 2e-3
        assert np.abs(g - want[r]).max() <= tol * scale, (r, np.abs(g - want[r]).max(), scale)


def paged(k, v, page_size, n_pages, seed):
    """Keys [T, G, D] and values [T, G, Dv] of one request in shuffled pages: (k_pool, v_pool, table)."""
    T, G, Dk = k.shape
    Dv = v.shape[2]
    blocks = -(-T // page_size)
    table = np.random.default_rng(seed).permutation(n_pages)[:blocks]
    kp = np.full((n_pages, G, page_size, Dk), np.nan)
    vp = np.full((n_pages, G, page_size, Dv), np.nan)
    for j in range(T):
        kp[table[j // page_size], :, j % page_size] = k[j]
        vp[table[j // page_size], :, j % page_size] = v[j]
    return kp, vp, table


def attend(kernel, q, kp, vp, table, rows, dtype, scale, size, keep_first, exponent, H, G, Dk, Dv, page_size):
    """The kernel's output [len(rows), H * Dv] for the queries at positions `rows` of one request."""
    from velox_b200.csrc import ops
    T = len(rows)
    bt = torch.full((1, 64), -1, dtype=torch.int32, device=DEV)
    bt[0, :len(table)] = ints(table)
    qd = dev(q[rows].reshape(T, H * Dk), dtype)
    args = (qd, qd.shape[1], dev(kp, dtype), dev(vp, dtype), bt)
    if kernel == "general":
        return ops.paged_attention_generic(*args, ints([0] * T), ints(rows), scale, size, H, G, Dk, T, v_head_dim=Dv,
                                           keep_first=keep_first, bias_exponent=exponent)
    if kernel == "single":   # (few keys: one block a token and kv head; many: the keys cut into runs and joined)
        return ops.biased_decode_attention(*args, ints([0] * T), ints(rows), scale, size, keep_first, exponent, H, G, Dk, Dv, T,
                                           max_kv=max(rows) + 1)
    assert rows == list(range(rows[0], rows[0] + T))
    return ops.biased_prefill_attention(*args, ints([0, T]), ints([rows[0]]), scale, size, keep_first, exponent, H, G, Dk, Dv,
                                        1, T, T)


KERNELS = [("general", torch.float32), ("general", torch.bfloat16), ("single", torch.bfloat16), ("portion", torch.bfloat16)]


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("H,G,Dk,Dv,size,keep", [(4, 2, 64, 32, 40, 4), (8, 1, 64, 128, 100, 17), (2, 2, 128, 64, 16, 0),
                                                 (4, 4, 64, 64, 300, 1), (6, 2, 128, 128, 33, 16)])
def test_biased_window_attention_against_the_plain_function(kernel, dtype, H, G, Dk, Dv, size, keep):
    rng = np.random.default_rng(H * size)
    T, S, scale = 200, 16, 0.11
    q, k, v = bf(rng.normal(size=(T, H, Dk))), bf(rng.normal(size=(T, G, Dk))), bf(rng.normal(size=(T, G, Dv)))
    want = D.biased_window_attention(q, k, v, scale, size, keep).reshape(T, H * Dv)
    kp, vp, table = paged(k, v, S, 40, 3)
    for rows in (list(range(0, 200)), list(range(150, 200)), list(range(37, 39)), [199], [0], [size - 1], [size], [size + keep]):
        rows = [p for p in rows if p < T]
        if not rows:
            continue
        if kernel == "single" and len(rows) > 60:
            rows = rows[::7]
        if kernel == "portion" and len(rows) == 1:
            continue
        got = attend(kernel, q, kp, vp, table, rows, dtype, scale, size, keep, 8.0, H, G, Dk, Dv, S)
        close(got, want[rows], TOL[dtype])


@pytest.mark.parametrize("kernel,dtype", KERNELS)
def test_one_key_that_stands_out_is_seen_exactly_where_the_mask_says(kernel, dtype):
    """One key is made to dominate (a large dot product with every query) and its value is marked.  A query sees
    the mark iff the key is inside its window or among the kept first tokens: at the window's last position and not
    one further, at the last kept position and not the next, far away, at page borders, in a prompt's portion and
    for single tokens."""
    H, G, Dk, Dv, S, scale, T = 4, 2, 64, 32, 16, 0.25, 330
    rng = np.random.default_rng(4)
    for size, keep, spike in ((48, 3, 2), (48, 3, 3), (48, 3, 100), (32, 16, 15), (32, 16, 16), (64, 0, 0), (17, 5, 191)):
        q, k, v = bf(rng.normal(size=(T, H, Dk)) * 0.1), bf(rng.normal(size=(T, G, Dk)) * 0.1), bf(rng.normal(size=(T, G, Dv)) * 0.1)
        q[:, :, 0] = 8.0
        k[spike, :, 0] = 16.0    # score 0.25 * 128 = 32 above the rest; the distance bias takes at most 330 * 2^-2 from head 0 ...
        v[spike, :, :] = 100.0   # ... so head 3 (slope 2^-8) shows the mark at every distance
        kp, vp, table = paged(k, v, S, 30, 5)
        seen = [p for p in range(T) if spike <= p and (p - spike < size or spike < keep)]
        edge = sorted({spike, spike + size - 1, spike + size, spike + size + 1, T - 1, 255, 256} & set(range(spike, T)))
        for rows in ([[p] for p in edge] if kernel != "portion" else [list(range(max(0, spike - 3), T)), list(range(spike + size - 2, spike + size + 2))]):
            rows = [p for p in rows if p < T]
            if kernel == "portion" and len(rows) < 2:
                continue
            got = attend(kernel, q, kp, vp, table, rows, dtype, scale, size, keep, 8.0, H, G, Dk, Dv, S).float().cpu().numpy()
            got = got.reshape(len(rows), H, Dv)[:, 3, 0]
            for p, g in zip(rows, got):
                if p < spike:
                    continue
                assert (g > 50.0) == (p in seen), "window %d keep %d key %d query %d: %g" % (size, keep, spike, p, g)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,K,F,shared,T", [(3, 1, 40, 12, False, 150), (8, 3, 64, 48, True, 150), (5, 5, 72, 16, True, 150),
                                                 (16, 2, 128, 64, False, 150), (8, 3, 64, 48, True, 9), (16, 2, 128, 64, False, 40),
                                                 (4, 1, 200, 24, True, 1)])
def test_router_grouped_products_and_combination(dtype, E, top, K, F, shared, T):
    """150 tokens: row tiles of 64; 1, 9 and 40 tokens: in bfloat16 the row tiles of 16 of a decode step."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(E * top)
    h = bf(rng.normal(size=(T, K)))
    wr, b = bf(rng.normal(size=(E, K)) * 0.5), bf(rng.normal(size=E))
    w = {"router": wr, "router.b": b}
    for e in range(E):
        w.update({"e%d.gate" % e: bf(rng.normal(size=(F, K)) / 6), "e%d.up" % e: bf(rng.normal(size=(F, K)) / 6),
                  "e%d.down" % e: bf(rng.normal(size=(K, F)) / 4)})
    cfg = {"router": {"experts": E, "top": top}, "shared": None}
    want = D.routed_ff(h, w, "", cfg)
    chosen, weight = D.route(h, wr, b, top)
    rows_per_tile = ops.moe_tile_rows(dev(h, dtype), T * top) if F % 8 == 0 else ops.MOE_TILE_ROWS
    assert rows_per_tile == (16 if dtype == torch.bfloat16 and T * top <= 256 and F % 8 == 0 and K % 8 == 0 else 64)
    plan = ops.moe_route(dev(h, dtype), dev(wr), dev(b), E, top, rows_per_tile)
    assert (plan.chosen.view(T, top).cpu().numpy() == chosen).all()
    close(plan.weight, weight, 1e-5)
    # every assignment has a row of its own in expert order, experts ascending
    rows = plan.row_of.cpu().numpy()
    assert sorted(rows.tolist()) == list(range(T * top))
    assert (np.diff(chosen.reshape(-1)[np.argsort(rows)]) >= 0).all()
    tile = 8 if F % 8 == 0 else 0
    gu = np.stack([np.concatenate([w["e%d.gate" % e].reshape(-1, tile, K), w["e%d.up" % e].reshape(-1, tile, K)], 1).reshape(2 * F, K)
                   if tile else np.concatenate([w["e%d.gate" % e], w["e%d.up" % e]]) for e in range(E)])
    down = np.stack([w["e%d.down" % e] for e in range(E)])
    if tile:
        a = ops.moe_gemm(dev(h, dtype), dev(gu, dtype), plan, True, dtype, gated_activation="silu")
    else:
        a = ops.gated_act(ops.moe_gemm(dev(h, dtype), dev(gu, dtype), plan, True, torch.float32), "silu", 0, out_dtype=dtype)
    y = ops.moe_gemm(a, dev(down, dtype), plan, False, torch.float32)
    extra = bf(rng.normal(size=(T, K))) if shared else None
    got = ops.moe_combine(y, plan, dev(extra, dtype) if shared else None, dtype)
    close(got, want + (extra if shared else 0.0), TOL[dtype])
    # a second call on the same stream starts from clean counters
    plan2 = ops.moe_route(dev(h, dtype), dev(wr), dev(b), E, top, rows_per_tile)
    assert sorted(plan2.row_of.cpu().numpy().tolist()) == list(range(T * top))


@pytest.mark.parametrize("E,top,K,F,T", [(8, 2, 128, 64, 700), (4, 3, 256, 136, 400), (16, 1, 64, 8, 1500)])
def test_grouped_products_on_the_tcgen05_tensor_cores(E, top, K, F, T):
    """Enough assignments for row tiles of 128: the tokens' rows copied into expert order, both grouped products by
    the tcgen05 kernel (experts with no token, experts whose rows end inside a tile, a last column tile that ends
    inside the next expert's matrix), the combination from bfloat16 rows."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(T)
    h = bf(rng.normal(size=(T, K)))
    wr, b = bf(rng.normal(size=(E, K)) * 0.5), bf(rng.normal(size=E))
    b[E - 1] = -1e4   # the last expert never gets a token
    w = {"router": wr, "router.b": b}
    for e in range(E):
        w.update({"e%d.gate" % e: bf(rng.normal(size=(F, K)) / 6), "e%d.up" % e: bf(rng.normal(size=(F, K)) / 6),
                  "e%d.down" % e: bf(rng.normal(size=(K, F)) / 4)})
    want = D.routed_ff(h, w, "", {"router": {"experts": E, "top": top}, "shared": None}, store=bf)
    exact = D.routed_ff(h, w, "", {"router": {"experts": E, "top": top}, "shared": None})
    gu = np.stack([np.concatenate([w["e%d.gate" % e].reshape(-1, 8, K), w["e%d.up" % e].reshape(-1, 8, K)], 1).reshape(2 * F, K)
                   for e in range(E)])
    down = np.stack([w["e%d.down" % e] for e in range(E)])
    hd = dev(h, torch.bfloat16)
    assert ops.moe_tcgen05_supported(hd, T * top, 2 * F, K)
    plan = ops.moe_route(hd, dev(wr), dev(b), E, top, ops.MOE_TCGEN05_TILE_ROWS)
    a = ops.moe_gemm_tcgen05(ops.moe_gather_rows(hd, plan), dev(gu, torch.bfloat16), plan, gated_activation="silu")
    y = ops.moe_gemm_tcgen05(a, dev(down, torch.bfloat16), plan)
    got = ops.moe_combine(y, plan, None, torch.bfloat16)
    ops.check_device_errors()
    close(got, exact, 2e-2)
    # as far from the exact result as the plain implementation with the same roundings, give or take
    g = got.float().cpu().numpy().astype(np.float64)
    assert np.sqrt(np.mean((g - exact) ** 2)) <= 1.3 * np.sqrt(np.mean((want - exact) ** 2)) + 1e-6


@pytest.mark.parametrize("H,G,Dk,Dv,size,keep", [(8, 2, 128, 128, 1200, 4), (4, 4, 64, 32, 600, 0), (6, 2, 64, 64, 0, 0)])
def test_single_tokens_with_many_keys_are_cut_into_runs(H, G, Dk, Dv, size, keep):
    """Tokens deep in a sequence of 1,300 (a window of 600 or 1,200 keys, or every key) beside tokens near its start, in
    one call: the long ones' keys are cut into runs for several blocks and joined, the short ones' runs are mostly empty."""
    rng = np.random.default_rng(size + H)
    T, S, scale = 1300, 16, 0.1
    q, k, v = bf(rng.normal(size=(T, H, Dk))), bf(rng.normal(size=(T, G, Dk))), bf(rng.normal(size=(T, G, Dv)))
    want = D.biased_window_attention(q, k, v, scale, size if size else T + 1, keep).reshape(T, H * Dv)
    kp, vp, table = paged(k, v, S, 90, 7)
    rows = [1299, 0, 700, 15, 16, 1200, 599, 600, 601, 3]
    from velox_b200.csrc import ops
    bt = torch.full((1, 128), -1, dtype=torch.int32, device=DEV)
    bt[0, :len(table)] = ints(table)
    qd = dev(q[rows].reshape(len(rows), H * Dk), torch.bfloat16)
    got = ops.biased_decode_attention(qd, qd.shape[1], dev(kp, torch.bfloat16), dev(vp, torch.bfloat16), bt, ints([0] * len(rows)),
                                      ints(rows), scale, size, keep, 8.0, H, G, Dk, Dv, len(rows), max_kv=T)
    close(got, want[rows], TOL[torch.bfloat16])
