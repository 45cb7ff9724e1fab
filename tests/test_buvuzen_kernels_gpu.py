"""The kernels behind Buvuzen's mechanisms, each alone against its plain function (`plain_buvuzen.py`): the scaled
embedding with its rounded copy, the residual update that norms a sublayer's output and hands on the rounded stream,
the q/k norm with values of another size written into pages, attention with a sink and an output gate under a window
(far keys, page borders, the window's edge, a sink that dominates, in prompts and for single tokens, in the general
kernel and the tensor-core ones), the router (one softmax over all outputs, a correction that moves the choice only,
groups, identity experts, the shared expert's gate), the combination, and the scaled logits."""
import numpy as np
import pytest
import torch

import plain_buvuzen as B

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def dev(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def ints(x):
    return torch.tensor(list(x), dtype=torch.int32, device=DEV)


def bf(x):
    return B.store_bfloat16(x)


def close(got, want, tol):
    got = got.float().cpu().numpy().astype(np.float64)
    scale = max(1.0, float(np.abs(want).max()))
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= tol * scale, "largest error %g of scale %g" % (np.abs(got - want).max(), scale)


TOL = {torch.float32: 2e-5, torch.bfloat16: 8e-3}   # (a bfloat16 result is rounded once: 2^-8 of its size)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scaled_embedding_and_its_rounded_copy(dtype):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(0)
    table = bf(rng.normal(size=(50, 24)))
    ids = [3, 49, 0, 3, 17]
    rounded = torch.empty((5, 24), dtype=dtype, device=DEV)
    got = ops.embedding(ints(ids), dev(table, dtype), scale=1.75, rounded=rounded)
    want = B.scaled_embedding(ids, table, 1.75)
    close(got, want, 1e-6)
    assert torch.equal(rounded, got.to(dtype))
    close(ops.embedding(ints(ids), dev(table, dtype)), table[ids], 0.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 256, 1030])
def test_the_residual_takes_a_normed_output_and_hands_on_its_rounding(dtype, width):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(width)
    x, y, w = rng.normal(size=(7, width)) * 3, bf(rng.normal(size=(7, width))), bf(rng.normal(size=width) * 0.1)
    res = dev(x)
    one_plus = (dev(w) + 1.0).contiguous()
    h = ops.merge_norm_add_norm(res, dev(y, dtype), one_plus, 1.0, 1e-5, rounded=True)
    want = x.astype(np.float32).astype(np.float64) + B.one_plus_norm(y, w, 1e-5)
    close(res, want, 2e-6)
    assert h.dtype == dtype and torch.equal(h, res.to(dtype))
    assert ops.merge_norm_add_norm(res, dev(y, dtype), one_plus, 1.0, 1e-5) is None
    assert torch.equal(ops.cast_rows(res, dtype), res.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Dv,extra", [(4, 2, 24, 20, 4), (2, 2, 128, 128, 0), (3, 1, 64, 32, 5), (2, 1, 27, 40, 2)])
def test_qk_norm_with_values_of_another_size_into_pages(dtype, H, G, D, Dv, extra):
    """Rows [q | k | v | extra columns]: q normed in place, k normed into its pool, v copied into a pool of its own
    width, the extra columns (a gate's) untouched; a token with a negative slot writes nothing."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(D)
    T, S, pages, eps = 9, 4, 5, 1e-5
    row = bf(rng.normal(size=(T, (H + G) * D + G * Dv + extra)))
    wq, wk = bf(1 + 0.2 * rng.normal(size=D)), bf(1 + 0.2 * rng.normal(size=D))
    slots = [13, 2, -1, 7, 19, 0, 5, 6, 11]
    qkv = dev(row, dtype)
    kp = torch.full((pages, G, S, D), float("nan"), dtype=dtype, device=DEV)
    vp = torch.full((pages, G, S, Dv), float("nan"), dtype=dtype, device=DEV)
    ops.qk_norm_rope_kv(qkv, dev(wq), dev(wk), eps, None, 0, ints(range(T)), ints(slots), kp, vp, H, G, D, Dv)
    q = row[:, :H * D].reshape(T, H, D)
    k = row[:, H * D:(H + G) * D].reshape(T, G, D)
    v = row[:, (H + G) * D:(H + G) * D + G * Dv].reshape(T, G, Dv)
    close(qkv[:, :H * D], (B.rms(q, eps) * wq).reshape(T, H * D), TOL[dtype])
    assert torch.equal(qkv[:, (H + G) * D + G * Dv:], dev(row, dtype)[:, (H + G) * D + G * Dv:])
    kn = B.rms(k, eps) * wk
    for t, s in enumerate(slots):
        if s < 0:
            continue
        close(kp[s // S, :, s % S], kn[t], TOL[dtype])
        close(vp[s // S, :, s % S], v[t], 0.0)
    written = {s for s in slots if s >= 0}
    for s in range(pages * S):
        if s not in written:
            assert torch.isnan(kp[s // S, :, s % S]).all() and torch.isnan(vp[s // S, :, s % S]).all()


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


def attend(kernel, q, gates, kp, vp, table, rows, dtype, scale, size, sinks, H, G, Dk, Dv, blocks=96):
    """The kernel's output [len(rows), H * Dv] for the queries at positions `rows` of one request.  The query rows
    are [q heads | gate logits], as the fused projection leaves them."""
    from velox_b200.csrc import ops
    T = len(rows)
    bt = torch.full((1, blocks), -1, dtype=torch.int32, device=DEV)
    bt[0, :len(table)] = ints(table)
    pad = (-(H * Dk + H)) % 8
    qd = dev(np.concatenate([q[rows].reshape(T, H * Dk), gates[rows], np.zeros((T, pad))], axis=1), dtype)
    more = dict(sinks=None if sinks is None else dev(sinks), gate_col=H * Dk)
    args = (qd, qd.shape[1], dev(kp, dtype), dev(vp, dtype), bt)
    if kernel == "general":
        return ops.paged_attention_generic(*args, ints([0] * T), ints(rows), scale, size, H, G, Dk, T, v_head_dim=Dv, **more)
    if kernel == "single":
        return ops.biased_decode_attention(*args, ints([0] * T), ints(rows), scale, size, 0, 0.0, H, G, Dk, Dv, T,
                                           max_kv=max(rows) + 1, **more)
    assert rows == list(range(rows[0], rows[0] + T))
    if kernel == "portion_tc":   # (the tcgen05 kernel with the probabilities in two halves; key tiles in runs when there are many)
        got = ops.paged_prefill_attention_tc(*args, ints([0, T]), ints([rows[0]]), scale, size, H, G, Dk, 1, T, T,
                                             max_kv=rows[-1] + 1, halves=True, **more)
        ops.check_device_errors()
        return got
    return ops.biased_prefill_attention(*args, ints([0, T]), ints([rows[0]]), scale, size, 0, 0.0, H, G, Dk, Dv, 1, T, T, **more)


def gated_plain(q, k, v, gates, scale, size, sinks):
    o = B.sink_window_attention(q, k, v, scale, size, sinks) * B.sigmoid(gates)[:, :, None]
    return o.reshape(q.shape[0], -1)


KERNELS = [("general", torch.float32), ("general", torch.bfloat16), ("single", torch.bfloat16), ("portion", torch.bfloat16),
           ("portion_tc", torch.bfloat16)]


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("H,G,Dk,Dv,size", [(4, 2, 64, 32, 40), (8, 1, 64, 128, 100), (2, 2, 128, 64, 16), (4, 4, 64, 64, 300),
                                            (6, 2, 128, 128, 33), (3, 3, 64, 64, 0), (4, 2, 24, 20, 9), (5, 1, 48, 56, 70),
                                            (6, 3, 48, 48, 50), (4, 1, 32, 32, 21), (2, 2, 80, 80, 64), (4, 2, 96, 96, 17),
                                            (3, 1, 112, 112, 130), (8, 2, 128, 128, 100), (5, 1, 128, 128, 0), (4, 4, 128, 128, 300)])
def test_sink_and_gate_attention_against_the_plain_function(kernel, dtype, H, G, Dk, Dv, size):
    from velox_b200.csrc import ops
    if kernel == "portion_tc" and not (Dk == Dv == 128):
        pytest.skip("the tcgen05 kernel takes heads of 128")
    if kernel != "general" and not ops.biased_attention_supported(dtype, Dk, Dv, 16):
        pytest.skip("sizes the tensor-core kernels do not take")
    rng = np.random.default_rng(H * (size + 1))
    T, S, scale = 200, 16, 0.11
    q, k, v = bf(rng.normal(size=(T, H, Dk))), bf(rng.normal(size=(T, G, Dk))), bf(rng.normal(size=(T, G, Dv)))
    gates, sinks = bf(rng.normal(size=(T, H)) * 2), bf(rng.normal(size=H) * 2)
    want = gated_plain(q, k, v, gates, scale, size, sinks)
    kp, vp, table = paged(k, v, S, 40, 3)
    for rows in (list(range(0, 200)), list(range(150, 200)), list(range(37, 39)), [199], [0], [1], [size - 1], [size], [size + 1]):
        rows = [p for p in rows if 0 <= p < T]
        if not rows:
            continue
        if kernel == "single" and len(rows) > 60:
            rows = rows[::7]
        if kernel in ("portion", "portion_tc") and len(rows) == 1:
            continue
        got = attend(kernel, q, gates, kp, vp, table, rows, dtype, scale, size, sinks, H, G, Dk, Dv)
        close(got, want[rows], TOL[dtype])


@pytest.mark.parametrize("H,G,size", [(8, 2, 1200), (4, 4, 600), (5, 1, 0)])
def test_the_tcgen05_kernel_joins_runs_of_key_tiles_with_the_sink_counted_once(H, G, size):
    """A portion of 50 tokens on top of 1,250 cached ones: its key tiles are cut into runs for several blocks and joined;
    beside it the same queries as one long prompt from the start (no runs)."""
    rng = np.random.default_rng(size + H)
    T, S, scale, D = 1300, 16, 0.1, 128
    q, k, v = bf(rng.normal(size=(T, H, D))), bf(rng.normal(size=(T, G, D))), bf(rng.normal(size=(T, G, D)))
    gates, sinks = bf(rng.normal(size=(T, H)) * 2), bf(rng.normal(size=H) * 2 + 3)
    want = gated_plain(q, k, v, gates, scale, size, sinks)
    kp, vp, table = paged(k, v, S, 90, 7)
    for rows in (list(range(1250, 1300)), list(range(0, 1300)), list(range(700, 1100))):
        got = attend("portion_tc", q, gates, kp, vp, table, rows, torch.bfloat16, scale, size, sinks, H, G, D, D, blocks=128)
        close(got, want[rows], TOL[torch.bfloat16])


@pytest.mark.parametrize("kernel,dtype", KERNELS)
def test_a_sink_above_every_score_empties_the_row_and_one_far_below_changes_nothing(kernel, dtype):
    """Head 0's sink lies 40 above every score (its output is e^-40 of a value: nothing), head 1's 40 below (plain
    softmax), head 2 has the sink of a row's first token only (position 0: half of the weight goes to the sink when it
    equals the only score), head 3 a moderate one."""
    H, G, Dk, Dv, S, T, size, scale = 4, 2, 64, 32, 16, 70, 24, 0.125
    if kernel == "portion_tc":
        Dk = Dv = 128
    rng = np.random.default_rng(8)
    q, k, v = bf(rng.normal(size=(T, H, Dk)) * 0.3), bf(rng.normal(size=(T, G, Dk)) * 0.3), bf(rng.normal(size=(T, G, Dv)))
    q[0, 2], k[0, 1] = 0.0, 0.0
    q[0, 2, 0], k[0, 1, 0] = 4.0, 2.0            # the only score of row 0, head 2: 0.125 * 8 = 1
    sinks = np.asarray([40.0, -40.0, 1.0, 0.5])
    gates = np.full((T, H), 30.0)                # (gates wide open)
    kp, vp, table = paged(k, v, S, 8, 1)
    want = gated_plain(q, k, v, gates, scale, size, sinks)
    plain = B.sink_window_attention(q, k, v, scale, size, np.full(H, -np.inf)).reshape(T, H, Dv)
    for rows in ([0, 1], list(range(20, 70))) if kernel in ("portion", "portion_tc") else ([0], [1], [23], [24], [69]):
        got = attend(kernel, q, gates, kp, vp, table, rows, dtype, scale, size, sinks, H, G, Dk, Dv)
        close(got, want[rows], TOL[dtype])
        g = got.float().cpu().numpy().reshape(len(rows), H, Dv)
        assert np.abs(g[:, 0]).max() < 1e-12
        assert np.abs(g[:, 1] - plain[rows, 1]).max() <= TOL[dtype] * max(1.0, np.abs(plain).max())
        if rows[0] == 0:
            assert np.abs(g[0, 2] - 0.5 * v[0, 1]).max() <= TOL[dtype] * max(1.0, np.abs(v).max())


@pytest.mark.parametrize("Dk,Dv", [(64, 32), (48, 48), (96, 96), (128, 128)])
@pytest.mark.parametrize("kernel,dtype", KERNELS)
def test_one_key_that_stands_out_is_seen_exactly_as_long_as_the_window_says(kernel, dtype, Dk, Dv):
    if (kernel == "portion_tc") != (Dk == 128):
        pytest.skip("heads of 128 on the tcgen05 kernel, the others on the rest")
    """One key is made to dominate (a large dot product with every query) and its value is marked.  A query sees the
    mark iff the key is inside its window: at the window's last position and not one further, far away under no window,
    at page borders, with the key in the request's first page, in a prompt's portion and for single tokens.  A closed
    gate hides it again."""
    H, G, S, scale, T = 4, 2, 16, 0.25, 330
    rng = np.random.default_rng(4)
    sinks = np.asarray([0.0, 3.0, -2.0, 1.0])
    for size, spike in ((48, 2), (48, 100), (32, 15), (32, 16), (64, 0), (17, 191), (0, 1), (1, 200), (300, 17)):
        q, k, v = bf(rng.normal(size=(T, H, Dk)) * 0.1), bf(rng.normal(size=(T, G, Dk)) * 0.1), bf(rng.normal(size=(T, G, Dv)) * 0.1)
        gates = np.full((T, H), 30.0)
        gates[:, 2] = -30.0                       # head 2's gate is shut at every token
        q[:, :, 0] = 8.0
        k[spike, :, 0] = 16.0                     # score 0.25 * 128 = 32 above the rest and above every sink
        v[spike, :, :] = 100.0
        kp, vp, table = paged(k, v, S, 30, 5)
        seen = [p for p in range(T) if spike <= p and (size == 0 or p - spike < size)]
        far = size if size else T
        edge = sorted({spike, spike + far - 1, spike + far, spike + far + 1, T - 1, 255, 256} & set(range(spike, T)))
        if kernel not in ("portion", "portion_tc"):
            cases = [[p] for p in edge]
        else:
            cases = [list(range(max(0, spike - 3), T)), list(range(max(0, spike + far - 2), min(T, spike + far + 2)))]
        for rows in cases:
            if kernel in ("portion", "portion_tc") and len(rows) < 2:
                continue
            got = attend(kernel, q, gates, kp, vp, table, rows, dtype, scale, size, sinks, H, G, Dk, Dv)
            got = got.float().cpu().numpy().reshape(len(rows), H, Dv)
            for p, g in zip(rows, got):
                if p < spike:
                    continue
                for head in (0, 1, 3):
                    assert (g[head, 0] > 50.0) == (p in seen), "window %d key %d query %d head %d: %g" % (size, spike, p, head, g[head, 0])
                assert abs(g[2, 0]) < 1e-9


@pytest.mark.parametrize("H,G,Dk,Dv,size", [(8, 2, 128, 128, 1200), (4, 4, 64, 32, 600), (6, 2, 64, 64, 0), (6, 6, 48, 48, 700),
                                            (2, 1, 112, 112, 0)])
def test_single_tokens_with_many_keys_join_their_runs_with_the_sink_counted_once(H, G, Dk, Dv, size):
    """Tokens deep in a sequence of 1,300 beside tokens near its start, in one call: the long ones' keys are cut into
    runs for several blocks and joined; the sink enters the joined denominator once, the gate the joined output."""
    from velox_b200.csrc import ops
    rng = np.random.default_rng(size + H)
    T, S, scale = 1300, 16, 0.1
    q, k, v = bf(rng.normal(size=(T, H, Dk))), bf(rng.normal(size=(T, G, Dk))), bf(rng.normal(size=(T, G, Dv)))
    gates, sinks = bf(rng.normal(size=(T, H)) * 2), bf(rng.normal(size=H) * 2 + 3)
    want = gated_plain(q, k, v, gates, scale, size, sinks)
    kp, vp, table = paged(k, v, S, 90, 7)
    rows = [1299, 0, 700, 15, 16, 1200, 599, 600, 601, 3]
    got = attend("single", q, gates, kp, vp, table, rows, torch.bfloat16, scale, size, sinks, H, G, Dk, Dv, blocks=128)
    close(got, want[rows], TOL[torch.bfloat16])


def router_case(rng, R, K, T, identity, shared, F):
    h = bf(rng.normal(size=(T, K)))
    w = {"router": bf(rng.normal(size=(R, K)) * 0.6), "correction": bf(rng.normal(size=R) * 0.08)}
    for e in range(R - identity):
        w.update({"e%d.gate" % e: bf(rng.normal(size=(F, K)) / 6), "e%d.up" % e: bf(rng.normal(size=(F, K)) / 6),
                  "e%d.down" % e: bf(rng.normal(size=(K, F)) / 4)})
    if shared:
        w.update({"shared.gate": bf(rng.normal(size=(F, K)) / 6), "shared.up": bf(rng.normal(size=(F, K)) / 6),
                  "shared.down": bf(rng.normal(size=(K, F)) / 4), "shared.sg": bf(rng.normal(size=(1, K)) * 0.5)})
    return h, w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("R,identity,top,groups,keep,K,F,shared,T", [
    (6, 1, 3, 3, 2, 40, 12, True, 150), (8, 2, 3, 4, 2, 64, 48, True, 150), (4, 0, 4, 1, 1, 72, 16, False, 150),
    (16, 4, 4, 2, 1, 128, 64, True, 150), (8, 2, 3, 4, 2, 64, 48, True, 9), (16, 0, 2, 8, 3, 128, 64, False, 40),
    (3, 2, 1, 1, 1, 200, 24, True, 1), (40, 8, 6, 5, 2, 64, 16, True, 33), (9, 3, 9, 3, 3, 48, 8, False, 20)])
def test_router_with_groups_identity_experts_and_a_gated_shared_expert(dtype, R, identity, top, groups, keep, K, F, shared, T):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(R * top + T)
    h, w = router_case(rng, R, K, T, identity, shared, F)
    E = R - identity
    r = {"experts": E, "identity": identity, "top": top, "scale": 1.75, "groups": {"count": groups, "keep": keep}}
    cfg = {"router": r, "expert": {"ff": F}, "shared": {"ff": F} if shared else None}
    want = B.routed_ff(h, w, "", cfg)
    chosen, weight, _, _ = B.route(h, w["router"], w["correction"], r)
    margin = B.route_margin(h, w["router"], w["correction"], r)
    sure = margin > 1e-4                       # (float32 logits differ from the plain ones in the last bits)
    wr = np.concatenate([w["router"], w["shared.sg"]]) if shared else w["router"]
    hd = dev(h, dtype)
    rows_per_tile = ops.moe_tile_rows(hd, T * top) if F % 8 == 0 else ops.MOE_TILE_ROWS
    plan = ops.moe_route(hd, dev(wr), None, R, top, rows_per_tile, scores="softmax_all", correction=dev(w["correction"]),
                         groups=groups, keep_groups=keep, route_scale=1.75, identity=identity, shared_gate=shared)
    got_chosen = plan.chosen.view(T, top).cpu().numpy()
    assert (got_chosen[sure] == chosen[sure]).all()
    close(plan.weight[torch.from_numpy(sure).to(DEV)], weight[sure], 1e-5)
    if shared:
        close(plan.shared_gate, B.sigmoid(h @ w["shared.sg"].T)[:, 0], 1e-5)
    # the tiles cover exactly the assignments that went to experts with matrices
    tiles = plan.tiles.cpu().numpy()[:3 * int(plan.n_tiles.item())].reshape(-1, 3)
    assert tiles[:, 2].sum() == int((got_chosen < E).sum()) and (tiles[:, 0] < E).all()
    tile = 8 if F % 8 == 0 else 0
    gu = np.stack([np.concatenate([w["e%d.gate" % e].reshape(-1, tile, K), w["e%d.up" % e].reshape(-1, tile, K)], 1).reshape(2 * F, K)
                   if tile else np.concatenate([w["e%d.gate" % e], w["e%d.up" % e]]) for e in range(E)])
    down = np.stack([w["e%d.down" % e] for e in range(E)])
    if tile:
        a = ops.moe_gemm(hd, dev(gu, dtype), plan, True, dtype, gated_activation="silu")
    else:
        a = ops.gated_act(ops.moe_gemm(hd, dev(gu, dtype), plan, True, torch.float32), "silu", 0, out_dtype=dtype)
    y = ops.moe_gemm(a, dev(down, dtype), plan, False, torch.float32)
    if identity:                                  # rows of identity experts are never computed, and never read
        lost = plan.row_of[(plan.chosen >= E)].long()
        y[lost] = float("nan")
    extra = bf(B.gated_expert(h, w, "shared.")) if shared else None
    got = ops.moe_combine(y, plan, dev(extra, dtype) if shared else None, dtype, h=hd)
    if shared:
        want = want - B.sigmoid(h @ w["shared.sg"].T) * (B.gated_expert(h, w, "shared.") - extra)
    ok = torch.from_numpy(sure).to(DEV)
    close(got[ok], want[sure], TOL[dtype])


def test_a_correction_moves_the_choice_and_not_the_weights_and_a_dropped_group_is_out_whatever_it_scores():
    """Two tokens made by hand.  Outputs 0..5 in three groups of two, one kept group... the best single output lies in
    a group that the correction pushes out; negative choice scores inside the kept groups still beat dropped ones."""
    from velox_b200.csrc import ops
    K = 8
    h = np.zeros((2, K))
    h[:, 0] = 1.0
    router = np.zeros((6, K))
    router[:, 0] = [2.0, 0.0, 1.0, 0.5, 0.0, -1.0]          # scores: output 0 is far the best
    s = np.exp(router[:, 0]) / np.exp(router[:, 0]).sum()
    correction = np.asarray([-2.0, -2.0, 0.0, -1.0, -0.05, -0.06])
    plan = ops.moe_route(dev(h), dev(router), None, 6, 3, 64, scores="softmax_all", correction=dev(correction), groups=3,
                         keep_groups=2, route_scale=2.0, identity=1)
    # choice scores: [s0-2, s1-2, s2, s3-1, s4-.05, s5-.06]: groups 1 and 2 stay; inside them 2 first, then 4, then 5
    # (negative, but of a kept group), never 3 before them and never 0 or 1
    assert plan.chosen.view(2, 3).cpu().tolist() == [[2, 4, 5]] * 2
    close(plan.weight, np.asarray([[2 * s[2], 2 * s[4], 2 * s[5]]] * 2), 1e-6)
    y = torch.full((6, K), float("nan"), device=DEV)
    got = ops.moe_combine(y.nan_to_num(7.0), plan, None, torch.float32, h=dev(h))
    # output 5 is the identity expert: the token itself; outputs 2 and 4 take their rows of y (all 7 here)
    close(got, 2 * (s[2] + s[4]) * 7.0 + 2 * s[5] * h, 1e-5)


@pytest.mark.parametrize("T", [700, 1500])
def test_identity_experts_beside_the_tcgen05_grouped_products(T):
    from velox_b200.csrc import ops
    rng = np.random.default_rng(T)
    R, identity, top, K, F = 10, 2, 3, 128, 64
    h, w = router_case(rng, R, K, T, identity, True, F)
    E = R - identity
    r = {"experts": E, "identity": identity, "top": top, "scale": 2.0, "groups": {"count": 5, "keep": 3}}
    exact = B.routed_ff(h, w, "", {"router": r, "expert": {"ff": F}, "shared": None})
    sure = B.route_margin(h, w["router"], w["correction"], r) > 1e-4
    gu = np.stack([np.concatenate([w["e%d.gate" % e].reshape(-1, 8, K), w["e%d.up" % e].reshape(-1, 8, K)], 1).reshape(2 * F, K)
                   for e in range(E)])
    down = np.stack([w["e%d.down" % e] for e in range(E)])
    hd = dev(h, torch.bfloat16)
    assert ops.moe_tcgen05_supported(hd, T * top, 2 * F, K)
    plan = ops.moe_route(hd, dev(w["router"]), None, R, top, ops.MOE_TCGEN05_TILE_ROWS, scores="softmax_all",
                         correction=dev(w["correction"]), groups=5, keep_groups=3, route_scale=2.0, identity=identity)
    a = ops.moe_gemm_tcgen05(ops.moe_gather_rows(hd, plan), dev(gu, torch.bfloat16), plan, gated_activation="silu")
    y = ops.moe_gemm_tcgen05(a, dev(down, torch.bfloat16), plan)
    got = ops.moe_combine(y, plan, None, torch.bfloat16, h=hd)
    ops.check_device_errors()
    close(got[torch.from_numpy(sure).to(DEV)], exact[sure], 2e-2)


def test_logits_times_a_number():
    from velox_b200.csrc import ops
    x = torch.randn(5, 333, device=DEV)
    assert torch.equal(ops.scale_rows(x, 0.3), x * 0.3)
