"""Kupedra on the GPU against the plain implementation (tests/plain_kupedra.py): each mechanism
alone, then whole models under every way of cutting a trace, then generation through the scheduler."""
import copy
import os

import numpy as np
import pytest

import plain_kupedra as pk
from helpers import (error_stats, make_model_folder, run_trace_inprocess, run_trace_program, tokens_needed,
                     trace_mixed, trace_portions, trace_tail_decode, trace_whole)
from kupedra_helpers import SMALL, SPREAD, attention, config, moe, parallel, plain_logits, random_config, sequences
from ritizen_helpers import make_ctx

pytestmark = pytest.mark.gpu

F32_MAX = 2e-4      # largest error over the largest logit, 32-bit engine against the 64-bit plain model
BF16_MAX, BF16_RMS = 0.10, 0.04


def _torch():
    import torch
    return torch


def _t(a, dtype=None):
    torch = _torch()
    t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    return t if dtype is None else t.to(dtype)


def _np(t):
    return t.double().cpu().numpy()


def _dtypes():
    torch = _torch()
    return (torch.float32, torch.bfloat16)


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S,H,scalar", [(1, 40, True), (2, 52, True), (3, 64, False), (5, 30, True), (8, 16, False)])
def test_streams_read_write_and_norm(S, H, scalar):
    """The residual of several streams: copies of the embedding output, the read with its norm (weight one number
    or a vector; all rows or gathered ones; the plain sum), the write of all streams at once from the old ones,
    alone and with the next sublayer's read in its pass, from whole and from split-K partial products."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(S)
    T, eps = 9, 1e-5
    for dtype in _dtypes():
        tol = 1e-5 if dtype == torch.float32 else 3e-2
        x0 = _t(rng.standard_normal((T, H)))
        X = ops.hyper_expand(x0, S)
        assert X.shape == (T, S, H) and all(np.array_equal(_np(X[:, s]), _np(x0)) for s in range(S))
        X = _t(rng.standard_normal((T, S, H)))
        c_in, c_out, mix = _t(rng.random(S)), _t(rng.standard_normal(S)), _t(rng.standard_normal((S, S)))
        w = _t(1 + 0.2 * rng.standard_normal(() if scalar else (H,)), dtype).reshape(-1)
        wn = _np(w)[0] if scalar else _np(w)
        u = np.einsum("s,tsw->tw", _np(c_in), _np(X))
        assert np.abs(_np(ops.hyper_read_norm(X, c_in, w, eps)) - pk.unit_rms(u, eps) * wn).max() < tol
        rows = torch.tensor([T - 1, 0, 3], dtype=torch.int32, device="cuda")
        got = ops.hyper_read_norm(X, None, w, eps, rows=rows)
        assert np.abs(_np(got) - (pk.unit_rms(_np(X).sum(1), eps) * wn)[[T - 1, 0, 3]]).max() < tol
        for y in (_t(rng.standard_normal((T, H))), _t(rng.standard_normal((3, T, H)))):
            yn = _np(y) if y.dim() == 2 else _np(y).sum(0)
            ref = np.einsum("sr,tsw->trw", _np(mix), _np(X)) + _np(c_out)[None, :, None] * yn[:, None, :]
            A = X.clone()
            assert ops.hyper_write(A, y, mix, c_out) is None
            assert np.abs(_np(A) - ref).max() < 1e-5
            B = X.clone()
            h = ops.hyper_write(B, y, mix, c_out, c_in, w, eps)
            assert np.array_equal(_np(A), _np(B)) and h.dtype == dtype
            assert np.abs(_np(h) - pk.unit_rms(np.einsum("s,tsw->tw", _np(c_in), ref), eps) * wn).max() < tol
    ops.take_device_errors()


def test_normed_sum_scaled_embedding_and_scaled_logits():
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(1)
    T, H, V = 7, 44, 30
    for dtype in _dtypes():
        wa, wb = _t(1 + 0.3 * rng.standard_normal(H), dtype), _t(1 + 0.3 * rng.standard_normal(H), dtype)
        for a, b in ((_t(rng.standard_normal((T, H))), _t(rng.standard_normal((2, T, H)))),
                     (_t(rng.standard_normal((4, T, H))), None)):
            an = _np(a) if a.dim() == 2 else _np(a).sum(0)
            ref = 0.5 * pk.unit_rms(an, 1e-6) * _np(wa)
            if b is not None:
                ref = ref + 0.25 * pk.unit_rms(_np(b).sum(0), 1e-6) * _np(wb)
            got = ops.normed_sum(a, wa, 0.5, b, wb if b is not None else None, 0.25, 1e-6)
            assert got.dtype == torch.float32 and np.abs(_np(got) - ref).max() < 1e-5
        table = _t(rng.standard_normal((V, H)), dtype)
        ids = torch.from_numpy(rng.integers(0, V, size=T).astype(np.int32)).cuda()
        x = ops.embed_position(ids, None, table, None, scale=0.37)
        assert np.abs(_np(x) - 0.37 * _np(table)[ids.cpu().numpy()]).max() < 1e-6
    z = _t(rng.standard_normal((5, 33)))
    assert np.abs(_np(ops.scale_rows(z.clone(), 1.7)) - 1.7 * _np(z)).max() < 1e-6
    ops.take_device_errors()


@pytest.mark.parametrize("H,G,D,V,rot,norm,temp", [(4, 2, 16, 24, 8, "unit", True), (3, 3, 24, 8, 24, "weight", False),
                                                   (5, 1, 10, 10, 0, "weight", True), (2, 1, 64, 64, 32, "unit", False),
                                                   (1, 1, 160, 40, 6, None, True)])
def test_head_norms_temperatures_and_paged_store(H, G, D, V, rot, norm, temp):
    """q and k rotated pair by pair, normed per head (without a weight, or with one shared by the heads), q times a
    number per head and times the temperature that grows with the position; q rounded, k and v in their page slots
    with zeros beyond their sizes; from whole and from partial products."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(H * 100 + D)
    page, eps = 8, 1e-5
    q_lens, pos0 = [5, 1, 9], [0, 130, 61]
    ctx, table = make_ctx(q_lens, pos0, [0, 1, 2], page_size=page, num_pages=64, shuffle=rng.permutation(64))
    T = sum(q_lens)
    head = ops.padded_head(D, V)
    width = H * D + G * D + G * V
    base, factor, coef, every = 300.0, 1.7, 0.6, 4
    inv = (base ** (-2.0 * np.arange(rot // 2) / max(rot, 1)) / factor).astype(np.float32)
    pos = _np(ctx.row_pos).astype(np.int64)
    for dtype in _dtypes():
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        for proj in (_t(rng.standard_normal((T, width))), _t(rng.standard_normal((3, T, width)))):
            wq = _t(1 + 0.3 * rng.standard_normal(D), dtype) if norm == "weight" else None
            wk = _t(1 + 0.3 * rng.standard_normal(D), dtype) if norm == "weight" else None
            hs = _t(1 + 0.5 * rng.random(H)) if temp else None
            ck = torch.full((64, G, page, head), float("nan"), dtype=dtype, device="cuda")
            cv = torch.full((64, G, page, head), float("nan"), dtype=dtype, device="cuda")
            q = ops.head_prep_store(proj, None, ctx.row_pos, _t(inv), rot, ctx.groups[0].row_slot, ck, cv, H, G, D, V,
                                    head, H * D, H * D + G * D, dtype, norm_eps=eps if norm else 0.0, q_norm_w=wq,
                                    k_norm_w=wk, q_head_scale=hs, temp_coef=coef, temp_every=every)
            p = _np(proj) if proj.dim() == 2 else _np(proj).sum(0)
            qr = pk.rotate_pairs(p[:, : H * D].reshape(T, H, D), pos, base, rot, factor)
            kr = pk.rotate_pairs(p[:, H * D: H * D + G * D].reshape(T, G, D), pos, base, rot, factor)
            if norm:
                qr, kr = pk.unit_rms(qr, eps), pk.unit_rms(kr, eps)
            if norm == "weight":
                qr, kr = qr * _np(wq), kr * _np(wk)
            if temp:
                qr = qr * _np(hs)[None, :, None]
            qr = qr * (1.0 + coef * np.log(np.floor((pos + 1) / every) + 1.0))[:, None, None]
            got = _np(q).reshape(T, H, head)
            assert np.abs(got[:, :, :D] - qr).max() < tol * max(1.0, np.abs(qr).max()) and not got[:, :, D:].any()
            slots = _np(ctx.groups[0].row_slot).astype(np.int64)
            for t in range(T):
                kk, vv = _np(ck[slots[t] // page, :, slots[t] % page]), _np(cv[slots[t] // page, :, slots[t] % page])
                assert np.abs(kk[:, :D] - kr[t]).max() < tol * max(1.0, np.abs(kr).max()) and not kk[:, D:].any()
                assert np.abs(vv[:, :V] - p[t, H * D + G * D:].reshape(G, V)).max() < tol * 4 and not vv[:, V:].any()
            # rows that were given no slot stay untouched
            assert int(torch.isnan(ck.float()).sum()) == (64 * page - T) * G * head
    ops.take_device_errors()


def _reference_attention(q, k, v, scale, bias, sink):
    """q [n, H, D] at positions p0 .. p0 + n - 1 over keys k, v [L, G, D]: scaled scores plus bias[h, distance],
    causal, a sink per head in the denominator."""
    n, H, _ = q.shape
    L, G, _ = k.shape
    p0 = L - n
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        i, j = np.arange(p0, L)[:, None], np.arange(L)[None, :]
        if bias is not None:
            s = s + bias[h][np.minimum(np.maximum(i - j, 0), bias.shape[1] - 1)]
        w = pk.sink_softmax(s[None], (j <= i)[None], np.array([sink[h]]) if sink is not None else np.array([-np.inf]))[0]
        out[:, h] = w @ v[:, g]
    return out


def _fill_cache(rng, ctx, table, lens, G, D, page, dtype, pages=64):
    """Keys and values of whole sequences written through the block table; returns the caches and the arrays."""
    torch = _torch()
    ck = torch.zeros((pages, G, page, D), dtype=dtype, device="cuda")
    cv = torch.zeros((pages, G, page, D), dtype=dtype, device="cuda")
    ks, vs = [], []
    for r, L in enumerate(lens):
        k, v = _t(rng.standard_normal((L, G, D)), dtype), _t(rng.standard_normal((L, G, D)), dtype)
        for j in range(L):
            pg = int(table[r, j // page])
            ck[pg, :, j % page] = k[j]
            cv[pg, :, j % page] = v[j]
        ks.append(_np(k))
        vs.append(_np(v))
    return ck, cv, ks, vs


@pytest.mark.parametrize("D,H,G,page,L,sink", [(16, 4, 2, 4, 9, True), (48, 4, 2, 16, 40, True), (64, 4, 1, 8, 130, False),
                                               (24, 2, 2, 16, 1, True), (128, 2, 1, 32, 200, True)])
def test_attention_with_a_distance_table_and_learned_sinks(D, H, G, page, L, sink):
    """Every attention kernel (the plain one in both storage types; the tensor-core prefill and decode kernels, with
    the keys split inside a cluster and through the merge kernel) with a bias by distance whose table ends inside
    and beyond the sequences, and a learned number per head in the denominator; pages in shuffled order; a long
    portion, short portions and single tokens side by side."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(D + L)
    q_lens, pos0 = [70, 1, 5, 1], [60, 199, 0, 8]
    ctx, table = make_ctx(q_lens, pos0, [0, 1, 2, 3], page_size=page, num_pages=128, shuffle=rng.permutation(128),
                          dtype=torch.float32)
    lens = [p + n for p, n in zip(pos0, q_lens)]
    scale = 0.8 * D ** -0.5
    bias = _t(3.0 * rng.standard_normal((H, L)))
    sinks = _t(2.0 * rng.standard_normal(H)) if sink else None
    for dtype in _dtypes():
        ck, cv, ks, vs = _fill_cache(rng, ctx, table, lens, G, D, page, dtype, pages=128)
        q = _t(rng.standard_normal((sum(q_lens), H * D)), dtype)
        ref = np.concatenate([_reference_attention(_np(q)[s: s + n].reshape(n, H, D), ks[r], vs[r], scale, _np(bias),
                                                   _np(sinks) if sink else None)
                              for r, (s, n) in enumerate(zip(np.cumsum([0] + q_lens[:-1]), q_lens))]).reshape(-1, H * D)
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        variants = [dict()] if dtype == torch.float32 else [dict(plain=True), dict(cluster=True), dict(cluster=False)]
        for how in variants:
            old_plain, old_cluster = ops.force_plain(bool(how.get("plain"))), ops.CLUSTER_MERGE
            ops.CLUSTER_MERGE = bool(how.get("cluster", True))
            try:
                got = ops.attention(q, ck, cv, ctx, ctx.groups[0], H, G, D, 0, scale, sink=sinks, dist_bias=bias)
            finally:
                ops.force_plain(old_plain)
                ops.CLUSTER_MERGE = old_cluster
            assert np.abs(_np(got) - ref).max() < tol * max(1.0, np.abs(ref).max()), (dtype, how)
    ops.take_device_errors()


@pytest.mark.parametrize("decode", [False, True])
def test_a_key_that_stands_out_far_back_and_at_borders(decode):
    """One key is made to match the query; it is found hundreds of positions back, at page and tile borders, at
    position 0, and right before the query.  The distance table's rows sit where the design puts them: a table with
    one large row lifts exactly the keys of that row's distances; the sink takes the weight when it is large."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.parts.window_attention import distance_table
    rng = np.random.default_rng(5)
    D, H, G, page, L = 32, 2, 1, 16, 600
    n = 1 if decode else 40
    ctx, table = make_ctx([n], [L - n], [0], page_size=page, num_pages=64, dtype=torch.float32)
    for dtype in _dtypes():
        ck, cv, ks, vs = _fill_cache(rng, ctx, table, [L], G, D, page, dtype)
        for target in (0, 15, 16, 63, 64, 300, L - n - 1, L - 2):
            q = 0.05 * rng.standard_normal((n, H, D))
            q[-1] += 6.0 * ks[0][target, 0] / np.linalg.norm(ks[0][target, 0])
            got = ops.attention(_t(q.reshape(n, H * D), dtype), ck, cv, ctx, ctx.groups[0], H, G, D, 0, 1.0)
            got = _np(got).reshape(n, H, D)[-1]
            assert np.abs(got - vs[0][target, 0]).max() < 0.08 * np.abs(vs[0]).max(), (dtype, target)
        # a table of 12 rows that ends at distance 100: row 9 alone is large
        rows, far = 12, 100.0
        rel = np.zeros((rows, H))
        rel[9] = 40.0
        lifted = [d for d in range(L) if pk.distance_bucket(d, rows, far) == 9]
        assert lifted and lifted[0] > rows // 2 and lifted[-1] < far
        bias = distance_table(_t(rel), rows, far)
        q = 0.01 * rng.standard_normal((n, H * D))
        got = _np(ops.attention(_t(q, dtype), ck, cv, ctx, ctx.groups[0], H, G, D, 0, 1.0, dist_bias=bias))
        p = L - 1
        ref = np.mean([vs[0][p - d, 0] for d in lifted], axis=0)
        assert np.abs(got.reshape(n, H, D)[-1] - ref).max() < 0.08 * np.abs(vs[0]).max(), dtype
        # a sink far above every score takes all the weight: the output vanishes
        sinks = _t(np.full(H, 60.0))
        got = _np(ops.attention(_t(q, dtype), ck, cv, ctx, ctx.groups[0], H, G, D, 0, 1.0, sink=sinks))
        assert np.abs(got).max() < 1e-6
    ops.take_device_errors()


def test_distance_rows_follow_the_plain_rule():
    from llm_inference_lab_b200.parts.window_attention import distance_bucket
    for rows, far in ((16, 200.0), (7, 40.0), (1, 3.0), (2, 9.0), (12, 5000.0), (40, 21.0)):
        for n in range(0, 6000, 1 if rows < 10 else 7):
            assert distance_bucket(n, rows, far) == pk.distance_bucket(n, rows, far)
        assert distance_bucket(int(far) + 1, rows, far) == rows - 1


@pytest.mark.parametrize("tokens,n_out,k", [(3, 200, 64), (70, 96, 328), (300, 520, 128), (4100, 512, 264), (9, 50, 36)])
def test_capped_gate_in_the_products_epilogue(tokens, n_out, k):
    """g' = min(g, limit), u' = clamp(u, -limit, limit), g' * sigmoid(1.702 g') * (u' + 1) as the epilogue of the
    gated product: both orientations of the tensor-core kernel, the kernel on pairs of SMs, and the plain kernel."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(tokens)
    limit = 1.3
    for dtype in _dtypes():
        x, w = _t(rng.standard_normal((tokens, k)), dtype), _t(2.0 * rng.standard_normal((2 * n_out, k)) / np.sqrt(k), dtype)
        got = ops.linear_gated(x, w, limit=limit)
        g, u = _np(x) @ _np(w)[:n_out].T, _np(x) @ _np(w)[n_out:].T
        g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
        ref = g * pk.sigmoid(1.702 * g) * (u + 1.0)
        assert (np.abs(g) >= limit).any() and (np.abs(u) >= limit).any()      # the caps are met
        tol = 2e-5 if dtype == torch.float32 else 0.01
        assert got.dtype == dtype and (np.abs(_np(got) - ref) / (1.0 + np.abs(ref))).max() < tol
        plain = ops.linear_gated(x, w)                                         # limit 0 stays the SiLU gate
        g0, u0 = _np(x) @ _np(w)[:n_out].T, _np(x) @ _np(w)[n_out:].T
        ref0 = g0 * pk.sigmoid(g0) * u0
        assert (np.abs(_np(plain) - ref0) / (1.0 + np.abs(ref0))).max() < tol
    ops.take_device_errors()


@pytest.mark.parametrize("E,top,T,K,F,kernel", [(5, 2, 3, 24, 10, "auto"), (7, 7, 33, 40, 16, "auto"), (3, 1, 300, 72, 40, "auto"),
                                                (6, 2, 40, 72, 40, "tc"), (4, 2, 50, 41, 19, "tiles")])
def test_routed_experts_with_scores_as_they_are_and_capped_experts(E, top, T, K, F, kernel):
    """The router's weights without renormalisation, and the experts' capped form in all three grouped products."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(E * T)
    limit = 0.9
    for dtype in _dtypes():
        if kernel == "tc" and dtype == torch.float32:
            continue
        logits = _t(3.0 * rng.standard_normal((T, E + 1)))
        chosen, weight, gate = ops.moe_route(logits, E, top, gate_col=E, renorm=False)
        z = _np(logits)[:, :E]
        s = np.exp(z - z.max(-1, keepdims=True))
        s /= s.sum(-1, keepdims=True)
        ch = chosen.cpu().numpy()
        for t in range(T):
            order = sorted(range(E), key=lambda e: (-s[t, e], e))[:top]
            assert list(ch[t]) == order and np.abs(_np(weight)[t] - s[t, order]).max() < 1e-6
        assert np.abs(_np(gate) - pk.sigmoid(_np(logits)[:, E])).max() < 1e-6
        x = _t(rng.standard_normal((T, K)), dtype)
        w_gu = _t(2.0 * rng.standard_normal((E, 2 * F, K)) / np.sqrt(K), dtype)
        w_down = _t(rng.standard_normal((E, K, F)) / np.sqrt(F), dtype)
        old, ops.GROUPED_KERNEL = ops.GROUPED_KERNEL, kernel
        try:
            lay = ops.moe_layout(chosen, E, dtype, K, F)
            act = ops.moe_experts_up(x, w_gu, lay, top, limit=limit)
            y = ops.moe_experts_down(act, w_down, lay)
        finally:
            ops.GROUPED_KERNEL = old
        out = _np(ops.moe_combine(y, lay.pos_of, weight, None, None))
        ref = np.zeros((T, K))
        for t in range(T):
            for k in range(top):
                m = _np(w_gu[ch[t, k]])
                g, u = np.minimum(_np(x[t]) @ m[:F].T, limit), np.clip(_np(x[t]) @ m[F:].T, -limit, limit)
                hidden = g * pk.sigmoid(1.702 * g) * (u + 1.0)
                ref[t] += _np(weight)[t, k] * (_np(_t(hidden, dtype)) @ _np(w_down[ch[t, k]]).T)
        assert np.abs(out - ref).max() < (1e-4 if dtype == torch.float32 else 0.03) * max(1.0, np.abs(ref).max())
    ops.take_device_errors()


def _memory_mixer(spec_params, weights, dtype):
    torch = _torch()
    from llm_inference_lab_b200.parts.matrix_memory import MatrixMemory
    from llm_inference_lab_b200.parts.spec import PartSpec
    spec = PartSpec("matrix_memory", spec_params, prefix="m.")
    w = {k: _t(v, dtype) for k, v in weights.items()}
    return MatrixMemory(spec, w, dtype, torch.device("cuda:0")), spec


@pytest.mark.parametrize("H,D,V,cap", [(3, 16, 8, 9.0), (1, 32, 40, 15.0), (2, 24, 20, 3.0), (4, 64, 64, 12.0), (2, 6, 130, 5.0)])
def test_matrix_memory_against_plain(H, D, V, cap):
    """The matrix memory mixer against the plain recurrence: a prompt in one step, in portions down to one token,
    two requests side by side in used slots, a call that may not write; gates that open and close."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.parts.base import CacheView
    from llm_inference_lab_b200.parts.spec import FixedState
    rng = np.random.default_rng(H * D + V)
    width, eps, T = 40, 1e-5, 37
    names = {"q": (H * D, width), "k": (H * D, width), "v": (H * V, width), "g": (H * V, width), "o": (width, H * V),
             "i": (H, width), "f": (H, width)}
    wn = {"m." + n: rng.standard_normal(s) / np.sqrt(s[1]) for n, s in names.items()}
    wn["m.i"] *= 4.0
    wn["m.f"] *= 4.0
    wn["m.norm"] = 1 + 0.2 * rng.standard_normal(H * V)
    wn["m.i.b"], wn["m.f.b"] = 2.0 * rng.standard_normal(H), 3.0 + 2.0 * rng.standard_normal(H)
    params = {"hidden": width, "heads": H, "dim": D, "vdim": V, "gate_cap": cap, "eps": eps}
    for dtype in _dtypes():
        mixer, _ = _memory_mixer(params, wn, dtype)
        wr = {k: _np(_t(v, dtype)) for k, v in wn.items()}        # the weights as the engine stores them
        h = [_t(rng.standard_normal((n, width)), dtype) for n in (T, 11)]
        ref = [pk.matrix_memory(_np(x), wr, "m.", {"heads": H, "dim": D, "vdim": V, "gate_cap": cap}, eps) for x in h]
        tol = (3e-5 if dtype == torch.float32 else 4e-2) * max(1.0, max(np.abs(r).max() for r in ref))

        def views():
            need = type(mixer).cache_need(mixer.spec)
            parts = [CacheView(need=n, state=torch.full((4,) + tuple(n.shape), 7.0, device="cuda")) for n in need.parts]
            return CacheView(need=need, parts=parts)

        def zero(cache, slot):
            for part in cache.parts:
                part.state[slot] = 0

        # both requests whole, side by side, in slots 2 and 0
        cache = views()
        zero(cache, 2), zero(cache, 0)
        ctx, _ = make_ctx([T, 11], [0, 0], [2, 0], dtype=dtype)
        got = _np(mixer.forward(torch.cat(h), ctx, cache))
        if got.ndim == 3:
            got = got.sum(0)
        assert np.abs(got[:T] - ref[0]).max() < tol and np.abs(got[T:] - ref[1]).max() < tol
        assert float(cache.parts[0].state[1].min()) == 7.0        # other slots untouched
        # the first request in portions, the second decoded token by token beside it
        cache = views()
        zero(cache, 1), zero(cache, 3)
        at, at2, outs, outs2 = 0, 0, [], []
        for n in (1, 2, 7, 1, 16, 3, 5, 2):
            take2 = 1 if at2 < 11 else 0
            ctx, _ = make_ctx([n] + [1] * take2, [at] + [at2] * take2, [1] + [3] * take2, dtype=dtype)
            rows = [h[0][at: at + n]] + ([h[1][at2: at2 + 1]] if take2 else [])
            got = _np(mixer.forward(torch.cat(rows), ctx, cache))
            got = got.sum(0) if got.ndim == 3 else got
            outs.append(got[:n])
            if take2:
                outs2.append(got[n:])
            at, at2 = at + n, at2 + take2
        assert at == T and np.abs(np.concatenate(outs) - ref[0]).max() < tol
        assert np.abs(np.concatenate(outs2) - ref[1][:at2]).max() < tol
        # a call that may not write leaves the state as it was
        before = [p.state.clone() for p in cache.parts]
        ctx, _ = make_ctx([3], [at2], [3], dtype=dtype)
        mixer.forward(h[1][at2: at2 + 3], ctx, CacheView(need=cache.need, parts=cache.parts, write=False))
        assert all(bool((a == p.state).all()) for a, p in zip(before, cache.parts))
    ops.take_device_errors()


def test_memory_survives_gates_at_their_caps():
    """Input gates at +cap and forget gates that close: the running maximum keeps every exponential finite, and a
    long sequence of wide-open input gates does not overflow."""
    torch = _torch()
    rng = np.random.default_rng(3)
    H, D, V, width, cap, eps, T = 2, 8, 8, 16, 30.0, 1e-6, 300
    wn = {"m." + n: rng.standard_normal(s) / 4.0 for n, s in
          {"q": (H * D, width), "k": (H * D, width), "v": (H * V, width), "g": (H * V, width), "o": (width, H * V),
           "i": (H, width), "f": (H, width)}.items()}
    wn["m.norm"] = np.ones(H * V)
    wn["m.i.b"], wn["m.f.b"] = np.array([200.0, -200.0]), np.array([-200.0, 200.0])
    params = {"hidden": width, "heads": H, "dim": D, "vdim": V, "gate_cap": cap, "eps": eps}
    from llm_inference_lab_b200.parts.base import CacheView
    mixer, _ = _memory_mixer(params, wn, torch.float32)
    need = type(mixer).cache_need(mixer.spec)
    cache = CacheView(need=need, parts=[CacheView(need=n, state=torch.zeros((1,) + tuple(n.shape), device="cuda"))
                                        for n in need.parts])
    h = rng.standard_normal((T, width))
    ctx, _ = make_ctx([T], [0], [0], page_size=16, dtype=torch.float32)
    got = _np(mixer.forward(_t(h), ctx, cache))
    got = got.sum(0) if got.ndim == 3 else got
    ref = pk.matrix_memory(h, wn, "m.", {"heads": H, "dim": D, "vdim": V, "gate_cap": cap}, eps)
    assert np.isfinite(got).all() and np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())


# ---------------------------------------------------------------------------------------------
# whole models under every cut
# ---------------------------------------------------------------------------------------------
def _engine(folder, dtype, opt, steps, **kw):
    from llm_inference_lab_b200.engine import Engine
    page = opt["page_size"]
    unit = max(64, page)
    pool = tokens_needed(steps, unit)
    return Engine(folder, dtype, max_tokens=pool, page_size=page, max_requests=4, max_batch_tokens=max(pool, 64),
                  max_seq_len=pool, **kw)


def _check(got, want, dtype, label):
    """32-bit: every position within F32_MAX.  bfloat16: the rms error over all positions within BF16_RMS and
    all but one position in a hundred within BF16_MAX (a mixer's output is divided by its root mean square, so
    where it is nearly zero its direction hangs on the last bits of bfloat16 products; a routed layer may also
    pick another expert where two scores are a rounding apart)."""
    worst, rms, where = error_stats(got, want)
    if dtype == "float32":
        assert worst < F32_MAX, (label, worst, where)
        return
    peak = max(float(np.abs(v).max()) for v in want.values())
    over = [key for key, row in got.items() if np.abs(row - want[key[0]][key[1]]).max() > BF16_MAX * peak]
    assert rms < BF16_RMS and len(over) <= max(1, len(got) // 100), (label, worst, rms, over[:5])


ONE_LAYER = {
    "attention": config([attention(4, 2, 16, 24, 8, base=100.0, factor=3.0, scale=0.3)], vocab=53, width=32, streams=2),
    "attention+moe": config([attention(3, 1, 24, 8, 24, scale=0.25, ff=moe(6, 2, 16, 1.1, (12, 0.7)))], vocab=53, width=40,
                            streams=3, logit_scale=2.5),
    "parallel": config([parallel((4, 2, 16, 8, 0.3, (0.5, 5), 8, 20), (2, 16, 24, 8.0))], vocab=53, width=32, streams=2,
                       embed_scale=0.4),
    "parallel+moe": config([parallel((2, 2, 24, 24, 0.25, None, 5, 9), (3, 8, 8, 20.0), ff=moe(4, 3, 8, 2.0))], vocab=53,
                           width=48, streams=0),
    "looped": config([parallel((1, 1, 8, 16, 0.4, (0.3, 2), 4, 6), (1, 24, 8, 6.0), ff=moe(2, 1, 8, 1.0, (8, 1.0)))],
                     vocab=53, width=24, streams=4, loop=(0, 1, 3)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_one_layer_models(tmp_path, name, dtype):
    rng = np.random.default_rng(3)
    cfg = ONE_LAYER[name]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 21, dtype, std=0.08, scales=SPREAD)
    seqs = sequences(rng, cfg["vocab"], [45, 1, 30])
    want = plain_logits(folder, seqs)
    for label, steps in (("whole", trace_whole(seqs)), ("tail", trace_tail_decode(seqs, tail=25)),
                         ("portions", trace_portions(seqs))):
        eng = _engine(folder, dtype, dict(page_size=8), steps)
        _check(run_trace_inprocess(eng, steps), want, dtype, (name, label))
        assert eng.cache.live_requests == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SMALL))
def test_models_under_every_cut(tmp_path, name, dtype):
    """Whole prompts; the tail decoded token by token, past the distance table's last row and several steps of
    the temperature; portions of 2 to 11 tokens; up to four live requests with portions beside single tokens,
    in a pool so small that pages and state slots are used again."""
    cfg, opt = SMALL[name]
    if name == "C" and dtype == "bfloat16":
        # C runs its side-by-side layer three times over with one head of few entries on each side, and picks one
        # expert of two.  Each run divides both sides' results by their root mean squares, which at single
        # positions are nearly zero: measured against the 32-bit engine on the same weights, the median
        # error doubles with every run and single positions jump to a third of the logits' size, and a score that
        # bfloat16 rounds to the other expert changes every later position through the memory.  In bfloat16 the
        # layer therefore runs once and the routers take all their experts; the loop and the choice are held
        # against the plain model in 32-bit.
        cfg = copy.deepcopy(cfg)
        del cfg["loop"]
        for layer in cfg["layers"]:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    rng = np.random.default_rng(opt["seed"])
    folder = make_model_folder(str(tmp_path / "m"), cfg, opt["seed"], dtype, std=0.08, scales=SPREAD)
    seqs = sequences(rng, cfg["vocab"], [150, 3, 61, 90, 1, 77, 40])
    want = plain_logits(folder, seqs)
    traces = {"whole": trace_whole(seqs), "tail": trace_tail_decode(seqs, tail=70), "portions": trace_portions(seqs),
              "mixed": trace_mixed(seqs, np.random.default_rng(1), max_live=4)}
    for label, steps in traces.items():
        eng = _engine(folder, dtype, opt, steps)
        got = run_trace_inprocess(eng, steps)
        assert len(got) == sum(len(v) for v in seqs.values())
        _check(got, want, dtype, (name, label))
        assert eng.cache.live_requests == 0 and all(f == eng.num_pages for f in eng.free_pages())


def test_long_portions_and_long_decoding(tmp_path):
    """Portions of more than a hundred tokens beside single tokens, and a tail of 150 decoded tokens, at heads of
    64 entries with many experts."""
    cfg, opt = SMALL["D"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, opt["seed"], "bfloat16", std=0.08, scales=SPREAD)
    seqs = sequences(np.random.default_rng(9), cfg["vocab"], [400, 130, 260])
    want = plain_logits(folder, seqs)
    for label, steps in (("whole", trace_whole(seqs)), ("tail", trace_tail_decode(seqs, tail=150)),
                         ("mixed", trace_mixed(seqs, np.random.default_rng(2), max_live=3, max_portion=140))):
        eng = _engine(folder, "bfloat16", opt, steps)
        _check(run_trace_inprocess(eng, steps), want, "bfloat16", label)


@pytest.mark.parametrize("trial", range(int(os.environ.get("LAB_RANDOM_KUPEDRA", "6"))))
def test_random_configurations_and_traces(tmp_path, trial):
    """Random configurations (layer orders, sizes that are no multiples of 8 or 16, zero to five streams, loops,
    distance tables of 1 to 40 rows, 1 to 9 experts, page sizes 4 to 64) under mixed batches with pages and slots
    used again, in 32-bit.  `LAB_RANDOM_KUPEDRA=N` runs N."""
    rng = np.random.default_rng(3000 + trial)
    cfg, page = random_config(rng)
    seqs = sequences(rng, cfg["vocab"], [int(n) for n in rng.integers(1, 150, size=6)])
    steps = trace_mixed(seqs, np.random.default_rng(trial), max_live=4, max_portion=int(rng.choice([9, 40, 140])))
    folder = make_model_folder(str(tmp_path / "m"), cfg, trial, "float32", std=0.08, scales=SPREAD)
    want = plain_logits(folder, seqs)
    eng = _engine(folder, "float32", dict(page_size=page), steps)
    got = run_trace_inprocess(eng, steps)
    worst, rms, where = error_stats(got, want)
    # A head of the memory whose S^T q nearly cancels is then divided by its root mean square: at such a position
    # 32-bit arithmetic alone is off by more (one was met at a cancellation of 1,000 where the median is 4.5: a
    # plain NumPy evaluation in 32-bit was 8e-5 off in that head's output there, the engine 2e-5).  So single
    # positions (two, or one in a hundred) may pass the bound, within ten times of it.
    peak = max(float(np.abs(v).max()) for v in want.values())
    over = [key for key, row in got.items() if np.abs(row - want[key[0]][key[1]]).max() > F32_MAX * peak]
    assert worst < 10 * F32_MAX and len(over) <= max(2, len(got) // 100), (trial, cfg, worst, where, over[:5])
    assert eng.cache.live_requests == 0


def test_cuts_agree_in_32_bit(tmp_path):
    """In 32-bit the logits of a position do not depend on how a prompt was cut or on what else is in the batch,
    beyond the rounding of sums taken in another order (the experts' products of few and of many pairs)."""
    cfg, opt = SMALL["A"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 5, "float32", std=0.08, scales=SPREAD)
    seqs = sequences(np.random.default_rng(2), cfg["vocab"], [70, 33, 9])
    results = []
    for steps in (trace_whole(seqs), trace_portions(seqs), trace_mixed(seqs, np.random.default_rng(3), max_live=3)):
        results.append(run_trace_inprocess(_engine(folder, "float32", opt, steps), steps))
    for other in results[1:]:
        for key, row in results[0].items():
            assert np.abs(row - other[key]).max() <= 1e-5, key


def test_trace_program_and_a_failed_step(tmp_path):
    """bin/trace_run on a Kupedra folder; and a step that fails leaves every part's state and the pages as they
    were."""
    from llm_inference_lab_b200.engine import Entry
    cfg, opt = SMALL["A"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 8, "float32", std=0.08, scales=SPREAD)
    seqs = sequences(np.random.default_rng(4), cfg["vocab"], [50, 20, 35, 8, 41])
    want = plain_logits(folder, seqs)
    steps = trace_mixed(seqs, np.random.default_rng(6), max_live=4)
    out = str(tmp_path / "out")
    os.makedirs(out)
    got = run_trace_program(folder, "float32", steps, out, tokens_needed(steps, 64))
    _check(got, want, "float32", "program")
    ids = seqs["s0"]
    eng = _engine(folder, "float32", opt, trace_whole(seqs))
    # layers 0 and 1 run twice, layer 2 once; the two parallel layers keep a memory and its running maximum per run
    assert len(eng.views) == 5 and len(eng.state_tensors) == 6
    eng.step([Entry(0, ids[:20], [])])
    states = [t.clone() for t in eng.state_tensors]
    free = eng.free_pages()
    head = eng.model.head
    try:
        old = head.forward
        head.forward = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("injected"))   # fails after the layers ran
        with pytest.raises(RuntimeError):
            eng.step([Entry(0, ids[20:30], [9])])
    finally:
        head.forward = old
    assert all(bool((a == b).all()) for a, b in zip(states, eng.state_tensors)) and eng.free_pages() == free
    logits = eng.step([Entry(0, ids[20:], [len(ids) - 21])]).cpu().numpy()
    assert np.abs(logits[0] - want["s0"][-1]).max() < F32_MAX * max(1.0, np.abs(want["s0"]).max())


# ---------------------------------------------------------------------------------------------
# generation through the scheduler
# ---------------------------------------------------------------------------------------------
def _greedy(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(pk.forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_scheduler(tmp_path, name):
    """More requests than state slots, prompts cut under a small token budget: greedy tokens in 32-bit equal
    the plain model's."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.sampling import SamplingConfig
    cfg, opt = SMALL[name]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 17, "float32", std=0.08, scales=SPREAD)
    pcfg, w = pk.read_folder(folder)
    rng = np.random.default_rng(7)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], size=n)] for n in (5, 40, 1, 23, 12, 31)]
    llm = LLM(folder, "float32", page_size=opt["page_size"], kv_tokens=512, max_requests=3, max_batch_tokens=24,
              max_seq_len=128, device="cuda:0")
    results = llm.generate(prompts, SamplingConfig(max_new_tokens=12, ignore_eos=True))
    ops.take_device_errors()
    for prompt, res in zip(prompts, results):
        assert res.finish_reason == "length"
        assert res.tokens == _greedy(pcfg, w, prompt, 12)
    assert llm.engine.cache.live_requests == 0


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16")])
def test_decode_steps_from_cuda_graphs(tmp_path, name, dtype):
    """Decode steps replayed from CUDA graphs although the model keeps fixed-size state: batches padded with
    requests of length zero, a batch that shrinks as requests finish.  32-bit: the plain model's tokens;
    bfloat16: the tokens of the same engine stepping eagerly."""
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.kernels import ops
    from llm_inference_lab_b200.sampling import SamplingConfig
    cfg, opt = SMALL[name]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 23, dtype, std=0.08, scales=SPREAD)
    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], size=n)] for n in (7, 30, 2, 19, 11)]
    sampling = [SamplingConfig(max_new_tokens=n, ignore_eos=True) for n in (20, 5, 14, 9, 17)]

    def run(graph):
        llm = LLM(folder, dtype, page_size=opt["page_size"], kv_tokens=1024, max_requests=8, max_batch_tokens=64,
                  max_seq_len=128, device="cuda:0", cuda_graph=graph)
        assert llm.cuda_graph == graph
        out = [r.tokens for r in llm.generate(prompts, sampling)]
        ops.take_device_errors()
        assert llm.engine.cache.live_requests == 0
        if graph:
            assert llm.graphs.replays >= 10 and llm.graphs.captures >= 3
        return out

    got = run(True)
    if dtype == "float32":
        pcfg, w = pk.read_folder(folder)
        assert got == [_greedy(pcfg, w, p, s.max_new_tokens) for p, s in zip(prompts, sampling)]
    else:
        assert got == run(False)


def test_command_line_generates(tmp_path):
    import json
    import subprocess
    import sys
    cfg, opt = SMALL["C"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 19, "float32", std=0.08, scales=SPREAD)
    pcfg, w = pk.read_folder(folder)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-m", "llm_inference_lab_b200.cli", "--model-dir", folder, "--dtype", "f32",
                           "--prompt-ids", "3,14,15,9,2,6", "--max-new-tokens", "6", "--kv-tokens", "256"],
                          cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["generated_ids"] == _greedy(pcfg, w, [3, 14, 15, 9, 2, 6], 6)
