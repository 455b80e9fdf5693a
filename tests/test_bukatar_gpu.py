"""Bukatar on the GPU against the plain implementation (tests/plain_bukatar.py): each mechanism
alone, then whole models under every way of cutting a trace, then generation through the scheduler."""
import os

import numpy as np
import pytest

import plain_bukatar as pb
from bukatar_helpers import (SMALL, SPREAD, attention, config, latent, mamba1, plain_logits, random_config, sequences)
from helpers import (error_stats, make_model_folder, run_trace_inprocess, run_trace_program, tokens_needed,
                     trace_mixed, trace_portions, trace_tail_decode, trace_whole)
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
def test_sandwich_sum_and_stream_embedding():
    """x += norm(product) with the next sublayer's norm of the new row in the same pass, from whole and from
    split-K partial products; the token embedding onto the 32-bit stream."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(0)
    T, H, V = 11, 52, 30
    for dtype in _dtypes():
        table = _t(rng.standard_normal((V, H)), dtype)
        ids = torch.from_numpy(rng.integers(0, V, size=T).astype(np.int32)).cuda()
        x = ops.embed_position(ids, None, table, None)
        assert x.dtype == torch.float32 and np.array_equal(_np(x), _np(table)[ids.cpu().numpy()])
        w, w_next = _t(1 + 0.2 * rng.standard_normal(H), dtype), _t(1 + 0.2 * rng.standard_normal(H), dtype)
        for a in (_t(rng.standard_normal((T, H))), _t(rng.standard_normal((3, T, H)))):
            y = x.clone()
            h = ops.stream_norm_add(y, a, w, 1e-5, next_weight=w_next)
            prod = _np(a) if a.dim() == 2 else _np(a).sum(0)
            ref = _np(x) + pb.rms_norm(prod, _np(w), 1e-5)
            assert np.abs(_np(y) - ref).max() < 1e-5
            assert h.dtype == dtype
            assert np.abs(_np(h) - pb.rms_norm(ref, _np(w_next), 1e-5)).max() < (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("tokens,n_out,k", [(3, 200, 64), (70, 96, 328), (300, 520, 128), (4100, 512, 2112), (9, 50, 36)])
def test_relu_squared_in_the_products_epilogue(tokens, n_out, k):
    """max(z, 0)^2 as the epilogue of a product: both orientations of the tensor-core kernel, the kernel on pairs
    of SMs, and the plain kernel (rows of no 16-byte multiple, 32-bit)."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(tokens)
    for dtype in _dtypes():
        x, w = _t(rng.standard_normal((tokens, k)), dtype), _t(rng.standard_normal((n_out, k)) / np.sqrt(k), dtype)
        got = ops.linear(x, w, None, act="relu2")
        ref = pb.relu_squared(_np(x) @ _np(w).T)
        err = (np.abs(_np(got) - ref) / (1.0 + np.abs(ref))).max()
        assert got.dtype == dtype and err < (1e-5 if dtype == torch.float32 else 0.01)
    ops.take_device_errors()


@pytest.mark.parametrize("H,G,D,rot,base", [(4, 2, 16, 8, 10000.0), (3, 3, 24, 24, 100.0), (5, 1, 10, 0, 5.0),
                                            (2, 1, 64, 16, 250000.0)])
def test_pair_rotation_and_paged_store(H, G, D, rot, base):
    """q and k rotated pair by pair over their first `rot` entries, the bias added, the values stored as the
    keys before rotation, heads padded with zeros, from whole and partial products, a row of padding skipped."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(D)
    page, pages = 4, 16
    q_lens, pos0 = [5, 1, 7], [3, 130, 0]
    ctx, table = make_ctx(q_lens, pos0, [0, 1, 2], page_size=page, num_pages=64, shuffle=rng.permutation(64))
    T, head = sum(q_lens), ops.padded_head(D, D)
    inv = torch.from_numpy((base ** (-2.0 * np.arange(rot // 2) / max(rot, 1))).astype(np.float32)).cuda()
    pos = ctx.row_pos.cpu().numpy()
    for dtype in _dtypes():
        for splits in (1, 3):
            proj = _t(rng.standard_normal((splits, T, (H + G) * D)))
            bias = _t(rng.standard_normal((H + G) * D), dtype)
            ck = torch.full((64, G, page, head), float("nan"), dtype=dtype, device="cuda")
            cv = torch.full_like(ck, float("nan"))
            slots = ctx.groups[0].row_slot.clone()
            slots[2] = -1                                      # a row of padding: nothing stored
            q = ops.rope_pairs_store(proj if splits > 1 else proj[0], bias, ctx.row_pos, inv, rot, slots, ck, cv, H, G, D,
                                     D, head, H * D, H * D, dtype)
            full = _np(proj).sum(0) + _np(bias)
            want_q = pb.rotate_pairs(full[:, : H * D].reshape(T, H, D), pos, base, rot) if rot else full[:, : H * D].reshape(T, H, D)
            k_plain = full[:, H * D:].reshape(T, G, D)
            want_k = pb.rotate_pairs(k_plain, pos, base, rot) if rot else k_plain
            tol = 2e-5 if dtype == torch.float32 else 0.04
            got_q = _np(q).reshape(T, H, head)
            assert np.abs(got_q[:, :, :D] - want_q).max() < tol and not got_q[:, :, D:].any()
            for t in range(T):
                s = int(slots[t])
                if s < 0:
                    continue
                rk, rv = _np(ck[s // page, :, s % page]), _np(cv[s // page, :, s % page])
                assert np.abs(rk[:, :D] - want_k[t]).max() < tol and np.abs(rv[:, :D] - k_plain[t]).max() < tol
                assert not rk[:, D:].any() and not rv[:, D:].any()
            s = int(ctx.groups[0].row_slot[2])
            assert torch.isnan(ck[s // page, :, s % page]).all()
    ops.take_device_errors()


def _plain_attention(q, k, v, pos_q, scale, window, keep, sink):
    """q [n, H, D] at positions pos_q over keys k, v [L, G, D] at positions 0..L-1."""
    n, H, D = q.shape
    L, G = k.shape[0], k.shape[1]
    out = np.zeros((n, H, v.shape[2]))
    j = np.arange(L)[None, :]
    i = np.asarray(pos_q)[:, None]
    seen = j <= i
    if window > 0:
        seen &= (i - j < window) | (j < keep)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale
        out[:, h] = pb.softmax_weights(s, seen, extra_one=sink) @ v[:, h // (H // G)]
    return out


@pytest.mark.parametrize("window,keep,sink", [(0, 0, True), (13, 0, True), (13, 5, False), (32, 40, True), (7, 3, True),
                                              (1, 1, True)])
def test_window_with_kept_first_tokens_random(window, keep, sink):
    """The plain attention kernel with a window, kept first tokens and the denominator's extra one, on random
    inputs with shuffled pages: prompts' portions and single tokens, in both storage types."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(window * 100 + keep)
    H, G, D, page = 4, 2, 16, 8
    q_lens, pos0 = [9, 1, 30, 1], [50, 99, 0, 6]
    ctx, table = make_ctx(q_lens, pos0, [0, 1, 2, 3], page_size=page, num_pages=96, shuffle=rng.permutation(96))
    for dtype in _dtypes():
        ck = torch.full((96, G, page, D), float("nan"), dtype=dtype, device="cuda")
        cv = torch.full_like(ck, float("nan"))
        keys, vals = [], []
        for r, (n, p0) in enumerate(zip(q_lens, pos0)):
            k, v = _t(rng.standard_normal((p0 + n, G, D)), dtype), _t(rng.standard_normal((p0 + n, G, D)), dtype)
            keys.append(_np(k)); vals.append(_np(v))
            for p in range(p0 + n):
                ck[table[r, p // page], :, p % page] = k[p]
                cv[table[r, p // page], :, p % page] = v[p]
        q = _t(rng.standard_normal((sum(q_lens), H * D)), dtype)
        got = _np(ops.attention(q, ck, cv, ctx, ctx.groups[0], H, G, D, window, 0.4, keep_first=keep, sink_one=sink))
        at = 0
        for r, (n, p0) in enumerate(zip(q_lens, pos0)):
            want = _plain_attention(_np(q[at: at + n]).reshape(n, H, D), keys[r], vals[r], range(p0, p0 + n), 0.4, window,
                                    keep, sink)
            assert np.abs(got[at: at + n].reshape(n, H, D) - want).max() < (1e-5 if dtype == torch.float32 else 0.03)
            at += n
    ops.take_device_errors()


@pytest.mark.parametrize("decode", [False, True])
def test_window_edges_kept_tokens_and_the_extra_one(decode):
    """One key made to stand out (its score is far above the rest): the output is its value while the key is the
    window's last place or one of the kept first tokens, and not one place further; at page borders; for rows of
    a portion and for single tokens.  With no key that matters the extra one takes the weight: the output shrinks
    to nothing."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    H, G, D, page, window, keep = 2, 1, 16, 8, 24, 5
    L = 200                          # the query sits at position L - 1
    for target, seen in ((L - 1, True), (L - window, True), (L - window - 1, False), (keep - 1, True), (keep, False),
                         (0, True), (7, False), (8, False), (L - 17, True), (L - 16, True)):
        rng = np.random.default_rng(target)
        n = 1 if decode else 6
        ctx, table = make_ctx([n], [L - n], [0], page_size=page, num_pages=40, shuffle=rng.permutation(40))
        k = 0.05 * rng.standard_normal((L, G, D))
        v = rng.standard_normal((L, G, D))
        k[target, 0, 3] = 30.0
        q = np.zeros((n, H, D))
        q[:, :, 3] = 1.0
        ck = torch.zeros((40, G, page, D), device="cuda")
        cv = torch.zeros_like(ck)
        for p in range(L):
            ck[table[0, p // page], :, p % page] = _t(k[p])
            cv[table[0, p // page], :, p % page] = _t(v[p])
        got = _np(ops.attention(_t(q.reshape(n, -1)), ck, cv, ctx, ctx.groups[0], H, G, D, window, 1.0, keep_first=keep,
                                sink_one=True))[-1].reshape(H, D)
        if seen:
            assert np.abs(got - v[target, 0]).max() < 1e-3, target
        else:
            want = _plain_attention(q[-1:], k, v, [L - 1], 1.0, window, keep, True)[0]
            assert np.abs(got - want).max() < 1e-5 and np.abs(got - v[target, 0]).max() > 0.1, target
    # scores far below zero: the extra one holds all the weight
    ctx, table = make_ctx([1], [9], [0], page_size=page, num_pages=4)
    ck = torch.zeros((4, G, page, D), device="cuda")
    ck[..., 0] = -50.0
    cv = torch.ones_like(ck)
    q = torch.zeros((1, H * D), device="cuda")
    q[:, 0::D] = 1.0
    out = ops.attention(q, ck, cv, ctx, ctx.groups[0], H, G, D, window, 1.0, keep_first=keep, sink_one=True)
    assert float(out.abs().max()) < 1e-15
    ops.take_device_errors()


def _fill_pages(ck, cv, table, r, k, v, page):
    """Keys and values k, v [L, G, D] of request r into its pages."""
    L = k.shape[0]
    for b in range(-(-L // page)):
        n = min(page, L - b * page)
        ck[table[r, b], :, :n] = k[b * page: b * page + n].transpose(0, 1)
        cv[table[r, b], :, :n] = v[b * page: b * page + n].transpose(0, 1)


@pytest.mark.parametrize("D,H,G,page,window,keep,sink,prefill,cluster", [
    (64, 4, 2, 16, 150, 70, True, "auto", True), (64, 4, 2, 16, 150, 70, True, "mma", False),
    (128, 3, 1, 32, 40, 200, True, "auto", True), (64, 2, 2, 8, 300, 1, False, "auto", False),
    (32, 6, 3, 16, 33, 64, True, "auto", True), (128, 2, 1, 64, 1000, 129, True, "auto", False),
    (64, 20, 1, 16, 0, 0, True, "auto", True), (48, 2, 1, 16, 64, 65, False, "mma", True)])
def test_tensor_core_attention_with_kept_first_tokens_and_the_extra_one(D, H, G, page, window, keep, sink, prefill,
                                                                      cluster):
    """The tensor-core attention kernels (tcgen05 prefill for long portions of heads of 64 and 128, mma.sync
    prefill, split-key decode merged in a cluster or by the merge kernel) with a window, kept first tokens that
    span several tiles, and the denominator's extra one, on shuffled pages: long and short portions beside single
    tokens near and far from the start."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(D + window + keep)
    q_lens, pos0 = [200, 1, 70, 1, 1, 3], [300, 900, 0, 40, 2500, 127]
    pages = sum(-(-(n + p) // page) for n, p in zip(q_lens, pos0)) + 5
    ctx, table = make_ctx(q_lens, pos0, list(range(len(q_lens))), page_size=page, num_pages=pages,
                          shuffle=rng.permutation(pages))
    dtype = torch.bfloat16
    ck = torch.full((pages, G, page, D), float("nan"), dtype=dtype, device="cuda")
    cv = torch.full_like(ck, float("nan"))
    keys, vals = [], []
    for r, (n, p0) in enumerate(zip(q_lens, pos0)):
        k, v = _t(rng.standard_normal((p0 + n, G, D)), dtype), _t(rng.standard_normal((p0 + n, G, D)), dtype)
        keys.append(_np(k)); vals.append(_np(v))
        _fill_pages(ck, cv, table, r, k, v, page)
    ck, cv = torch.nan_to_num(ck, nan=0.0), torch.nan_to_num(cv, nan=0.0)      # rows past a request's length
    q = _t(rng.standard_normal((sum(q_lens), H * D)), dtype)
    scale = 2.0 * D ** -0.5
    old = ops.PREFILL_KERNEL, ops.CLUSTER_MERGE
    ops.PREFILL_KERNEL, ops.CLUSTER_MERGE = prefill, cluster
    try:
        launches = ops.COUNTER.launches
        got = _np(ops.attention(q, ck, cv, ctx, ctx.groups[0], H, G, D, window, scale, keep_first=keep, sink_one=sink))
        assert ops.COUNTER.launches - launches >= 2        # a prefill kernel and a decode kernel, not the plain one
    finally:
        ops.PREFILL_KERNEL, ops.CLUSTER_MERGE = old
    at = 0
    for r, (n, p0) in enumerate(zip(q_lens, pos0)):
        want = _plain_attention(_np(q[at: at + n]).reshape(n, H, D), keys[r], vals[r], range(p0, p0 + n), scale, window,
                                keep, sink)
        err = np.abs(got[at: at + n].reshape(n, H, D) - want).max()
        assert err < 0.03, (r, err)
        at += n
    ops.take_device_errors()


@pytest.mark.parametrize("n", [1, 6, 140])
@pytest.mark.parametrize("D,page,window,keep", [(64, 16, 150, 70), (128, 32, 260, 130), (64, 8, 64, 64)])
def test_tensor_core_window_edges_and_kept_tokens(n, D, page, window, keep):
    """One key made to stand out in bfloat16 on the tensor-core kernels: the last row's output is its value while
    the key is the window's last place or one of the kept first tokens, and not one place further; at tile and
    page borders; for a single token, a short portion and a portion of more than one tile of rows."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    H, G, L = 2, 1, 1000
    dtype = torch.bfloat16
    for target, seen in ((L - 1, True), (L - window, True), (L - window - 1, False), (keep - 1, True), (keep, False),
                         (0, True), (63, True), (64, keep > 64), (127, keep > 127), (128, keep > 128),
                         (L - window + 1, True), (L - window - page, False), (500, L - 500 <= window)):
        rng = np.random.default_rng(target)
        pages = -(-L // page) + 3
        ctx, table = make_ctx([n], [L - n], [0], page_size=page, num_pages=pages, shuffle=rng.permutation(pages))
        k = 0.05 * rng.standard_normal((L, G, D))
        v = rng.standard_normal((L, G, D))
        k[target, 0, 3] = 40.0
        q = np.zeros((n, H, D))
        q[:, :, 3] = 1.0
        ck = torch.zeros((pages, G, page, D), dtype=dtype, device="cuda")
        cv = torch.zeros_like(ck)
        _fill_pages(ck, cv, table, 0, _t(k, dtype), _t(v, dtype), page)
        got = _np(ops.attention(_t(q.reshape(n, -1), dtype), ck, cv, ctx, ctx.groups[0], H, G, D, window, 1.0,
                                keep_first=keep, sink_one=True))[-1].reshape(H, D)
        v_t = _np(_t(v[target, 0], dtype))
        if seen:
            assert np.abs(got - v_t).max() < 0.02, target
        else:
            want = _plain_attention(_np(_t(q[-1:], dtype)), _np(_t(k, dtype)), _np(_t(v, dtype)), [L - 1], 1.0, window,
                                    keep, True)[0]
            assert np.abs(got - want).max() < 0.02 and np.abs(got - v_t).max() > 0.1, target
    ops.take_device_errors()


@pytest.mark.parametrize("channels,N,taps", [(16, 8, 4), (40, 5, 2), (24, 12, 1), (50, 40, 5), (32, 64, 3), (8, 70, 4)])
def test_selective_scan_against_plain(channels, N, taps):
    """The convolution with kept inputs and the walk, against the plain recurrence: a whole sequence, portions
    down to one token (shorter than the convolution's reach), two requests side by side in used slots, and a call
    that may not write."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(channels + N)
    L = 37
    for dtype in _dtypes():
        conv_w, conv_b = _t(rng.standard_normal((channels, taps)) * 0.5, dtype), _t(rng.standard_normal(channels) * 0.1, dtype)
        a_log, skip = _t(rng.standard_normal((channels, N)) * 0.5, dtype), _t(1 + 0.1 * rng.standard_normal(channels), dtype)
        dt_bias = _t(rng.standard_normal(channels) * 0.5, dtype)
        data = []
        for r in range(2):
            xin, z = rng.standard_normal((L, channels)), rng.standard_normal((L, channels))
            dt_pre, bc = rng.standard_normal((L, channels)), rng.standard_normal((L, 2 * N))
            x = pb.silu(pb.causal_conv(xin, _np(conv_w), _np(conv_b)))
            dt = pb.softplus(dt_pre + _np(dt_bias))
            A = -np.exp(_np(a_log))
            S, y = np.zeros((channels, N)), np.zeros((L, channels))
            for t in range(L):
                S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * bc[t, None, :N]
                y[t] = S @ bc[t, N:] + _np(skip) * x[t]
            data.append((xin, z, dt_pre, bc, y * pb.silu(z), S))
        state = torch.full((3, channels, N), 7.0, device="cuda")
        kept = torch.full((3, max(taps - 1, 0), channels), 7.0, device="cuda")
        slots = [2, 0]
        for s in slots:
            state[s].zero_(); kept[s].zero_()
        got = [np.zeros((L, channels)), np.zeros((L, channels))]
        at = [0, 0]
        for sizes in ((1, 9), (2, 1), (5, 1), (1, 1), (20, 14), (8, 11)):
            q_lens = [min(n, L - a) for n, a in zip(sizes, at)]
            live = [r for r in range(2) if q_lens[r] > 0]
            ctx, _ = make_ctx([q_lens[r] for r in live], [at[r] for r in live], [slots[r] for r in live])
            rows = lambda i: np.concatenate([data[r][i][at[r]: at[r] + q_lens[r]] for r in live])  # noqa: E731
            proj = _t(np.concatenate([rows(0), rows(1)], axis=1))
            for write in (False, True):      # the first call must leave state and kept inputs as they were
                x32, xt = ops.conv_silu(proj, 0, channels, taps, conv_w, conv_b, kept, ctx, write=write)
                out = ops.selective_scan(x32, _t(rows(2)), _t(rows(3)), 0, N, proj[:, channels:], a_log, skip, dt_bias,
                                         state, ctx, write=write)
            assert xt.dtype == dtype and out.dtype == dtype
            o = _np(out)
            k = 0
            for r in live:
                got[r][at[r]: at[r] + q_lens[r]] = o[k: k + q_lens[r]]
                k += q_lens[r]
                at[r] += q_lens[r]
        tol = 2e-4 if dtype == torch.float32 else 0.05
        for r in range(2):
            scale = np.abs(data[r][4]).max()
            assert np.abs(got[r] - data[r][4]).max() < tol * scale
            assert np.abs(_np(state[slots[r]]) - data[r][5]).max() < 2e-4 * max(1.0, np.abs(data[r][5]).max())
        assert float(state[1].min()) == 7.0 and (taps == 1 or float(kept[1].min()) == 7.0)     # the unused slot
    ops.take_device_errors()


@pytest.mark.parametrize("E,top,T", [(12, 4, 50), (1, 1, 7), (7, 7, 33), (5, 2, 1), (70, 3, 300)])
def test_router_layout_and_grouped_products(E, top, T):
    """The router's choice and weights (ties go to the smaller index), the layout of the pairs in rows grouped
    by expert (every pair once, every expert's rows on tile borders), the grouped products against one product
    per pair, and the weighted sum with the shared expert's gated share."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(E * 10 + top)
    K, F = 24, 10
    logits = rng.standard_normal((T, E + 1)) * 2
    if E > 2:
        logits[0, :E] = 0.5            # all equal: the first `top` experts
        logits[T // 2, 1] = logits[T // 2, 2] = logits[T // 2].max() + 1
    chosen, weight, gate = ops.moe_route(_t(logits), E, top, gate_col=E)
    z = logits[:, :E] - logits[:, :E].max(-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    want = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    ch = chosen.cpu().numpy()
    exact = np.abs(np.take_along_axis(s, ch, -1) - np.take_along_axis(s, want, -1)).max(-1) == 0
    assert exact.all() and np.array_equal(ch[0], want[0]) and np.array_equal(ch[T // 2], want[T // 2])
    picked = np.take_along_axis(s, ch, -1)
    assert np.abs(_np(weight) - picked / (picked.sum(-1, keepdims=True) + 1e-20)).max() < 1e-6
    assert np.abs(_np(gate) - pb.sigmoid(logits[:, E])).max() < 1e-6
    tile = ops.grouped_tile_rows()
    row_src, tile_group, pos_of = (t.cpu().numpy() for t in ops.moe_align(chosen, E, tile))
    assert sorted(row_src[row_src >= 0]) == list(range(T * top)) and np.array_equal(row_src[pos_of], np.arange(T * top))
    for r in np.nonzero(row_src >= 0)[0]:
        assert tile_group[r // tile] == ch.reshape(-1)[row_src[r]]
    for dtype in _dtypes():
        x = _t(rng.standard_normal((T, K)), dtype)
        w_gu, w_down = _t(rng.standard_normal((E, 2 * F, K)) * 0.3, dtype), _t(rng.standard_normal((E, K, F)) * 0.3, dtype)
        rs, tg, po = ops.moe_align(chosen, E, tile)
        act = ops.linear_grouped(x, w_gu, rs, top, tg, rs.numel(), gated=True)
        y = ops.linear_grouped(act, w_down, None, 1, tg, rs.numel(), out_f32=True)
        shared = _t(rng.standard_normal((T, K)))
        out = _np(ops.moe_combine(y, po, weight, shared, gate))
        ref = np.zeros((T, K))
        for t in range(T):
            for k in range(top):
                e = ch[t, k]
                g = _np(w_gu[e])
                hidden = pb.silu(_np(x[t]) @ g[:F].T) * (_np(x[t]) @ g[F:].T)
                ref[t] += _np(weight)[t, k] * (hidden @ _np(w_down[e]).T)
        ref += _np(gate)[:, None] * _np(shared)
        assert np.abs(out - ref).max() < (1e-4 if dtype == torch.float32 else 0.05) * max(1.0, np.abs(ref).max())
    ops.take_device_errors()


@pytest.mark.parametrize("E,top,T,K,F", [(5, 2, 3, 24, 10), (4, 1, 1, 1100, 7), (3, 3, 20, 2088, 33), (7, 2, 30, 41, 19)])
def test_grouped_products_for_few_rows(E, top, T, K, F):
    """The experts' products by the kernel for a handful of rows: rows of whole 16-byte units and others, more
    inputs than wait in shared memory at a time, an odd count of columns, experts with more live rows than a
    pass takes and experts with none; against the plain products, and the layout picks it for such a step."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(E + K)
    logits = rng.standard_normal((T, E)) * 2
    if T > 8:
        logits[: T - 2, 0] = 40.0                              # one expert takes most tokens: several passes
        logits[:, E - 1] = -40.0                               # and one takes none
    chosen, weight, _ = ops.moe_route(_t(logits), E, top)
    ch = chosen.cpu().numpy()
    for dtype in _dtypes():
        lay = ops.moe_layout(chosen, E, dtype, K, F)
        assert lay.few and not lay.tc
        x = _t(rng.standard_normal((T, K)), dtype)
        w_gu = _t(rng.standard_normal((E, 2 * F, K)) * K ** -0.5, dtype)
        w_down = _t(rng.standard_normal((E, K, F)) * 0.3, dtype)
        act = ops.moe_experts_up(x, w_gu, lay, top)
        y = ops.moe_experts_down(act, w_down, lay)
        out = _np(ops.moe_combine(y, lay.pos_of, weight, None, None))
        rows = lay.pos_of.cpu().numpy().reshape(T, top)
        ref = np.zeros((T, K))
        tol = 1e-4 if dtype == torch.float32 else 0.03
        for t in range(T):
            for k in range(top):
                g = _np(w_gu[ch[t, k]])
                hidden = pb.silu(_np(x[t]) @ g[:F].T) * (_np(x[t]) @ g[F:].T)
                assert np.abs(_np(act[rows[t, k]]) - hidden).max() < tol * max(1.0, np.abs(hidden).max()), (t, k)
                ref[t] += _np(weight)[t, k] * (_np(act[rows[t, k]]) @ _np(w_down[ch[t, k]]).T)
        assert np.abs(out - ref).max() < (1e-4 if dtype == torch.float32 else 0.01) * max(1.0, np.abs(ref).max())
    ops.take_device_errors()


@pytest.mark.parametrize("E,top,T,K,F,force", [(6, 2, 40, 72, 40, True), (9, 3, 700, 136, 200, False),
                                               (3, 1, 260, 64, 24, False), (16, 2, 9, 320, 264, True)])
def test_grouped_products_on_the_tensor_cores(E, top, T, K, F, force):
    """The experts' products on the tcgen05 kernel over rows gathered into tiles of 128: experts without a pair
    (their tiles are skipped), experts with more than one tile, feature counts that are no multiple of a tile;
    chosen by the layout itself from a few hundred pairs on, forced below that."""
    torch = _torch()
    from llm_inference_lab_b200.kernels import ops
    rng = np.random.default_rng(E + T)
    logits = rng.standard_normal((T, E)) * 2
    logits[:, E // 2] = -50.0                                  # an expert nobody picks
    if E > 4:
        logits[: T // 2, 1] = 50.0                             # an expert half of the tokens pick
    chosen, weight, _ = ops.moe_route(_t(logits), E, top)
    ch = chosen.cpu().numpy()
    dtype = torch.bfloat16
    x = _t(rng.standard_normal((T, K)), dtype)
    w_gu, w_down = _t(rng.standard_normal((E, 2 * F, K)) * 0.2, dtype), _t(rng.standard_normal((E, K, F)) * 0.2, dtype)
    old = ops.GROUPED_KERNEL
    ops.GROUPED_KERNEL = "tc" if force else "auto"
    try:
        lay = ops.moe_layout(chosen, E, dtype, K, F)
        assert lay.tc and lay.tile == 128 and lay.rows % 128 == 0
        act = ops.moe_experts_up(x, w_gu, lay, top)
        y = ops.moe_experts_down(act, w_down, lay)
    finally:
        ops.GROUPED_KERNEL = old
    out = _np(ops.moe_combine(y, lay.pos_of, weight, None, None))
    act_np, rows = _np(act), lay.pos_of.cpu().numpy().reshape(T, top)
    ref = np.zeros((T, K))
    for t in range(T):
        for k in range(top):
            g = _np(w_gu[ch[t, k]])
            hidden = pb.silu(_np(x[t]) @ g[:F].T) * (_np(x[t]) @ g[F:].T)
            assert np.abs(act_np[rows[t, k]] - hidden).max() < 0.02 * max(1.0, np.abs(hidden).max()), (t, k)
            ref[t] += _np(weight)[t, k] * (_np(_t(hidden, dtype)) @ _np(w_down[ch[t, k]]).T)
    assert np.abs(out - ref).max() < 0.02 * max(1.0, np.abs(ref).max())
    ops.take_device_errors()


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
    all but one position in a hundred within BF16_MAX (a sublayer's output is divided by its root mean square,
    so where it is nearly zero its direction hangs on the last bits of bfloat16 products; a routed layer may
    also pick another expert where two scores are a rounding apart)."""
    worst, rms, where = error_stats(got, want)
    if dtype == "float32":
        assert worst < F32_MAX, (label, worst, where)
        return
    peak = max(float(np.abs(v).max()) for v in want.values())
    over = [key for key, row in got.items() if np.abs(row - want[key[0]][key[1]]).max() > BF16_MAX * peak]
    assert rms < BF16_RMS and len(over) <= max(1, len(got) // 100), (label, worst, rms, over[:5])


ONE_LAYER = {
    "mamba1": config([mamba1(48, 8, 4, 4)], vocab=53, width=32),
    "mamba1+ff": config([mamba1(40, 20, 2, 3, ff=40)], vocab=53, width=24),
    "attention": config([attention(4, 2, 16, 11, 2, 8)], vocab=53, width=32),
    "attention+moe": config([attention(3, 1, 24, 5, 0, 24, ff=(6, 2, 16, 12))], vocab=53, width=40),
    "latent": config([latent(2, 16, 8, 16, 24)], vocab=53, width=32),
    "latent+moe": config([latent(3, 8, 16, 24, 16, rot_dims=6, ff=(4, 3, 8, None))], vocab=53, width=48),
    "borrowed": config([latent(2, 16, 8, 8, 32, ff=24), latent(4, 8, 8, 16, 32, kv_from=0)], vocab=53, width=32),
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
    """Whole prompts; the tail decoded token by token, long enough for every window to pass over decoded tokens;
    portions of 2 to 11 tokens; up to four live requests with portions beside single tokens, in a pool so
    small that pages and state slots are used again."""
    cfg, opt = SMALL[name]
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
    """Portions of more than a hundred tokens beside single tokens, and a tail of 150 decoded tokens over which
    the window passes, with many experts."""
    cfg, opt = SMALL["D"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, opt["seed"], "bfloat16", std=0.08, scales=SPREAD)
    seqs = sequences(np.random.default_rng(9), cfg["vocab"], [400, 130, 260])
    want = plain_logits(folder, seqs)
    for label, steps in (("whole", trace_whole(seqs)), ("tail", trace_tail_decode(seqs, tail=150)),
                         ("mixed", trace_mixed(seqs, np.random.default_rng(2), max_live=3, max_portion=140))):
        eng = _engine(folder, "bfloat16", opt, steps)
        _check(run_trace_inprocess(eng, steps), want, "bfloat16", label)


@pytest.mark.parametrize("trial", range(int(os.environ.get("LAB_RANDOM_BUKATAR", "6"))))
def test_random_configurations_and_traces(tmp_path, trial):
    """Random configurations (layer orders, sizes that are no multiples of 8 or 16, windows of 1 to 500 keys, kept
    first tokens, 1 to 5 taps, 1 to 9 experts, borrowed latents, page sizes 4 to 64) under mixed batches with pages
    and slots used again, in 32-bit.  `LAB_RANDOM_BUKATAR=N` runs N."""
    rng = np.random.default_rng(2000 + trial)
    cfg, page = random_config(rng)
    seqs = sequences(rng, cfg["vocab"], [int(n) for n in rng.integers(1, 150, size=6)])
    steps = trace_mixed(seqs, np.random.default_rng(trial), max_live=4, max_portion=int(rng.choice([9, 40, 140])))
    folder = make_model_folder(str(tmp_path / "m"), cfg, trial, "float32", std=0.08, scales=SPREAD)
    want = plain_logits(folder, seqs)
    eng = _engine(folder, "float32", dict(page_size=page), steps)
    worst, rms, where = error_stats(run_trace_inprocess(eng, steps), want)
    assert worst < F32_MAX, (trial, cfg, worst, where)
    assert eng.cache.live_requests == 0


def test_cuts_agree_in_32_bit(tmp_path):
    """In 32-bit no sum's order depends on how a prompt was cut or on what else is in the batch."""
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
    """bin/trace_run on a Bukatar folder; and a step that fails leaves every part's state and the pages as they
    were."""
    from llm_inference_lab_b200.engine import Entry
    cfg, opt = SMALL["B"]
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
    assert len(eng.state_tensors) == 2      # the state-space mixer's state and its kept inputs
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
        tokens.append(int(np.argmax(pb.forward(cfg, w, tokens)[-1])))
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
    pcfg, w = pb.read_folder(folder)
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
        pcfg, w = pb.read_folder(folder)
        assert got == [_greedy(pcfg, w, p, s.max_new_tokens) for p, s in zip(prompts, sampling)]
    else:
        assert got == run(False)


def test_command_line_generates(tmp_path):
    import json
    import subprocess
    import sys
    cfg, opt = SMALL["C"]
    folder = make_model_folder(str(tmp_path / "m"), cfg, 19, "float32", std=0.08, scales=SPREAD)
    pcfg, w = pb.read_folder(folder)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-m", "llm_inference_lab_b200.cli", "--model-dir", folder, "--dtype", "f32",
                           "--prompt-ids", "3,14,15,9,2,6", "--max-new-tokens", "6", "--kv-tokens", "256"],
                          cwd=root, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["generated_ids"] == _greedy(pcfg, w, [3, 14, 15, 9, 2, 6], 6)
