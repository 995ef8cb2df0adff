"""CPU tests of the Degavik pieces that need no GPU: the NumPy restatement against independent formulations of the same
mechanisms (closed-form decayed sums, a matrix form of the delta rule, a masked batched attention, a direct convolution),
invariance of the restatement to how a sequence is cut, layers that share tensors, the synthetic-model writer, and the
host-only model detection of the C ABI."""
import json

import numpy as np

from ai00_server_b200 import capi, synth
from oracle import degavik_numpy as D

L = synth.degavik_layer


def model(layers, **kw):
    cfgb, st, w = synth.make_degavik(layers, **kw)
    return json.loads(cfgb), st, w


def test_writer_round_trips_and_skips_layers_without_tensors():
    cfg, st, w = model([L("retention"), L("channel_delta", mlp="moe"), L("channel_delta", mlp="moe", weights_of=1)], seed=2)
    back = D.read_safetensors(bytes(st))
    assert set(back) == set(w) and not any(k.startswith("l2.") for k in w)
    for k in w:
        assert np.array_equal(back[k], w[k]), k


def test_rotation_pairings_are_relative():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((2, 12)), rng.standard_normal((2, 12))
    for inter in (False, True):
        a = (D.rotate(q, 17, 8, 100.0, inter) * D.rotate(k, 11, 8, 100.0, inter)).sum()
        b = (D.rotate(q, 106, 8, 100.0, inter) * D.rotate(k, 100, 8, 100.0, inter)).sum()
        assert abs(a - b) < 1e-9
        assert np.array_equal(D.rotate(q, 5, 8, 100.0, inter)[:, 8:], q[:, 8:])          # entries past `dims` pass unchanged
    x = np.arange(8.0)[None]
    half = D.rotate(x, 1, 8, 1.0, False)          # base 1: every pair turns by 1 rad
    pair = D.rotate(x, 1, 8, 1.0, True)
    c, s = np.cos(1.0), np.sin(1.0)
    assert np.allclose(half[0, [0, 4]], [0 * c - 4 * s, 4 * c + 0 * s])
    assert np.allclose(pair[0, [0, 1]], [0 * c - 1 * s, 1 * c + 0 * s])


def test_retention_equals_the_closed_form_decayed_sum():
    cfg, st, w = model([L("retention", heads=3, dim=8, vdim=6, rot_dims=4, mlp=None)], width=24, seed=1)
    c, p = cfg["layers"][0]["mixer"], "l0.mix."
    rng = np.random.default_rng(3)
    hs = rng.standard_normal((9, 24))
    mem, got = {}, []
    for t, h in enumerate(hs):
        got.append(D.retention(w, p, c, 1e-5, h, mem, t))
    H, dk, dv = 3, 8, 6
    q = np.stack([D.rotate((w[p + "q"] @ h).reshape(H, dk), t, 4, c["rot"]["base"], False) for t, h in enumerate(hs)])
    k = np.stack([D.rotate((w[p + "k"] @ h).reshape(H, dk), t, 4, c["rot"]["base"], False) for t, h in enumerate(hs)]) / np.sqrt(dk)
    v = np.stack([(w[p + "v"] @ h).reshape(H, dv) for h in hs])
    for t in range(9):
        o = np.zeros((H, dv))
        for i in range(H):
            for s in range(t + 1):
                o[i] += c["decay"][i] ** (t - s) * (q[t, i] @ k[s, i]) * v[s, i]
        o = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-5)
        want = w[p + "o"] @ (o.reshape(-1) * D.silu(w[p + "g"] @ hs[t]))
        assert np.allclose(got[t], want, atol=1e-10)


def test_short_convolution_against_a_direct_sum():
    rng = np.random.default_rng(2)
    x, taps = rng.standard_normal((7, 5)), rng.standard_normal((5, 4))
    tail, got = np.zeros((3, 5)), []
    for row in x:
        y, tail = D.short_conv(taps, row, tail)
        got.append(y)
    pad = np.concatenate([np.zeros((3, 5)), x])
    want = np.stack([sum(taps[:, j] * pad[t + j] for j in range(4)) for t in range(7)])
    assert np.allclose(np.stack(got), D.silu(want))
    assert np.array_equal(tail, x[-3:])


def test_delta_rule_equals_its_matrix_form_and_shares_key_heads():
    cfg, st, w = model([L("channel_delta", heads=4, kv_heads=2, dim=6, vdim=5, conv=2, mlp=None)], width=20, seed=4)
    c, p = cfg["layers"][0]["mixer"], "l0.mix."
    rng = np.random.default_rng(5)
    hs = rng.standard_normal((6, 20))
    mem, got = {}, []
    for t, h in enumerate(hs):
        got.append(D.channel_delta(w, p, c, 1e-5, h, mem, t))
    H, G, dk, dv = 4, 2, 6, 5
    S = np.zeros((H, dk, dv))
    prev = {n: np.zeros(w[p + n].shape[0]) for n in "qkv"}
    for t, h in enumerate(hs):
        act = {}
        for n in "qkv":
            x = w[p + n] @ h
            act[n] = D.silu(w[p + n + ".conv"][:, 0] * prev[n] + w[p + n + ".conv"][:, 1] * x)
            prev[n] = x
        q, k, v = act["q"].reshape(G, dk), act["k"].reshape(G, dk), act["v"].reshape(H, dv)
        q = q / np.sqrt((q ** 2).sum(-1, keepdims=True) + 1e-6) / np.sqrt(dk)
        k = k / np.sqrt((k ** 2).sum(-1, keepdims=True) + 1e-6)
        beta = D.sigmoid(w[p + "b"] @ h)
        g = np.exp(-np.exp(w[p + "A_log"])[:, None] * D.softplus(w[p + "a2"] @ (w[p + "a1"] @ h) + w[p + "dt_bias"]).reshape(H, dk))
        o = np.zeros((H, dv))
        for i in range(H):
            kk = k[i // 2]
            S[i] = (np.eye(dk) - beta[i] * np.outer(kk, kk)) @ (np.diag(g[i]) @ S[i]) + beta[i] * np.outer(kk, v[i])
            o[i] = S[i].T @ q[i // 2]
        o = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-5) * w[p + "norm"]
        want = w[p + "o"] @ (o.reshape(-1) * D.sigmoid(w[p + "g2"] @ (w[p + "g1"] @ h)))
        assert np.allclose(got[t], want, atol=1e-10)
    assert np.all((g > 0) & (g < 1))


def test_attention_equals_a_masked_batched_form():
    cfg, st, w = model([L("attention", heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4, window=5, keep_first=2, softcap=3.0, mlp=None)],
                       width=24, seed=6)
    c, p = cfg["layers"][0]["mixer"], "l0.mix."
    rng = np.random.default_rng(7)
    n = 14
    hs = rng.standard_normal((n, 24))
    mem, got = {}, []
    for t, h in enumerate(hs):
        got.append(D.attention(w, p, c, 1e-5, h, mem, t))
    H, G, dk, dv = 4, 2, 8, 6
    nrm = lambda x, wt: x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * wt
    Q = np.stack([D.rotate(nrm((w[p + "q"] @ h).reshape(H, dk), w[p + "q.norm"]), t, 4, c["rot"]["base"], True) for t, h in enumerate(hs)])
    K = np.stack([D.rotate(nrm((w[p + "k"] @ h).reshape(G, dk), w[p + "k.norm"]), t, 4, c["rot"]["base"], True) for t, h in enumerate(hs)])
    V = np.stack([(w[p + "v"] @ h).reshape(G, dv) for h in hs])
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    mask = (j <= i) & ((i - j < 5) | (j < 2))
    assert mask[9].tolist() == [True, True, False, False, False, True, True, True, True, True, False, False, False, False]
    s = np.einsum("ihd,jhd->hij", Q, np.repeat(K, 2, 1)) * c["scale"] * w[p + "temp"][:, None, None]
    s = 3.0 * np.tanh(s / 3.0)
    s = np.where(mask[None], s, -np.inf)
    P = np.exp(s - s.max(-1, keepdims=True))
    P = P / P.sum(-1, keepdims=True)
    P = np.einsum("hg,gij->hij", w[p + "talk"], P)
    O = np.einsum("hij,jhd->ihd", P, np.repeat(V, 2, 1))
    for t in range(n):
        assert np.allclose(got[t], w[p + "o"] @ O[t].reshape(-1), atol=1e-10)


def test_router_takes_the_largest_logits_and_normalises_over_them():
    idx, wt = D.route(np.array([0.1, 2.0, -1.0, 2.0, 1.5]), 3)
    assert idx.tolist() == [1, 3, 4]
    e = np.exp(np.array([2.0, 2.0, 1.5]))
    assert np.allclose(wt, e / e.sum())
    idx, wt = D.route(np.array([-5.0, -7.0]), 1)
    assert idx.tolist() == [0] and wt.tolist() == [1.0]
    cfg, st, w = model([L("retention", mlp="moe", experts=5, top=2, shared_ff=8, ff=12)], width=16, seed=8)
    h = np.random.default_rng(1).standard_normal(16)
    w2 = dict(w)
    w2["l0.mlp.router.b"] = np.array([-30.0, 30.0, -30.0, 29.0, -30.0])       # the bias is part of the logits: it picks and it weighs
    z = w2["l0.mlp.router"] @ h + w2["l0.mlp.router.b"]
    a = np.exp(z[[1, 3]] - z[1])
    a = a / a.sum()
    want = a[0] * D.gated_unit(w, "l0.mlp.e1.", h) + a[1] * D.gated_unit(w, "l0.mlp.e3.", h) + D.gated_unit(w, "l0.mlp.shared.", h)
    assert np.allclose(D.feed_forward(w2, "l0.mlp.", cfg["layers"][0]["mlp"], h), want)


def test_shared_tensors_equal_copied_tensors_with_separate_memory():
    a = [L("channel_delta", mlp="moe"), L("attention", kv_heads=2, mlp="dense"), L("channel_delta", mlp="moe", weights_of=0),
         L("attention", kv_heads=2, mlp="dense", weights_of=1)]
    cfg, st, w = model(a, seed=10)
    b = json.loads(json.dumps(cfg))
    w2 = dict(w)
    for i, src in ((2, 0), (3, 1)):
        del b["layers"][i]["weights_of"]
        for k in list(w):
            if k.startswith("l%d." % src):
                w2["l%d." % i + k[len("l%d." % src):]] = w[k]
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg["vocab"], 15)]
    assert np.array_equal(D.run(cfg, w, toks), D.run(b, w2, toks))


def test_sequence_memory_makes_the_cut_irrelevant():
    cfg, st, w = model([L("retention"), L("channel_delta", conv=4), L("attention", window=4, keep_first=1, mlp="moe")], seed=9)
    toks = [int(t) for t in np.random.default_rng(4).integers(0, cfg["vocab"], 23)]
    whole = D.run(cfg, w, toks)
    mem, parts, at = D.new_memory(cfg), [], 0
    for c in (2, 1, 7, 13):
        parts.append(D.run(cfg, w, toks[at:at + c], mem=mem))
        at += c
    assert np.array_equal(np.concatenate(parts), whole)
    assert mem["pos"] == 23 and len(mem["layers"][2]["k"]) == 23


def test_model_detection_and_info_without_a_gpu():
    cfg, st, w = model([L("retention"), L("attention"), L("retention", weights_of=0)], width=48, vocab=80)
    info = capi.info_from_st(st)
    assert info["version"] == capi.ARCH_DEGAVIK
    assert (info["num_emb"], info["num_vocab"]) == (48, 80)
