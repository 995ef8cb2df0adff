"""CPU tests of the Kemirax pieces that need no GPU: the NumPy restatement against independent formulations of the same
mechanisms (a batched causal attention over materialised keys / values, a closed-form decayed sum), invariance of the
restatement to how a sequence is cut, the synthetic-model writer, and the host-only model detection of the C ABI."""
import json

import numpy as np
import pytest

from ai00_server_b200 import capi, synth
from oracle import kemirax_numpy as K

LA = synth.kemirax_layer
YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}


def model(layers, **kw):
    cfgb, st, w = synth.make_kemirax(layers, **kw)
    return json.loads(cfgb), st, w, cfgb


def test_writer_round_trips_through_the_reader():
    cfg, st, w, _ = model([LA("latent_attention"), LA("gla")], seed=2)
    back = K.read_safetensors(bytes(st))
    assert set(back) == set(w)
    for k in w:
        assert np.array_equal(back[k], w[k]), k
        assert np.array_equal(K.bf16_round(back[k].astype(np.float32)), back[k].astype(np.float32)), k


def test_rotation_is_orthogonal_up_to_its_magnitude_and_relative():
    rot = {"base": 100.0, "dims": 8, "scaling": YARN}
    f, mag = K.rotary_tables(rot)
    assert mag == pytest.approx(0.1 * np.log(4.0) + 1.0)
    assert (np.diff(f) < 0).all()
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal(10), rng.standard_normal(10)      # two trailing entries pass unchanged
    ra, rb = K.rotate(a, 7, rot), K.rotate(b, 3, rot)
    assert np.allclose(ra[8:], a[8:]) and np.linalg.norm(ra[:8]) == pytest.approx(mag * np.linalg.norm(a[:8]))
    ra2, rb2 = K.rotate(a, 107, rot), K.rotate(b, 103, rot)
    assert np.dot(ra[:8], rb[:8]) == pytest.approx(np.dot(ra2[:8], rb2[:8]))     # depends on the distance only
    plain = {"base": 100.0, "dims": 8}
    assert K.rotary_tables(plain)[1] == 1.0 and np.allclose(K.rotate(a, 0, plain), a)


def test_latent_attention_equals_batched_causal_attention():
    cfg, st, w, _ = model([LA("latent_attention", mlp=False, scaling=YARN)], seed=5)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    rng = np.random.default_rng(1)
    n, W = 9, cfg["width"]
    hs = rng.standard_normal((n, W))
    cache, tok = [], []
    for t in range(n):
        tok.append(K.latent_attention_token(w, "l0.mix.", m, eps, hs[t], t, cache))
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    kv = hs @ w["l0.mix.dkv"].T
    c = K.rms_unit(kv[:, :rk], eps) * w["l0.mix.dkv.norm"]
    kr = np.stack([K.rotate(kv[t, rk:], t, m["rot"]) for t in range(n)])
    q = (K.rms_unit(hs @ w["l0.mix.dq"].T, eps) * w["l0.mix.dq.norm"]) @ w["l0.mix.uq"].T
    q = q.reshape(n, H, dn + dr)
    keys = (c @ w["l0.mix.uk"].T).reshape(n, H, dn)
    vals = (c @ w["l0.mix.uv"].T).reshape(n, H, dv)
    out = np.zeros((n, H, dv))
    for h in range(H):
        qr = np.stack([K.rotate(q[t, h, dn:], t, m["rot"]) for t in range(n)])
        s = (q[:, h, :dn] @ keys[:, h].T + qr @ kr.T) * m["scale"]
        s = np.where(np.tril(np.ones((n, n), bool)), s, -np.inf)
        p = np.exp(s - s.max(1, keepdims=True))
        out[:, h] = (p / p.sum(1, keepdims=True)) @ vals[:, h]
    want = out.reshape(n, -1) @ w["l0.mix.o"].T
    assert np.allclose(np.stack(tok), want, rtol=1e-9, atol=1e-11)


def test_gla_state_is_the_decayed_sum_of_outer_products():
    cfg, st, w, _ = model([LA("gla", mlp=False, heads=2, dim=5, vdim=7, tau=3.0)], seed=6)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    rng = np.random.default_rng(2)
    hs = rng.standard_normal((6, cfg["width"]))
    S = np.zeros((2, 5, 7))
    for t in range(6):
        K.gla_token(w, "l0.mix.", m, eps, hs[t], S)
    k = (hs @ w["l0.mix.k"].T).reshape(6, 2, 5)
    v = (hs @ w["l0.mix.v"].T).reshape(6, 2, 7)
    z = (hs @ w["l0.mix.a1"].T) @ w["l0.mix.a2"].T + w["l0.mix.a2.b"]
    la = (np.log(K.sigmoid(z)) / 3.0).reshape(6, 2, 5)
    want = np.zeros_like(S)
    for t in range(6):
        decay = np.exp(la[t + 1:].sum(0))                       # product of the later steps' decays
        want += decay[:, :, None] * k[t][:, :, None] * v[t][:, None, :]
    assert np.allclose(S, want, rtol=1e-9, atol=1e-12)


def test_router_weights_identity_experts_and_shared_gate():
    cfg, st, w, _ = model([LA("gla", experts=3, identity=2, top=2, ff=6, shared_ff=4)], seed=7)
    mlp = cfg["layers"][0]["mlp"]
    h = np.random.default_rng(3).standard_normal(cfg["width"])
    p = "l0.mlp."
    s = K.softmax(w[p + "router"] @ h)
    pick = np.argsort(-(s + w[p + "correction"]), kind="stable")[:2]
    want = sum(s[e] * (h if e >= 3 else K.clamped_expert(w, p + "e%d." % e, 2.0, h)) for e in pick)
    want = want + K.sigmoid(w[p + "shared.sg"] @ h)[0] * K.clamped_expert(w, p + "shared.", 1.5, h)
    assert np.allclose(K.moe_token(w, p, mlp, h), want)
    w2 = dict(w)
    w2[p + "correction"] = np.where(np.arange(5) >= 3, 10.0, -10.0)       # the selection bias forces both identity experts ...
    w2[p + "shared.down"] = np.zeros_like(w[p + "shared.down"])
    assert np.allclose(K.moe_token(w2, p, mlp, h), (s[3] + s[4]) * h)      # ... but the weights stay the unbiased scores
    g = K.clamped_expert({"gate": np.eye(2) * 9, "up": np.eye(2) * -9, "down": np.eye(2)}, "", 2.0, np.ones(2))
    assert np.allclose(g, 2.0 * K.sigmoid(1.702 * 2.0) * (-2.0 + 1.0))


def test_sequence_memory_makes_the_cut_irrelevant():
    layers = [LA("latent_attention", scaling=YARN), LA("gla"), LA("latent_attention", kv_from=0)]
    cfg, st, w, _ = model(layers, seed=9)
    toks = [int(t) for t in np.random.default_rng(4).integers(0, cfg["vocab"], 23)]
    whole = K.run(cfg, w, toks)
    seq, parts, at = K.Sequence(cfg), [], 0
    for c in (2, 1, 7, 13):
        parts.append(K.run(cfg, w, toks[at:at + c], seq))
        at += c
    assert np.array_equal(np.concatenate(parts), whole)
    assert seq.pos == 23 and len(seq.cache[0]) == 23 and len(seq.cache[2]) == 0


def test_model_detection_and_info_without_a_gpu():
    cfg, st, w, _ = model([LA("latent_attention"), LA("gla"), LA("gla", mlp=False)], width=48, vocab=80)
    info = capi.info_from_st(st)
    assert info["version"] == capi.ARCH_KEMIRAX
    assert (info["num_layer"], info["num_emb"], info["num_vocab"]) == (3, 48, 80)
