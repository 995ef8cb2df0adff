"""Plain NumPy restatement of the Degavik decoder: one function per mechanism, token by token, written for clarity.  It
shares no code with the CUDA engine and is test infrastructure only.

Notation: W[out, in] applied as W @ x; `cfg` is the parsed config.json; weights are a dict name -> float64 array.
A model is a stack of blocks with the norm on the sublayer's output,
    x <- x + rms(Mixer(x)) * w1,    x <- x + rms(FF(x)) * w2        (FF may be absent),
mixers: retention (fixed per-head decay, rotated q / k), a gated delta rule behind short causal convolutions, or softmax
attention with a sliding window that keeps the first tokens, capped scores and a mix of the heads' weights; feed-forward: one
gated unit or routed experts (largest logits, softmax over the chosen) plus an always-on shared expert.  A layer may use
another layer's tensors while keeping sequence memory of its own.
"""
from __future__ import annotations

import numpy as np

from .kemirax_numpy import bf16_round, read_safetensors  # noqa: F401  (file helpers only)

ROUND_OPERANDS = False      # True: the activation operand of every projection is rounded to bfloat16 first (noise-floor runs)
UNIT_EPS = 1e-6             # under the root of the delta rule's unit norms


def lin(W, x):
    return W @ (bf16_round(x) if ROUND_OPERANDS else x)


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def rotate(x, pos, dims, base, interleaved):
    """Rotary embedding of the leading `dims` entries of every row of x [heads, d] at position pos.  interleaved: entry 2i
    pairs with 2i + 1; otherwise entry i pairs with i + dims / 2.  Pair (u, v) -> (u cos a - v sin a, v cos a + u sin a),
    a = pos * base^(-2i / dims)."""
    x = np.array(x, np.float64)
    half = dims // 2
    a = pos * base ** (-2.0 * np.arange(half) / dims)
    c, s = np.cos(a), np.sin(a)
    ui, vi = (np.arange(0, dims, 2), np.arange(1, dims, 2)) if interleaved else (np.arange(half), np.arange(half) + half)
    u, v = x[:, ui].copy(), x[:, vi].copy()
    x[:, ui] = u * c - v * s
    x[:, vi] = v * c + u * s
    return x


# ----------------------------------------------------------------------------------------------------------------------
# mixers: (weights, prefix, mixer config, eps, input row, per-layer memory dict, position) -> output row
# ----------------------------------------------------------------------------------------------------------------------
def retention(w, p, c, eps, h, mem, pos):
    H, dk, dv = c["heads"], c["dim"], c["vdim"]
    q = lin(w[p + "q"], h).reshape(H, dk)
    k = lin(w[p + "k"], h).reshape(H, dk)
    v = lin(w[p + "v"], h).reshape(H, dv)
    q = rotate(q, pos, c["rot"]["dims"], c["rot"]["base"], False)
    k = rotate(k, pos, c["rot"]["dims"], c["rot"]["base"], False) * dk ** -0.5
    S = mem.setdefault("S", np.zeros((H, dk, dv)))
    out = np.zeros((H, dv))
    for i in range(H):
        S[i] = c["decay"][i] * S[i] + np.outer(k[i], v[i])
        out[i] = S[i].T @ q[i]
    out = rms(out, eps).reshape(-1) * silu(lin(w[p + "g"], h))
    return lin(w[p + "o"], out)


def short_conv(w_taps, x, tail):
    """Causal per-channel convolution: w_taps [C, taps] (last column = the current input), tail [taps - 1, C] = the inputs
    before this one (zeros at the start).  Returns (silu(conv), new tail)."""
    full = np.concatenate([tail, x[None]], 0)
    y = np.einsum("tc,ct->c", full, w_taps)
    return silu(y), full[1:]


def channel_delta(w, p, c, eps, h, mem, pos):
    H, G, dk, dv, taps = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c["vdim"], c["conv"]
    outs = {}
    for n in "qkv":
        x = lin(w[p + n], h)
        tail = mem.setdefault("tail_" + n, np.zeros((taps - 1, x.size)))
        outs[n], mem["tail_" + n] = short_conv(w[p + n + ".conv"], x, tail)
    q = outs["q"].reshape(G, dk)
    k = outs["k"].reshape(G, dk)
    v = outs["v"].reshape(H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + UNIT_EPS) * dk ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + UNIT_EPS)
    beta = sigmoid(lin(w[p + "b"], h))
    step = softplus(lin(w[p + "a2"], lin(w[p + "a1"], h)) + w[p + "dt_bias"]).reshape(H, dk)
    g = np.exp(-np.exp(w[p + "A_log"])[:, None] * step)
    S = mem.setdefault("S", np.zeros((H, dk, dv)))
    out = np.zeros((H, dv))
    for i in range(H):
        j = i // (H // G)
        S[i] = g[i][:, None] * S[i]
        u = beta[i] * (v[i] - S[i].T @ k[j])
        S[i] = S[i] + np.outer(k[j], u)
        out[i] = S[i].T @ q[j]
    out = rms(out, eps) * w[p + "norm"][None, :]
    out = out.reshape(-1) * sigmoid(lin(w[p + "g2"], lin(w[p + "g1"], h)))
    return lin(w[p + "o"], out)


def visible(i, j, size, keep):
    return j <= i and (i - j < size or j < keep)


def attention(w, p, c, eps, h, mem, pos):
    H, G, dk, dv = c["heads"], c.get("kv_heads", c["heads"]), c["dim"], c["vdim"]
    q = lin(w[p + "q"], h).reshape(H, dk)
    k = lin(w[p + "k"], h).reshape(G, dk)
    v = lin(w[p + "v"], h).reshape(G, dv)
    q = rotate(rms(q, eps) * w[p + "q.norm"], pos, c["rot"]["dims"], c["rot"]["base"], True)
    k = rotate(rms(k, eps) * w[p + "k.norm"], pos, c["rot"]["dims"], c["rot"]["base"], True)
    mem.setdefault("k", []).append(k)
    mem.setdefault("v", []).append(v)
    size, keep = c["mask"]["size"], c["mask"].get("keep_first", 0)
    js = [j for j in range(pos + 1) if visible(pos, j, size, keep)]
    P = np.zeros((H, len(js)))
    for i in range(H):
        s = np.array([mem["k"][j][i // (H // G)] @ q[i] for j in js]) * c["scale"] * w[p + "temp"][i]
        cap = c.get("softcap", 0.0)
        if cap:
            s = cap * np.tanh(s / cap)
        e = np.exp(s - s.max())
        P[i] = e / e.sum()
    P = w[p + "talk"] @ P
    out = np.stack([sum(P[i, n] * mem["v"][j][i // (H // G)] for n, j in enumerate(js)) for i in range(H)])
    return lin(w[p + "o"], out.reshape(-1))


MIXERS = {"retention": retention, "channel_delta": channel_delta, "attention": attention}


# ----------------------------------------------------------------------------------------------------------------------
# feed-forward
# ----------------------------------------------------------------------------------------------------------------------
def gated_unit(w, p, h):
    return lin(w[p + "down"], silu(lin(w[p + "gate"], h)) * lin(w[p + "up"], h))


def route(z, top):
    """The `top` largest logits (ties: lower index) and the softmax over just those."""
    idx = np.argsort(-z, kind="stable")[:top]
    e = np.exp(z[idx] - z[idx].max())
    return idx, e / e.sum()


def feed_forward(w, p, c, h):
    if c["kind"] == "dense":
        return gated_unit(w, p, h)
    z = w[p + "router"] @ h + w[p + "router.b"]          # the router reads the unrounded row
    idx, wt = route(z, c["router"]["top"])
    y = sum(wt[n] * gated_unit(w, p + "e%d." % e, h) for n, e in enumerate(idx))
    if c.get("shared"):
        y = y + gated_unit(w, p + "shared.", h)
    return y


# ----------------------------------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------------------------------
def new_memory(cfg):
    return {"pos": 0, "layers": [dict() for _ in cfg["layers"]]}


def step(cfg, w, mem, token, residuals=None):
    """One token through the stack; returns the logits row and advances `mem`."""
    eps = cfg["norm"]["eps"]
    x = np.array(w["embed"][token], np.float64)
    for i, l in enumerate(cfg["layers"]):
        src = l["weights_of"] if l.get("weights_of") is not None else i
        p = "l%d." % src
        y = MIXERS[l["type"]](w, p + "mix.", l["mixer"], eps, x, mem["layers"][i], mem["pos"])
        x = x + rms(y, eps) * w[p + "norm1"]
        if l.get("mlp"):
            x = x + rms(feed_forward(w, p + "mlp.", l["mlp"], x), eps) * w[p + "norm2"]
        if residuals is not None:
            residuals.append(x.copy())
    mem["pos"] += 1
    return lin(w["head"], rms(x, eps) * w["final.norm"])


def run(cfg, w, toks, layers=False, mem=None):
    """Logits rows [len(toks), vocab] (and, with layers, the residual after every layer [L, len(toks), width])."""
    mem = mem if mem is not None else new_memory(cfg)
    rows, res = [], []
    for t in toks:
        r = []
        rows.append(step(cfg, w, mem, int(t), r))
        res.append(np.stack(r))
    if layers:
        return np.stack(rows), np.stack(res, 1)
    return np.stack(rows)
