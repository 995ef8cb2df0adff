"""Plain NumPy restatement of the Kemirax decoder: one function per mechanism, written for clarity, token by token where
that is the clearest form.  It shares no code with the CUDA engine and is test infrastructure only.

Notation: W[out, in] applied as W @ x; `cfg` is the parsed config.json; weights are a dict name -> float array.
A model is a stack of parallel blocks  x <- x + G1(h) * Mixer(shift(h)) + G2(h) * FF(h),  h = scalar_rms(x),
mixers are latent attention (low-rank queries, a shared latent for keys and values, a shared rotated key part, optionally
borrowing another layer's cache) or gated linear attention (a per-channel decayed outer-product state); the feed-forward is a
routed mixture of clamped gated experts with identity experts and a gated shared expert.
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


# ----------------------------------------------------------------------------------------------------------------------
# files
# ----------------------------------------------------------------------------------------------------------------------
def read_safetensors(path_or_bytes, dtype=np.float64) -> dict:
    raw = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray, memoryview)) else open(path_or_bytes, "rb").read()
    raw = bytes(raw)
    (hlen,) = struct.unpack("<Q", raw[:8])
    head = json.loads(raw[8:8 + hlen])
    out = {}
    for name, t in head.items():
        if name == "__metadata__":
            continue
        a, b = t["data_offsets"]
        buf = raw[8 + hlen + a:8 + hlen + b]
        if t["dtype"] == "BF16":
            u = np.frombuffer(buf, np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32)
        elif t["dtype"] == "F32":
            arr = np.frombuffer(buf, np.float32)
        elif t["dtype"] == "F16":
            arr = np.frombuffer(buf, np.float16)
        elif t["dtype"] == "I32":
            arr = np.frombuffer(buf, np.int32)
        else:
            raise ValueError("dtype " + t["dtype"])
        out[name] = arr.reshape(t["shape"]).astype(dtype if t["dtype"] != "I32" else np.int64)
    return out


def bf16_round(x):
    """Round-to-nearest-even to bfloat16, returned in the input's float type."""
    a = np.asarray(x, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.asarray(x).dtype if np.asarray(x).dtype.kind == "f" else np.float32)


# ----------------------------------------------------------------------------------------------------------------------
# small pieces
# ----------------------------------------------------------------------------------------------------------------------
ROUND_OPERANDS = False      # True: the activation operand of every projection is rounded to bfloat16 first (noise-floor runs)


def lin(Wm, x):
    """Projection Wm @ x; with ROUND_OPERANDS the activation is rounded to bfloat16 as a tensor-core operand would be."""
    return Wm @ (bf16_round(np.asarray(x, np.float64)) if ROUND_OPERANDS else x)


def rms_unit(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softmax(z):
    e = np.exp(z - np.max(z))
    return e / e.sum()


def rotary_tables(rot: dict):
    """Per-pair frequency and the common magnitude factor for a rotation description
    {base, dims, scaling?: {factor, original, fast, slow}} (the YaRN rule: low frequencies are divided by `factor`,
    high ones kept, a linear ramp between; both cos and sin grow by 0.1 ln(factor) + 1)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def turn_dim(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    return f, mag


def rotate(vec, pos: int, rot: dict):
    """Rotate the first rot['dims'] entries of `vec` (pairs i, i + dims/2) by pos * f_i; the rest pass."""
    f, mag = rotary_tables(rot)
    dims = int(rot["dims"])
    half = dims // 2
    a = pos * f
    c, s = np.cos(a) * mag, np.sin(a) * mag
    out = np.array(vec, dtype=np.float64, copy=True)
    u, v = vec[:half], vec[half:dims]
    out[:half] = u * c - v * s
    out[half:dims] = v * c + u * s
    return out


# ----------------------------------------------------------------------------------------------------------------------
# mixers (one token at a time; the caller owns the per-sequence memory)
# ----------------------------------------------------------------------------------------------------------------------
def latent_attention_token(w, pre, m, eps, h, pos, cache):
    """cache: list of (latent c [kv_rank], rotated shared key [rot_dim]) of positions 0..pos (this token appended by the
    layer that owns the cache before the call returns)."""
    H, dn, dr, dv, rk = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms_unit(lin(w[pre + "dq"], h), eps) * w[pre + "dq.norm"]
    q = lin(w[pre + "uq"], cq).reshape(H, dn + dr)
    if "kv_from" not in m:
        kv = lin(w[pre + "dkv"], h)
        c = rms_unit(kv[:rk], eps) * w[pre + "dkv.norm"]
        kr = rotate(kv[rk:], pos, m["rot"])
        cache.append((c, kr))
    assert len(cache) == pos + 1
    C = np.stack([e[0] for e in cache])            # [n, rk]
    KR = np.stack([e[1] for e in cache])           # [n, dr]
    Wuk = w[pre + "uk"].reshape(H, dn, rk)
    Wuv = w[pre + "uv"].reshape(H, dv, rk)
    out = np.zeros((H, dv))
    for hd in range(H):
        qn, qr = q[hd, :dn], rotate(q[hd, dn:], pos, m["rot"])
        K = C @ Wuk[hd].T                          # [n, dn]
        Vv = C @ Wuv[hd].T                         # [n, dv]
        s = (K @ qn + KR @ qr) * float(m["scale"])
        p = softmax(s)
        out[hd] = p @ Vv
    return lin(w[pre + "o"], out.reshape(-1))


def gla_token(w, pre, m, eps, h, S):
    """S: [heads, dim, vdim] float state, updated in place."""
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = lin(w[pre + "q"], h).reshape(H, dk) * dk ** -0.5
    k = lin(w[pre + "k"], h).reshape(H, dk)
    v = lin(w[pre + "v"], h).reshape(H, dv)
    z = lin(w[pre + "a2"], lin(w[pre + "a1"], h)) + w[pre + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / float(m["tau"]))).reshape(H, dk)
    o = np.zeros((H, dv))
    for hd in range(H):
        S[hd] = alpha[hd][:, None] * S[hd] + np.outer(k[hd], v[hd])
        o[hd] = rms_unit(S[hd].T @ q[hd], eps) * w[pre + "norm"]
    g = lin(w[pre + "g"], h)
    return lin(w[pre + "o"], o.reshape(-1) * (g * sigmoid(g)))


# ----------------------------------------------------------------------------------------------------------------------
# feed-forward
# ----------------------------------------------------------------------------------------------------------------------
def clamped_expert(w, pre, limit, h):
    g = np.minimum(lin(w[pre + "gate"], h), limit)
    u = np.clip(lin(w[pre + "up"], h), -limit, limit)
    return lin(w[pre + "down"], g * sigmoid(1.702 * g) * (u + 1.0))


def moe_token(w, pre, mlp, h):
    r = mlp["router"]
    E, ident, top = int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
    s = softmax(w[pre + "router"] @ h)
    pick = s + w[pre + "correction"] if (pre + "correction") in w else s
    order = sorted(range(E + ident), key=lambda e: (-pick[e], e))[:top]
    y = np.zeros_like(h)
    for e in order:
        y = y + s[e] * (h if e >= E else clamped_expert(w, pre + "e%d." % e, float(mlp["expert"]["limit"]), h))
    if mlp.get("shared"):
        y = y + sigmoid(w[pre + "shared.sg"] @ h)[0] * clamped_expert(w, pre + "shared.", float(mlp["shared"]["limit"]), h)
    return y


# ----------------------------------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------------------------------
class Sequence:
    """Per-sequence memory: position, previous normed row per layer, attention caches, recurrent states."""

    def __init__(self, cfg):
        self.pos = 0
        W = int(cfg["width"])
        self.prev = [np.zeros(W) for _ in cfg["layers"]]
        self.cache = [[] for _ in cfg["layers"]]
        self.S = [np.zeros((int(l["mixer"]["heads"]), int(l["mixer"]["dim"]), int(l["mixer"]["vdim"]))) if l["type"] == "gla" else None
                  for l in cfg["layers"]]


def step_token(cfg, w, seq: Sequence, token: int, layers_out=None):
    eps = float(cfg["norm"]["eps"])
    x = np.array(w["embed"][token], dtype=np.float64)
    for i, l in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = rms_unit(x, eps) * float(w[p + "norm1"])
        hs = h + (seq.prev[i] - h) * w[p + "shift"]
        seq.prev[i] = h
        m = l["mixer"]
        if l["type"] == "latent_attention":
            src = int(m["kv_from"]) if "kv_from" in m else i
            a = latent_attention_token(w, p + "mix.", m, eps, hs, seq.pos, seq.cache[src])
        elif l["type"] == "gla":
            a = gla_token(w, p + "mix.", m, eps, hs, seq.S[i])
        else:
            raise ValueError(l["type"])
        a = a * sigmoid(lin(w[p + "rg1"], h) + w[p + "rg1.b"])
        if l.get("mlp"):
            f = moe_token(w, p + "mlp.", l["mlp"], h) * sigmoid(lin(w[p + "rg2"], h) + w[p + "rg2.b"])
            x = x + (a + f)
        else:
            x = x + a
        if layers_out is not None:
            layers_out.append(x.copy())
    seq.pos += 1
    return lin(w["head"], rms_unit(x, eps) * float(w["final.norm"]))


def run(cfg, w, tokens, seq: Sequence | None = None, layers=False):
    seq = seq or Sequence(cfg)
    rows, lay = [], []
    for t in tokens:
        lo = [] if layers else None
        rows.append(step_token(cfg, w, seq, int(t), lo))
        if layers:
            lay.append(np.stack(lo))
    out = np.stack(rows)
    return (out, np.stack(lay, 1)) if layers else out
