"""Plain float64 restatement of the Latusun forward pass (test infrastructure only).

One function per mechanism, no cache, no batching: every call recomputes the whole sequence, keys and values are
expanded per head from the latent exactly as the equations below say (the product path never expands them), and the
attention loops over query positions.  The product path never imports this file.

Notation.  x[t] is the residual row of token t (width E), m the residual multiplier.  A layer computes, both branches
from the same x,
    x <- x + m * ( mixer(LN(x; w1, b1)) + moe(LN(x; w2, b2)) ),      LN(v; w, b) = (v - mean v) / sqrt(var v + eps) * w + b
(a layer without feed-forward drops the second term).  The latent-attention mixer with H heads, per head `dk` unrotated
and `dr` rotated query/key dimensions, value size dv and latent size R computes from its input a
    q = Wq a                      per head [dk unrotated | dr rotated]
    [c' | r] = Wdkv a             R + dr rows;  c = c' / rms(c') * wc  (the cached latent),  r rotated (the cached shared key part)
    k_j^h = Wuk^h c_j,  v_j^h = Wuv^h c_j
    e_ij^h = s * ( <qu_i^h, k_j^h> + <rot(qr_i^h, i), rot(r_j, j)> ),   j <= i;   p = softmax_j e;   o_i^h = sum_j p_ij v_j^h
    out = Wo ( concat_h o^h  [* sigmoid(Wg a)] )
The two mixer kinds differ in the rotation's pairing (half-split with frequency blending / interleaved, plain) and in the
output gate; a layer may read another layer's cached (c, rotated r) instead of computing its own.
"""
from __future__ import annotations

import math

import numpy as np


def layer_norm(v: np.ndarray, w: np.ndarray, b: np.ndarray, eps: float) -> np.ndarray:
    mu = v.mean(axis=-1, keepdims=True)
    d = v - mu
    return d / np.sqrt((d * d).mean(axis=-1, keepdims=True) + eps) * w + b


def rms_weight(v: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + eps) * w


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1.0 + np.exp(-z))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def rotary_frequencies(rot: dict) -> tuple:
    """(frequencies [dims/2], magnitude factor) of a rotation; with "scaling" the frequencies are blended between f and
    f / factor along a linear ramp over the pair index and cos / sin are scaled by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(t):  # pair index whose wavelength makes t turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v: np.ndarray, positions: np.ndarray, rot: dict, interleaved: bool) -> np.ndarray:
    """v [T, n] rotated on its first rot["dims"] entries; the rest passes unchanged."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = positions[:, None].astype(np.float64) * f[None, :]
    cos, sin = np.cos(ang) * mag, np.sin(ang) * mag
    out = v.copy()
    half = dims // 2
    if interleaved:
        a, b = v[:, 0:dims:2], v[:, 1:dims:2]
        out[:, 0:dims:2] = a * cos - b * sin
        out[:, 1:dims:2] = b * cos + a * sin
    else:
        a, b = v[:, :half], v[:, half:dims]
        out[:, :half] = a * cos - b * sin
        out[:, half:dims] = b * cos + a * sin
    return out


def latent_and_shared_key(a, W, pre, m, eps, interleaved):
    """What a layer caches: (c [T, R], rotated shared key part [T, dr])."""
    R = int(m["kv_rank"])
    d = a @ W[pre + "dkv"].T
    c = rms_weight(d[:, :R], W[pre + "dkv.norm"], eps)
    r = rotate(d[:, R:], np.arange(a.shape[0]), m["rot"], interleaved)
    return c, r


def causal_softmax_attention(qu, qr, ku, kr, v, scale):
    """One head: qu/ku [T, dk], qr/kr [T, dr], v [T, dv] -> [T, dv]."""
    T = qu.shape[0]
    out = np.zeros((T, v.shape[1]))
    for i in range(T):
        e = (ku[:i + 1] @ qu[i] + kr[:i + 1] @ qr[i]) * scale
        w = np.exp(e - e.max())
        out[i] = (w / w.sum()) @ v[:i + 1]
    return out


def latent_attention_mixer(a, W, pre, m, eps, *, interleaved, gated, cached):
    """cached = (c, rotated r) of the layer whose cache this layer reads (its own or another's)."""
    H, dk, dr, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    c, r = cached
    T = a.shape[0]
    q = (a @ W[pre + "q"].T).reshape(T, H, dk + dr)
    ku = (c @ W[pre + "uk"].T).reshape(T, H, dk)
    vv = (c @ W[pre + "uv"].T).reshape(T, H, dv)
    pos = np.arange(T)
    o = np.zeros((T, H, dv))
    for h in range(H):
        qr = rotate(q[:, h, dk:], pos, m["rot"], interleaved)
        o[:, h] = causal_softmax_attention(q[:, h, :dk], qr, ku[:, h], r, vv[:, h], float(m["scale"]))
    o = o.reshape(T, H * dv)
    if gated:
        o = o * sigmoid(a @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


def moe_route(a, W, pre, top, margins=None):
    """(chosen experts [T, top], their weights [T, top]): sigmoid scores, the `top` largest, not renormalised.
    margins (a list) receives, per token, the gap between the last chosen and the first rejected router logit."""
    z = a @ W[pre + "router"].T
    s = sigmoid(z)
    order = np.argsort(-s, axis=-1, kind="stable")
    idx = order[:, :top]
    if margins is not None and top < z.shape[1]:
        zs = np.take_along_axis(z, order, axis=-1)
        margins.extend((zs[:, top - 1] - zs[:, top]).tolist())
    return idx, np.take_along_axis(s, idx, axis=-1)


def expert(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def moe(a, W, pre, mlp, margins=None):
    """sum over the chosen experts of expert(weight * input): the weight scales what the expert reads."""
    top = int(mlp["router"]["top"])
    idx, wt = moe_route(a, W, pre, top, margins)
    out = np.zeros((a.shape[0], W[pre + "e0.down"].shape[0]))
    for t in range(a.shape[0]):
        for k in range(top):
            out[t] += expert(wt[t, k] * a[t], W, f"{pre}e{idx[t, k]}.")
    return out


MIXERS = {"latent_attention": dict(interleaved=False, gated=True), "latent_attention_2": dict(interleaved=True, gated=False)}


def forward(cfg, W, tokens, want_layers: bool = False, margins=None):
    """Logits [T, vocab] (and the residual stream after every layer) of one whole sequence; margins: see moe_route."""
    eps = float(cfg["norm"]["eps"])
    mult = float(cfg.get("residual_mult", 1.0))
    x = W["embed"][np.asarray(tokens)].astype(np.float64)
    caches, trace = {}, []
    for i, lc in enumerate(cfg["layers"]):
        kind = MIXERS[lc["type"]]
        m, pre = lc["mixer"], f"l{i}."
        a = layer_norm(x, W[pre + "norm1"], W[pre + "norm1.b"], eps)
        if m.get("kv_from") is None:
            caches[i] = latent_and_shared_key(a, W, pre + "mix.", m, eps, kind["interleaved"])
            cached = caches[i]
        else:
            cached = caches[int(m["kv_from"])]
        y = latent_attention_mixer(a, W, pre + "mix.", m, eps, cached=cached, **kind)
        if lc.get("mlp") is not None:
            if lc["mlp"]["kind"] != "moe":
                raise ValueError(lc["mlp"]["kind"])
            y = y + moe(layer_norm(x, W[pre + "norm2"], W[pre + "norm2.b"], eps), W, pre + "mlp.", lc["mlp"], margins)
        x = x + mult * y
        trace.append(x.copy())
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * np.tanh(logits / float(cap))
    return (logits, np.stack(trace)) if want_layers else logits
