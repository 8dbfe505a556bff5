"""Plain float64 restatement of the Pibidra forward pass (test infrastructure only).

One function per mechanism, no cache, no batching tricks: every call recomputes the whole sequence
with an explicit loop over query positions, so windows, sinks and loop passes are visible in the code.
The product path never imports this file.

Notation.  x[t] is the residual row of token t (width E).  A layer computes
    x <- x + N(mixer(N(x; n1)); n1b)        x <- x + N(ff(N(x; n2)); n2b)
with N(v; w) = v / sqrt(mean(v^2) + eps) * (1 + w).  The attention mixer of a layer with H query heads,
G key/value heads, key size dk, value size dv, window W, logit cap c, score scale s and a distance table
R[B][H] (D = largest distance the logarithmic buckets resolve) computes for query position i, head h:
    q = U(Wq a + bq; wq)   k = U(Wk a + bk; wk)   v = Wv a + bv      (U: RMS over the whole vector, plain weight)
    e_ij = c * tanh(s * <q_i^h, k_j^g> / c) + R[bucket(i - j)][h],  0 <= i - j < W,  g = h // (H / G)
    p_ij = exp(e_ij) / (1 + sum_j exp(e_ij))                         (an extra zero logit without a value)
    o_i^h = sum_j p_ij v_j^g;   out_i = Wo (concat_h o_i^h * sigmoid(Wg a_i))
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


def read_safetensors(path: str) -> dict:
    """name -> float64 array (BF16 / F16 / F32 widened exactly; I32 kept as int64)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, m in head.items():
        if name == "__metadata__":
            continue
        lo, hi = m["data_offsets"]
        raw = blob[lo:hi]
        if m["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif m["dtype"] == "F16":
            a = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif m["dtype"] == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif m["dtype"] == "I32":
            a = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"dtype {m['dtype']}")
        out[name] = a.reshape(m["shape"])
    return out


def unit_rms(v: np.ndarray, eps: float) -> np.ndarray:
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def norm_offset_weight(v: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """The layer norm of this design: weight stored as a deviation from one."""
    return unit_rms(v, eps) * (1.0 + w)


def norm_plain_weight(v: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """Query / key norm: one RMS over the whole projection, weight used as stored."""
    return unit_rms(v, eps) * w


def gelu_tanh(z: np.ndarray) -> np.ndarray:
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Exact for the first rows//2 distances, logarithmic up to `far`, the last row beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def windowed_sink_attention(q, k, v, rel, *, heads, kv_heads, dk, dv, window, scale, cap, far):
    """q [T, heads*dk], k [T, kv_heads*dk], v [T, kv_heads*dv], rel [rows, heads] -> [T, heads*dv]."""
    T = q.shape[0]
    rows = rel.shape[0]
    out = np.zeros((T, heads * dv))
    group = heads // kv_heads
    for i in range(T):
        lo = max(0, i - window + 1)
        bias_rows = np.array([distance_bucket(i - j, rows, far) for j in range(lo, i + 1)])
        for h in range(heads):
            g = h // group
            qi = q[i, h * dk:(h + 1) * dk]
            s = k[lo:i + 1, g * dk:(g + 1) * dk] @ qi * scale
            e = cap * np.tanh(s / cap) + rel[bias_rows, h]
            m = max(0.0, float(e.max()))
            w = np.exp(e - m)
            p = w / (math.exp(-m) + w.sum())
            out[i, h * dv:(h + 1) * dv] = p @ v[lo:i + 1, g * dv:(g + 1) * dv]
    return out


def attention_mixer(a, W, pre, m, eps):
    q = a @ W[pre + "q"].T + W[pre + "q.b"]
    k = a @ W[pre + "k"].T + W[pre + "k.b"]
    v = a @ W[pre + "v"].T + W[pre + "v.b"]
    q = norm_plain_weight(q, W[pre + "q.norm"], eps)
    k = norm_plain_weight(k, W[pre + "k.norm"], eps)
    o = windowed_sink_attention(q, k, v, W[pre + "rel"], heads=m["heads"], kv_heads=m["kv_heads"], dk=m["dim"], dv=m["vdim"],
                                window=m["mask"]["size"], scale=m["scale"], cap=m["softcap"], far=m["bias_max"])
    gate = 1.0 / (1.0 + np.exp(-(a @ W[pre + "g"].T)))
    return (o * gate) @ W[pre + "o"].T


def dense_ff(a, W, pre):
    return (gelu_tanh(a @ W[pre + "gate"].T) * (a @ W[pre + "up"].T)) @ W[pre + "down"].T


def layer(x, W, i, spec, eps):
    pre = f"l{i}."
    if spec["type"] != "attention":
        raise ValueError(spec["type"])
    x = x + norm_offset_weight(attention_mixer(norm_offset_weight(x, W[pre + "norm1"], eps), W, pre + "mix.", spec["mixer"], eps),
                               W[pre + "norm1b"], eps)
    if spec.get("mlp") is not None:
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(spec["mlp"]["kind"])
        x = x + norm_offset_weight(dense_ff(norm_offset_weight(x, W[pre + "norm2"], eps), W, pre + "mlp."), W[pre + "norm2b"], eps)
    return x


def layer_runs(cfg) -> list:
    """(layer index, pass number or None, first-of-pass) in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t, i == loop["start"]))
    runs += [(i, None, False) for i in range(loop["stop"], n)]
    return runs


def forward(cfg, W, tokens, want_layers: bool = False):
    """Logits [T, vocab] (and the residual stream after every layer run) of one whole sequence."""
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = x0.copy()
    trace = []
    for i, t, first in layer_runs(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        x = layer(x, W, i, cfg["layers"][i], eps)
        trace.append(x.copy())
    logits = norm_offset_weight(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(trace)) if want_layers else logits
