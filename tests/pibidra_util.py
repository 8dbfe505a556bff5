"""Shared helpers of the Pibidra tests: small random configurations, weights with a planted "needle", the float64 oracle."""
import importlib.util
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def oracle():
    name = "pibidra_oracle"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "oracle", "pibidra_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def bf16_values(weights: dict) -> dict:
    """Round every value to the nearest BF16 (ties to even): what the device will hold after the upload."""
    out = {}
    for k, v in weights.items():
        u = np.ascontiguousarray(v, dtype=np.float32).view(np.uint32).astype(np.uint64)
        r = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16).view(np.float32)
        out[k] = r.reshape(v.shape)
    return out


def w64(weights: dict) -> dict:
    return {k: v.astype(np.float64) for k, v in weights.items()}


def configs(S):
    """name -> (config, bias rows).  Sizes differ from one another on purpose: unequal head / key / value sizes, grouped and
    ungrouped key/value heads, widths and vocabularies that are no multiple of 8, layers without feed-forward, loops at the
    start, in the middle, of one layer, of one pass, and none."""
    L = S.pibidra_layer
    return {
        "plain": (S.pibidra_config(64, 96, [L(4, 2, 16, 16, 6, 96), L(4, 2, 16, 16, 6, 96)]), 8),
        "loop_mid": (S.pibidra_config(48, 80, [L(2, 1, 8, 24, 5, 40, bias_max=20.0), L(3, 3, 16, 8, 9, None, softcap=4.0),
                                                L(4, 2, 12, 12, 4, 72), L(2, 2, 24, 8, 7, 56)], loop=(1, 3, 3), eps=1e-5, embedding_scale=3.0), 6),
        "loop_start_odd": (S.pibidra_config(36, 51, [L(3, 1, 12, 20, 3, 30, scale=0.4), L(6, 2, 6, 6, 8, 44)], loop=(0, 1, 2)), 10),
        "loop_once_end": (S.pibidra_config(40, 64, [L(2, 2, 20, 20, 11, 64), L(5, 1, 8, 8, 2, None)], loop=(1, 2, 1), embedding_scale=1.0), 4),
        "window_one": (S.pibidra_config(32, 40, [L(2, 1, 16, 16, 1, 48), L(2, 1, 16, 16, 64, 48)]), 16),
        "big_head": (S.pibidra_config(72, 70, [L(1, 1, 40, 160, 10, 100, bias_max=9.0)]), 12),
        # shapes the tensor-core prefill kernels take (head sizes 64 / 128, widths in whole GEMM tiles), windows that end inside a key tile
        "tiles64": (S.pibidra_config(128, 256, [L(2, 1, 64, 64, 70, 256, bias_max=100.0), L(2, 1, 64, 64, 9, 256)], loop=(0, 2, 2)), 14),
        "tiles128": (S.pibidra_config(256, 384, [L(2, 2, 128, 128, 33, 128, bias_max=40.0), L(2, 1, 128, 128, 129, 384, bias_max=200.0)]), 8),
        "tiles192": (S.pibidra_config(128, 256, [L(2, 1, 192, 128, 77, 128, bias_max=90.0), L(2, 2, 192, 128, 20, 256, bias_max=30.0)]), 10),
    }


def needle_model(S, window: int, kv_heads: int = 1, seed: int = 3):
    """One layer whose attention is decided by ONE planted key: the embedding is (nearly) one-hot, so the query of token A and
    the key of token B can be aligned while all other pairs stay small.  Returns (config, weights, A, B, filler tokens)."""
    E, V, H, dk, dv = 64, 48, 4, 16, 16
    cfg = S.pibidra_config(E, V, [S.pibidra_layer(H, kv_heads, dk, dv, window, 64, softcap=100.0, bias_max=4.0 * window)], embedding_scale=1.0)
    w = S.pibidra_weights(cfg, seed, bias_rows=8)
    rng = np.random.default_rng(seed)
    emb = np.zeros((V, E), dtype=np.float32)
    emb[np.arange(V), np.arange(V)] = 1.0
    w["embed"] = emb
    w["l0.norm1"][:] = 0.0
    w["l0.mix.q"] *= 0.05
    w["l0.mix.k"] *= 0.05
    w["l0.mix.q.b"][:] = 0.0
    w["l0.mix.k.b"][:] = 0.0
    w["l0.mix.q.norm"][:] = 1.0
    w["l0.mix.k.norm"][:] = 1.0
    w["l0.mix.rel"] *= 0.1
    A, B = 5, 9
    u = rng.standard_normal(dk).astype(np.float32)
    u /= np.linalg.norm(u)
    w["l0.mix.q"][:, A] = np.tile(u, H)
    w["l0.mix.k"][:, B] = np.tile(u, kv_heads)
    w["l0.mix.v"][:, B] += 3.0 * rng.standard_normal(kv_heads * dv).astype(np.float32)
    fill = [t for t in range(V) if t not in (A, B)]
    return cfg, bf16_values(w), A, B, fill


def rel_rms(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.sqrt(np.mean((got - ref) ** 2)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


def dump_config(cfg):
    return json.dumps(cfg, sort_keys=True)
