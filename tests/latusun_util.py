"""Shared helpers of the Latusun tests: small random configurations, weights with a planted key, the float64 oracle."""
import importlib.util
import os
import sys

import numpy as np

from pibidra_util import bf16_values, rel_rms, w64  # noqa: F401

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BLEND = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}


def oracle():
    name = "latusun_oracle"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "oracle", "latusun_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def configs(S):
    """name -> config.  Sizes differ from one another on purpose: head counts 1 .. 5, unequal key / rotated / value / latent
    sizes, sizes that are no multiple of 4 or 8, one expert and all experts chosen, layers without feed-forward, a rotation
    over only part of the rotated entries, blended frequencies on either mixer kind and on neither, cache sharing over one and
    over two layers, both mixer kinds in both orders."""
    A, B = "latent_attention", "latent_attention_2"
    L = S.latusun_layer
    return {
        "mixed": S.latusun_config(48, 70, [
            L(A, 3, 8, 4, 12, 16, experts=5, top=2, ff=24, scaling=BLEND),
            L(B, 2, 12, 8, 8, 24, experts=3, top=1, ff=40),
            L(B, 4, 6, 8, 10, 24, experts=None, kv_from=1),
            L(A, 2, 16, 8, 4, 12, experts=4, top=3, ff=16, rope_dims=4),
            L(B, 1, 20, 8, 28, 24, experts=6, top=2, ff=8, kv_from=1)], residual_mult=0.4, logit_softcap=9.0),
        "odd": S.latusun_config(36, 51, [
            L(B, 5, 5, 6, 7, 9, experts=2, top=2, ff=10, base=500.0),
            L(A, 1, 9, 2, 3, 5, experts=1, top=1, ff=13, scaling={"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5})],
            eps=1e-5, residual_mult=1.0, logit_softcap=None),
        "shared_first": S.latusun_config(40, 64, [
            L(B, 2, 8, 4, 8, 8, experts=4, top=1, ff=32, scaling=BLEND), L(B, 3, 4, 4, 16, 8, experts=None, kv_from=0, scaling=BLEND),
            L(A, 2, 8, 8, 8, 8, experts=None), L(B, 2, 8, 4, 8, 8, experts=3, top=2, ff=20, kv_from=0, scaling=BLEND)], residual_mult=0.7, logit_softcap=30.0),
        # shapes the tcgen05 projections and the tensor-core attention take in BF16 mode: width in whole 64-column tiles, fused
    # projections of 384 and 256 rows, key size (unrotated + rotated) = value size = 64
        "tiles": S.latusun_config(128, 256, [
            L(A, 2, 48, 16, 64, 112, experts=4, top=2, ff=64, scaling=BLEND), L(B, 2, 48, 16, 64, 112, experts=4, top=1, ff=128),
            L(B, 2, 48, 16, 64, 112, experts=None, kv_from=1)], residual_mult=0.5),
        # key size = value size = 128: the other instance of the tensor-core attention; a fused projection padded to whole tiles
        "tiles128": S.latusun_config(128, 200, [
            L(B, 2, 96, 32, 128, 64, experts=3, top=2, ff=64), L(A, 3, 96, 32, 128, 40, experts=None, scaling=BLEND),
            L(B, 1, 96, 32, 128, 64, experts=2, top=1, ff=32, kv_from=0)], residual_mult=0.6, logit_softcap=12.0),
        # key size 192, value size 128: the third instance; layers 0 and 2 (latent of 64, 256 key and value columns) expand keys and
        # values on the tcgen05 GEMM, layer 1 on the any-shape kernel
        "tiles192": S.latusun_config(128, 160, [
            L(B, 2, 128, 64, 128, 64, experts=2, top=1, ff=64), L(A, 1, 128, 64, 128, 40, experts=None, scaling=BLEND),
            L(B, 2, 128, 64, 128, 64, experts=None, kv_from=0)], residual_mult=0.6, logit_softcap=None),
    }


def needle_model(S, kind: str, seed: int = 3):
    """One layer whose attention is decided by ONE planted key among hundreds.  The embedding is one-hot, so after the layer
    norm a token's row is (nearly) a multiple of its unit vector; the query of token A and the latent of token B are aligned
    through a rank-one W_uk while every other pair stays small, and B's value is large.  Returns (config, weights, A, B, fillers)."""
    E, V, H, dk, dr, dv, R = 64, 48, 3, 8, 4, 8, 12
    cfg = S.latusun_config(E, V, [S.latusun_layer(kind, H, dk, dr, dv, R, experts=2, top=1, ff=16, scale=1.0)], residual_mult=1.0, logit_softcap=None)
    w = S.latusun_weights(cfg, seed)
    rng = np.random.default_rng(seed)
    emb = np.zeros((V, E), dtype=np.float32)
    emb[np.arange(V), np.arange(V)] = 1.0
    w["embed"] = emb
    w["l0.norm1"][:] = 1.0
    w["l0.norm1.b"][:] = 0.0
    w["l0.mix.q"] *= 0.02
    w["l0.mix.dkv"] *= 0.3
    w["l0.mix.dkv.norm"][:] = 1.0
    A, B = 5, 9
    u = rng.standard_normal(dk).astype(np.float32)
    u /= np.linalg.norm(u)
    v = rng.standard_normal(R).astype(np.float32)
    v /= np.linalg.norm(v)
    for h in range(H):
        w["l0.mix.q"][h * (dk + dr):h * (dk + dr) + dk, A] = u  # the unrotated query part of every head
        w["l0.mix.uk"][h * dk:(h + 1) * dk] = 0.7 * np.outer(u, v)
    w["l0.mix.dkv"][:R, B] = 3.0 * v
    w["l0.mix.uv"] += 2.0 * np.outer(rng.standard_normal(H * dv), v).astype(np.float32)
    fill = [t for t in range(V) if t not in (A, B)]
    return cfg, bf16_values(w), A, B, fill


def decisive_routing(cfg, w, seed: int = 0):
    """Weights whose routers never face a close call, for comparisons in reduced precision (a flipped expert is a different
    function, not a rounding error).  The last X entries of the width are reserved for routing: a token's embedding holds there
    a ladder 0.5, 1, ... in an order of its own, no layer writes to them (those rows of every output and down projection are
    zero), the second norm passes them with unit weight and no bias, and router row e reads one of them.  Everything else stays
    random, and all other weights read the reserved entries like any other."""
    rng = np.random.default_rng(seed)
    E, V = cfg["width"], cfg["vocab"]
    X = max([lc["mlp"]["router"]["experts"] for lc in cfg["layers"] if lc["mlp"] is not None] + [1])
    w = {k: v.copy() for k, v in w.items()}
    for t in range(V):
        w["embed"][t, E - X:] = 0.5 * (1 + rng.permutation(X))
    for i, lc in enumerate(cfg["layers"]):
        w[f"l{i}.mix.o"][E - X:] = 0.0
        if lc["mlp"] is not None:
            n = lc["mlp"]["router"]["experts"]
            pick = rng.permutation(X)[:n]
            r = np.zeros((n, E), dtype=np.float32)
            r[np.arange(n), E - X + pick] = 4.0
            w[f"l{i}.mlp.router"] = r
            w[f"l{i}.norm2"][E - X:] = 1.0
            w[f"l{i}.norm2.b"][E - X:] = 0.0
            for e in range(n):
                w[f"l{i}.mlp.e{e}.down"][E - X:] = 0.0
    return bf16_values(w)


def min_margin(O, cfg, w, toks):
    m = []
    O.forward(cfg, w64(w), toks, margins=m)
    return min(m) if m else np.inf


def random_config(S, rng):
    """A random model: 1-6 layers of either kind in any order, random head counts and sizes (incl. the tensor-core shapes), rotation
    over all or part of the rotated entries with or without blended frequencies, cache readers, 1-33 experts with 1-4 chosen or no
    feed-forward, random constants."""
    A, B = "latent_attention", "latent_attention_2"
    E = int(rng.choice([24, 40, 64, 96, 128, 192, 256, 320]))
    V = int(rng.integers(30, 400))
    layers, owners = [], []
    for i in range(int(rng.integers(1, 7))):
        kind = A if rng.random() < 0.5 else B
        H, dk, dr = int(rng.choice([1, 2, 3, 4, 6, 8])), int(rng.choice([4, 8, 12, 16, 32, 48, 64, 96, 128])), int(rng.choice([2, 4, 8, 16, 32, 64]))
        dv, R = int(rng.choice([4, 8, 20, 32, 64, 80, 128])), int(rng.choice([4, 8, 16, 24, 64, 112, 128]))
        if rng.random() < 0.3 and dk + dr in (64, 128):
            dv = dk + dr
        if rng.random() < 0.15:
            dk, dr, dv = 128, 64, 128
        rope_dims = dr if rng.random() < 0.7 else int(rng.choice(list(range(2, dr + 1, 2))))
        sc = None
        if rng.random() < 0.5:
            sc = {"factor": float(rng.choice([2.0, 8.0, 40.0])), "original": int(rng.choice([16, 64, 1024])), "fast": float(rng.choice([4.0, 32.0])),
                  "slow": float(rng.choice([0.5, 1.0]))}
        kv_from, base = None, float(rng.choice([100.0, 10000.0, 500000.0]))
        if kind == B and owners and rng.random() < 0.4:
            kv_from = int(rng.choice(owners))
            m = layers[kv_from]["mixer"]
            R, dr, rope_dims, sc, base = m["kv_rank"], m["rot_dim"], m["rot"]["dims"], m["rot"].get("scaling"), m["rot"]["base"]
        experts, top, ff = None, 1, 8
        if rng.random() >= 0.2:
            experts = int(rng.choice([x for x in (1, 2, 3, 4, 8, 16, 33) if x <= E // 2]))
            top, ff = int(rng.integers(1, min(experts, 4) + 1)), int(rng.choice([8, 24, 64, 128, 192]))
        layers.append(S.latusun_layer(kind, H, dk, dr, dv, R, experts=experts, top=top, ff=ff, base=base, rope_dims=rope_dims, scaling=sc, kv_from=kv_from,
                                      scale=float(rng.choice([1.0, 0.5, 0.25])) * (dk + dr) ** -0.5))
        if kv_from is None and kind == B:
            owners.append(i)
    return S.latusun_config(E, V, layers, eps=float(rng.choice([1e-6, 1e-5])), residual_mult=float(rng.choice([0.3, 0.5, 1.0])),
                            logit_softcap=None if rng.random() < 0.3 else float(rng.choice([5.0, 15.0, 30.0])))
