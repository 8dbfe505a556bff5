"""CPU tests of the Latusun support code: config.json registry and the C-ABI structures, synthetic model directories, and
properties of the float64 oracle the GPU tests compare against (each mechanism on its own, and the identity the product path
rests on: folding the key expansion into the query and the value expansion behind the attention changes nothing)."""
import math

import numpy as np
import pytest

from latusun_util import BLEND, configs, decisive_routing, min_margin, needle_model, oracle, rel_rms, w64


def test_config_registry_and_abi_structs(pkg, tmp_path):
    S = pkg.synth
    cfg = configs(S)["mixed"]
    w = S.latusun_weights(cfg, 0)
    d = str(tmp_path / "m")
    S.write_model_dir(d, cfg, w)
    m = pkg.load_model(d, 77)
    c = m.configuration
    assert m.model_type == "LATUSUN" and c.arch == pkg.loader.ARCH_LATUSUN and c.context_length == 77
    assert (c.width, c.vocab_size, c.n_layers, c.block, c.residual_mult, c.logit_softcap, c.loop) == (48, 70, 5, "parallel", 0.4, 9.0, None)
    l0, l2, l3 = c.layers[0], c.layers[2], c.layers[3]
    assert (l0.mixer, l0.heads, l0.key_dim, l0.rot_dim, l0.value_dim, l0.kv_rank, l0.kv_from) == ("latent_attention", 3, 8, 4, 12, 16, -1)
    assert (l0.rope_layout, l0.gate, l0.yarn, l0.ff_kind, l0.ff_experts, l0.ff_top, l0.ff_dim, l0.ff_act) == ("half", True, (4.0, 64.0, 8.0, 1.0), "moe", 5, 2, 24, "silu")
    assert (l2.rope_layout, l2.gate, l2.kv_from, l2.ff_dim, l2.yarn[0]) == ("interleaved", False, 1, 0, 0.0)
    assert (l3.rope_dims, l3.rot_dim, l3.window) == (4, 8, 77)
    tt, dims, raw = m.tensors["l0.mlp.e4.down"]
    assert tt == pkg.loader.GGML_BF16 and dims == (24, 48) and raw.nbytes == 48 * 24 * 2
    lc, specs = pkg.plan.make_layered_config(m, "float32")
    assert (lc.arch, lc.block, lc.compute, lc.loop_times) == (4, 1, 1, -1) and abs(lc.residual_mult - 0.4) < 1e-7 and lc.logit_softcap == 9.0
    assert (specs[0].mixer, specs[0].ff_kind, specs[0].ff_experts, specs[0].ff_top, specs[0].rope_layout, specs[0].yarn_factor) == (2, 2, 5, 2, 0, 4.0)
    assert (specs[2].kv_from, specs[2].ff_kind, specs[2].rope_layout, specs[2].kv_rank, specs[2].rot_dim) == (1, 0, 1, 24, 8)
    # in-memory model = on-disk model
    mm = S.latusun_model(cfg, w, 77)
    assert mm.configuration == c and all(np.array_equal(mm.tensors[k][2], m.tensors[k][2]) for k in m.tensors)
    # defaults: no cap, multiplier one
    c2 = dict(cfg)
    del c2["logit_softcap"], c2["residual_mult"]
    cc = pkg.loader.latusun_configuration(c2, {}, 8)
    assert cc.logit_softcap == 0.0 and cc.residual_mult == 1.0
    bad = dict(cfg, layers=[dict(cfg["layers"][0], type="attention")])
    with pytest.raises(pkg.loader.UnsupportedModel):
        pkg.loader.latusun_configuration(bad, {}, 8)


def test_rotation_frequencies_and_pairing():
    O = oracle()
    f, mag = O.rotary_frequencies({"base": 100.0, "dims": 8})
    assert mag == 1.0 and np.allclose(f, [1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75])
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "original": 1000, "fast": 32.0, "slow": 1.0}}
    fb, mag = O.rotary_frequencies(rot)
    f0, _ = O.rotary_frequencies({"base": 10000.0, "dims": 32})
    assert mag == pytest.approx(0.1 * math.log(8.0) + 1.0)
    assert fb[0] == f0[0] and fb[-1] == pytest.approx(f0[-1] / 8.0)          # fast pairs keep their frequency, slow pairs are stretched
    assert np.all(np.diff(fb / f0) <= 1e-12) and np.all(fb <= f0 + 1e-18)    # and the blend falls monotonically in between
    # a score between two rotated vectors depends on the distance only, in both pairings; the magnitude enters squared
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 12)), rng.standard_normal((1, 12))
    for inter in (False, True):
        for r in ({"base": 50.0, "dims": 8}, dict(rot, dims=12, base=30.0)):
            s = [(O.rotate(q, np.array([i]), r, inter) @ O.rotate(k, np.array([j]), r, inter).T).item() for i, j in ((7, 3), (104, 100), (4, 0))]
            assert s[0] == pytest.approx(s[1]) == pytest.approx(s[2])
            same = (O.rotate(q, np.array([9]), r, inter) @ O.rotate(q, np.array([9]), r, inter).T).item()
            m2 = O.rotary_frequencies(r)[1] ** 2
            d = r["dims"]
            assert same == pytest.approx(m2 * (q[:, :d] @ q[:, :d].T).item() + (q[:, d:] @ q[:, d:].T).item())
    # the two pairings are different functions of the same vector, and entries beyond `dims` pass unchanged
    a, b = O.rotate(q, np.array([5]), {"base": 50.0, "dims": 8}, False), O.rotate(q, np.array([5]), {"base": 50.0, "dims": 8}, True)
    assert rel_rms(a[:, :8], b[:, :8]) > 0.1 and np.array_equal(a[:, 8:], q[:, 8:]) and np.array_equal(b[:, 8:], q[:, 8:])
    assert np.array_equal(O.rotate(q, np.array([0]), {"base": 50.0, "dims": 8}, True), q)


def test_norms_and_router():
    O = oracle()
    rng = np.random.default_rng(1)
    v = rng.standard_normal((3, 10)) + 2.0
    y = O.layer_norm(v, np.ones(10), np.zeros(10), 0.0)
    assert np.allclose(y.mean(-1), 0.0) and np.allclose((y * y).mean(-1), 1.0)
    assert np.allclose(O.layer_norm(v, 2 * np.ones(10), np.ones(10), 0.0), 2 * y + 1)
    r = O.rms_weight(v, np.ones(10), 0.0)
    assert np.allclose((r * r).mean(-1), 1.0) and not np.allclose(r.mean(-1), 0.0)  # no mean is taken off
    W = {"r.router": rng.standard_normal((6, 10))}
    idx, wt = O.moe_route(v, W, "r.", 3)
    s = O.sigmoid(v @ W["r.router"].T)
    for t in range(3):
        assert list(idx[t]) == list(np.argsort(-s[t])[:3]) and np.allclose(wt[t], np.sort(s[t])[::-1][:3])
        assert wt[t].sum() != pytest.approx(1.0)  # scores as they are, not renormalised


def test_expert_weight_scales_the_input(pkg):
    """sum_k expert(s_k * x): with all experts chosen the result is the plain sum over the experts of expert(s_e x), and it is
    NOT sum_k s_k expert(x)."""
    S, O = pkg.synth, oracle()
    cfg = S.latusun_config(16, 20, [S.latusun_layer("latent_attention_2", 1, 4, 4, 4, 4, experts=3, top=3, ff=8)])
    W = w64(S.latusun_weights(cfg, 2))
    a = np.random.default_rng(2).standard_normal((4, 16))
    s = O.sigmoid(a @ W["l0.mlp.router"].T)
    got = O.moe(a, W, "l0.mlp.", cfg["layers"][0]["mlp"])
    want = sum(np.stack([O.expert(s[t, e] * a[t], W, f"l0.mlp.e{e}.") for t in range(4)]) for e in range(3))
    assert np.allclose(got, want)
    outside = sum(s[:, e:e + 1] * O.expert(a, W, f"l0.mlp.e{e}.") for e in range(3))
    assert rel_rms(outside, want) > 0.05


@pytest.mark.parametrize("kind", ["latent_attention", "latent_attention_2"])
def test_folded_attention_equals_expanded_attention(pkg, kind):
    """The identity the kernels use: with q' = W_uk^T q_u per head, scores over the cached row [latent | rotated shared part] and
    values = latent, then W_uv on the result, the mixer's output equals the oracle's expanded-key computation."""
    S, O = pkg.synth, oracle()
    H, dk, dr, dv, R, E = 3, 6, 4, 5, 7, 24
    cfg = S.latusun_config(E, 30, [S.latusun_layer(kind, H, dk, dr, dv, R, experts=None, scaling=BLEND if kind == "latent_attention" else None)])
    W = w64(S.latusun_weights(cfg, 3))
    m = cfg["layers"][0]["mixer"]
    inter = O.MIXERS[kind]["interleaved"]
    a = np.random.default_rng(3).standard_normal((9, E))
    c, r = O.latent_and_shared_key(a, W, "l0.mix.", m, 1e-6, inter)
    want = O.latent_attention_mixer(a, W, "l0.mix.", m, 1e-6, cached=(c, r), **O.MIXERS[kind])
    q = (a @ W["l0.mix.q"].T).reshape(9, H, dk + dr)
    cache = np.concatenate([c, r], axis=1)
    o = np.zeros((9, H, dv))
    for h in range(H):
        Wuk, Wuv = W["l0.mix.uk"][h * dk:(h + 1) * dk], W["l0.mix.uv"][h * dv:(h + 1) * dv]
        qf = np.concatenate([q[:, h, :dk] @ Wuk, O.rotate(q[:, h, dk:], np.arange(9), m["rot"], inter)], axis=1)
        for i in range(9):
            e = cache[:i + 1] @ qf[i] * m["scale"]
            p = np.exp(e - e.max())
            o[i, h] = Wuv @ ((p / p.sum()) @ c[:i + 1])
    o = o.reshape(9, H * dv)
    if O.MIXERS[kind]["gated"]:
        o = o * O.sigmoid(a @ W["l0.mix.g"].T)
    assert np.allclose(o @ W["l0.mix.o"].T, want, rtol=1e-10, atol=1e-12)


def test_forward_is_causal_and_shares_caches(pkg):
    S, O = pkg.synth, oracle()
    cfg = configs(S)["shared_first"]
    W = w64(S.latusun_weights(cfg, 4))
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], 12).tolist()
    lg, tr = O.forward(cfg, W, toks, want_layers=True)
    assert tr.shape == (4, 12, 40) and lg.shape == (12, 64) and np.abs(lg).max() < 30.0  # the cap bounds the logits
    other = list(toks)
    other[8] = (other[8] + 1) % cfg["vocab"]
    lg2 = O.forward(cfg, W, other)
    assert np.array_equal(lg[:8], lg2[:8]) and rel_rms(lg2[8:], lg[8:]) > 1e-3
    # layer 1 reads layer 0's cache: changing layer 0's down-projection changes layer 1's mixer even with layer 0's own output cut off
    W2 = dict(W)
    W2["l0.mix.o"] = np.zeros_like(W["l0.mix.o"])
    for e in range(4):
        W2[f"l0.mlp.e{e}.down"] = np.zeros_like(W[f"l0.mlp.e{e}.down"])
    base = O.forward(cfg, W2, toks, want_layers=True)[1][1]
    W3 = dict(W2)
    W3["l0.mix.dkv"] = W2["l0.mix.dkv"] * 1.5 + 0.1
    assert rel_rms(O.forward(cfg, W3, toks, want_layers=True)[1][1], base) > 1e-3
    # without a cap the logits are the plain product
    c2 = dict(cfg)
    del c2["logit_softcap"]
    raw = O.forward(c2, W, toks)
    assert np.allclose(30.0 * np.tanh(raw / 30.0), lg)


def test_decisive_routing_and_needle_have_teeth(pkg):
    S, O = pkg.synth, oracle()
    cfg = configs(S)["mixed"]
    w = decisive_routing(cfg, S.latusun_weights(cfg, 5), 5)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 30).tolist()
    assert min_margin(O, cfg, w, toks) > 0.2
    m = []
    O.forward(cfg, w64(w), toks, margins=m)
    assert len(m) == 30 * 4  # one margin per token and layer with experts (layer 2 has none)
    for kind in ("latent_attention", "latent_attention_2"):
        cfg, w, A, B, fill = needle_model(S, kind)
        def row(dist):
            t = [fill[(5 * k + 1) % len(fill)] for k in range(121)]
            t[120] = A
            if dist is not None:
                t[120 - dist] = B
            return O.forward(cfg, w64(w), t)[120]
        assert rel_rms(row(120), row(None)) > 0.1 and rel_rms(row(1), row(None)) > 0.1


def test_generation_loop_serves_any_layered_plan(pkg):
    """engine.generate_tokens_layered needs only forward_batch_prefill / forward_decode: chunks of the prompt but its last
    token, then single steps."""
    calls = []

    class Fake:
        def forward_batch_prefill(self, toks, pos):
            calls.append(("p", list(toks), pos))

        def forward_decode(self, tok, pos, logits=False):
            calls.append(("d", tok, pos))
            return None, (tok + 1) % 50

    out = pkg.engine.generate_tokens_layered(Fake(), [3, 4, 5, 6, 7, 8], stop_tokens=[11], max_tokens=40, context_length=40, batch_size=2)
    assert calls[:3] == [("p", [3, 4], 0), ("p", [5, 6], 2), ("p", [7], 4)] and calls[3] == ("d", 8, 5)
    assert out == [9, 10, 11]
