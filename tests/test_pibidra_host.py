"""CPU tests of the Pibidra support code: safetensors container, config.json registry, the generation loop's chunking, and
sanity properties of the float64 oracle the GPU tests compare against (each mechanism on its own)."""
import json
import math
import os

import numpy as np
import pytest

from pibidra_util import configs, needle_model, oracle, w64


def test_safetensors_roundtrip(pkg, tmp_path):
    st = pkg.safetensors
    rng = np.random.default_rng(0)
    a = rng.standard_normal((5, 7)).astype(np.float32)
    bits = st.bf16_bits(a)
    back = st.bf16_to_f32(bits).reshape(a.shape)
    assert np.max(np.abs(back - a)) <= 2.0 ** -8 * np.max(np.abs(a))
    assert np.array_equal(st.bf16_bits(back), bits)  # representable values survive
    # round to nearest even at the tie
    tie = np.array([1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8], dtype=np.float32)
    assert st.bf16_to_f32(st.bf16_bits(tie)).tolist() == [1.0, 1.0 + 2.0 ** -6]
    path = str(tmp_path / "t.safetensors")
    st.write_safetensors(path, {"a": ("BF16", a.shape, bits), "b": ("F32", (3,), np.arange(3, dtype="<f4"))}, {"k": "v"})
    f = st.SafetensorsFile(path)
    assert f.metadata == {"k": "v"} and f.infos["a"][:2] == ("BF16", (5, 7))
    assert np.array_equal(f.tensor_bytes("a").view(np.uint16).reshape(5, 7), bits)
    assert np.array_equal(f.tensor_bytes("b").view("<f4"), np.arange(3, dtype=np.float32))
    assert np.array_equal(oracle().read_safetensors(path)["a"], back.astype(np.float64))
    f.close()


def test_safetensors_rejects_bad_offsets(pkg, tmp_path):
    import struct

    head = json.dumps({"a": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 6]}}).encode()
    p = tmp_path / "bad.safetensors"
    p.write_bytes(struct.pack("<Q", len(head)) + head + b"\0" * 8)
    with pytest.raises(ValueError):
        pkg.safetensors.SafetensorsFile(str(p))


def test_config_registry(pkg, tmp_path):
    S = pkg.synth
    cfg, rows = configs(S)["loop_mid"]
    w = S.pibidra_weights(cfg, 0, bias_rows=rows)
    d = str(tmp_path / "m")
    S.write_pibidra_dir(d, cfg, w)
    m = pkg.load_model(d, 77)
    c = m.configuration
    assert m.model_type == "PIBIDRA" and c.arch == pkg.loader.ARCH_PIBIDRA and c.context_length == 77
    assert (c.width, c.vocab_size, c.n_layers, c.loop, c.norm_eps, c.embedding_scale) == (48, 80, 4, (1, 3, 3), 1e-5, 3.0)
    assert c.layer_runs() == 8 == len(oracle().layer_runs(cfg))
    l1 = c.layers[1]
    assert (l1.heads, l1.kv_heads, l1.key_dim, l1.value_dim, l1.window, l1.bias_rows, l1.ff_dim, l1.softcap) == (3, 3, 16, 8, 9, 6, 0, 4.0)
    assert c.layers[0].bias_far == 20.0 and c.layers[0].ff_dim == 40
    tt, dims, raw = m.tensors["l0.mix.q"]
    assert tt == pkg.loader.GGML_BF16 and dims == (48, 16) and raw.nbytes == 16 * 48 * 2
    lc, specs = pkg.plan.make_layered_config(m, "float32")
    assert (lc.loop_start, lc.loop_stop, lc.loop_times, lc.compute, lc.n_layers) == (1, 3, 3, 1, 4)
    assert specs[1].ff_kind == 0 and specs[0].ff_kind == 1 and specs[2].window == 4
    bad = dict(cfg, architecture="Nothing")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(bad, f)
    with pytest.raises(pkg.loader.UnsupportedModel):
        pkg.load_model(d)


def test_in_memory_model_matches_directory(pkg, tmp_path):
    S = pkg.synth
    cfg, rows = configs(S)["plain"]
    w = S.pibidra_weights(cfg, 5, bias_rows=rows)
    d = str(tmp_path / "m")
    S.write_pibidra_dir(d, cfg, w)
    a, b = pkg.load_model(d, 32), S.pibidra_model(cfg, w, 32)
    assert a.configuration == b.configuration
    assert a.tensors.keys() == b.tensors.keys()
    for k in a.tensors:
        assert a.tensors[k][:2] == b.tensors[k][:2] and np.array_equal(a.tensors[k][2], b.tensors[k][2])


def test_generation_loop_chunks_and_decodes(pkg):
    calls = []

    class FakePlan:
        def forward_batch_prefill(self, tokens, start):
            calls.append(("prefill", list(tokens), start))

        def forward_decode(self, token, pos, logits=True):
            calls.append(("decode", token, pos))
            return None, token + 100

    out = pkg.engine.generate_tokens_layered(FakePlan(), [1, 2, 3, 4, 5, 6, 7, 8], stop_tokens=[308], max_tokens=12, context_length=64, batch_size=3)
    assert calls[:3] == [("prefill", [1, 2, 3], 0), ("prefill", [4, 5, 6], 3), ("prefill", [7], 6)]
    assert calls[3:] == [("decode", 8, 7), ("decode", 108, 8), ("decode", 208, 9)]
    assert out == [108, 208, 308]  # stops at the stop token
    calls.clear()
    out = pkg.engine.generate_tokens_layered(FakePlan(), [4], stop_tokens=[], max_tokens=3, context_length=64, batch_size=8)
    assert calls == [("decode", 4, 0), ("decode", 104, 1), ("decode", 204, 2)] and len(out) == 3


# ---- the oracle's mechanisms, one at a time ---------------------------------------------------------------------------
def test_oracle_distance_rows():
    O = oracle()
    rows, far = 16, 240.0
    b = [O.distance_bucket(n, rows, far) for n in range(400)]
    assert b[:8] == list(range(8))                     # exact below rows / 2
    assert all(x <= y for x, y in zip(b, b[1:]))       # monotone
    assert b[8] == 8 and b[239] == 15 and b[240] == 15 and max(b) == 15
    assert b[43] == 11 and b[44] == 12                 # the half-way point in log space is 8 * sqrt(30) = 43.8
    assert [O.distance_bucket(n, 4, 7.0) for n in range(9)] == [0, 1, 2, 2, 3, 3, 3, 3, 3]


def test_oracle_sink_and_window():
    O = oracle()
    rng = np.random.default_rng(0)
    T, H, G, dk, dv, W = 9, 2, 1, 4, 3, 4
    q, k, v = rng.standard_normal((T, H * dk)), rng.standard_normal((T, G * dk)), rng.standard_normal((T, G * dv))
    rel = np.zeros((4, H))
    kw = dict(heads=H, kv_heads=G, dk=dk, dv=dv, window=W, scale=0.5, cap=1e9, far=64.0)
    out = O.windowed_sink_attention(q, k, v, rel, **kw)
    # by hand for one (position, head): softmax with an extra zero logit, over the last W keys only
    i, h = 7, 1
    s = np.array([q[i, h * dk:(h + 1) * dk] @ k[j] * 0.5 for j in range(i - W + 1, i + 1)])
    p = np.exp(s) / (1.0 + np.exp(s).sum())
    assert np.allclose(out[i, h * dv:(h + 1) * dv], p @ v[i - W + 1:i + 1], atol=1e-12)
    assert p.sum() < 1.0
    # a key outside the window has no influence, the oldest key inside has
    k2, v2 = k.copy(), v.copy()
    k2[i - W], v2[i - W] = 50.0, 50.0
    assert np.array_equal(O.windowed_sink_attention(q, k2, v2, rel, **kw)[i], out[i])
    v2 = v.copy()
    v2[i - W + 1] += 1.0
    assert not np.allclose(O.windowed_sink_attention(q, k, v2, rel, **kw)[i], out[i])
    # very negative logits: the sink takes all the mass and the output vanishes
    rel[:] = -40.0
    assert np.max(np.abs(O.windowed_sink_attention(q, k, v, rel, **dict(kw, cap=5.0)))) < 1e-12


def test_oracle_cap_norms_activation():
    O = oracle()
    z = np.array([-3.0, -0.5, 0.0, 0.7, 4.0])
    want = [0.5 * x * (1 + math.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3))) for x in z]
    assert np.allclose(O.gelu_tanh(z), want, atol=1e-15)
    v = np.array([[3.0, -4.0, 0.0, 0.0]])
    assert np.allclose(O.norm_offset_weight(v, np.array([0.0, 1.0, 0.0, 0.0]), 0.0), [[1.2, -3.2, 0.0, 0.0]])
    assert np.allclose(O.norm_plain_weight(v, np.array([2.0, 1.0, 1.0, 1.0]), 0.0), [[2.4, -1.6, 0.0, 0.0]])
    assert np.allclose(O.unit_rms(np.zeros((1, 4)), 1e-6), 0.0)  # eps inside the root keeps a zero row finite


def test_oracle_loop_runs_and_pass_inputs(pkg):
    O, S = oracle(), pkg.synth
    cfg, rows = configs(S)["loop_mid"]
    assert [(i, t) for i, t, _ in O.layer_runs(cfg)] == [(0, None), (1, 0), (2, 0), (1, 1), (2, 1), (1, 2), (2, 2), (3, None)]
    assert [f for _, _, f in O.layer_runs(cfg)] == [False, True, False, True, False, True, False, False]
    w = w64(S.pibidra_weights(cfg, 2, bias_rows=rows))
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    base = O.forward(cfg, w, toks)
    w2 = dict(w)
    w2["loop.step"] = w["loop.step"].copy()
    w2["loop.step"][2] += 0.5  # the third pass's vector matters ...
    assert not np.allclose(O.forward(cfg, w2, toks), base)
    cfg1 = json.loads(json.dumps(cfg))
    cfg1["loop"]["times"] = 2     # ... and is not read when there are two passes
    w3 = dict(w2, **{"loop.step": w2["loop.step"][:2]})
    w4 = dict(w, **{"loop.step": w["loop.step"][:2]})
    assert np.array_equal(O.forward(cfg1, w3, toks), O.forward(cfg1, w4, toks))


def test_oracle_is_causal_and_prefix_stable(pkg):
    O, S = oracle(), pkg.synth
    for name, (cfg, rows) in configs(S).items():
        w = w64(S.pibidra_weights(cfg, 7, bias_rows=rows))
        rng = np.random.default_rng(1)
        toks = rng.integers(0, cfg["vocab"], 14).tolist()
        full = O.forward(cfg, w, toks)
        assert np.allclose(O.forward(cfg, w, toks[:9]), full[:9], atol=1e-10), name


def test_needle_decides_the_output(pkg):
    """The planted key carries the attention when it is inside the window and nothing when it is one step outside."""
    O, S = oracle(), pkg.synth
    W = 6
    cfg, w, A, B, fill = needle_model(S, W)
    w = w64(w)
    i = 12
    def run(dist):
        toks = [fill[(3 * t) % len(fill)] for t in range(i + 1)]
        toks[i] = A
        toks[i - dist] = B
        return O.forward(cfg, w, toks)[i]
    inside, outside, none = run(W - 1), run(W), run(W + 3)
    assert np.max(np.abs(inside - outside)) > 0.1 * np.max(np.abs(inside))
    toks_far = np.max(np.abs(outside - none))
    assert toks_far < 0.5 * np.max(np.abs(inside - outside))
