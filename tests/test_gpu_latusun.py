"""GPU tests of the parallel-block path of layered plans (csrc/latent.cuh, csrc/latent_plan.cuh) on small random Latusun models,
against the float64 oracle (oracle/latusun_oracle.py: keys and values expanded per head, no cache; it shares no code with the
product, which folds the key expansion into the query and attends over the cached latent).

Tolerances.  FP32 compute mode and the decode step (FP32 activations in either mode): relative RMS error of a logits row
<= 2e-5 (only the summation order differs).  BF16 compute mode, batched prefill: GEMM operands are rounded to BF16, <= 3e-2.
Where a test plants a key that decides the output, losing that key moves the row by more than 10 %."""
import numpy as np
import pytest

from latusun_util import bf16_values, configs, decisive_routing, min_margin, needle_model, oracle, random_config, rel_rms, w64

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 3e-2}
TOL_DECODE = 2e-5


def make_plan(pkg, cfg, weights, ctx=256, batch=16, compute="float32"):
    model = pkg.synth.latusun_model(cfg, weights, ctx)
    return pkg.B200MasterPlan.initialize_plan(model, prefill_batch_size=batch, compute=compute)


def weights(S, cfg, seed, compute):
    """Random weights; for comparisons in BF16 the routers are made decisive (FP32 runs keep fully random routers)."""
    w = S.latusun_weights(cfg, seed)
    return decisive_routing(cfg, w, seed) if compute == "bfloat16" else w


def prefill_all(plan, toks, batch, start=0):
    rows = []
    for c0 in range(0, len(toks), batch):
        part = toks[c0:c0 + batch]
        lg, _ = plan.forward_batch_logits(part, start + c0, list(range(len(part))))
        rows.append(lg)
    return np.concatenate(rows)


def assert_rows(got, ref, tol, what=""):
    worst = max(rel_rms(got[i], ref[i]) for i in range(len(ref)))
    assert worst <= tol, f"{what}: relative RMS error {worst:.3g} > {tol}"


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "shared_first", "tiles", "tiles128", "tiles192"])
def test_every_layer_matches_oracle(pkg, name, compute):
    """Residual stream after every layer and the logits: norms, both mixer kinds, shared caches, routing, cap."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    w = weights(S, cfg, 11, compute)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 21).tolist()
    ref_lg, ref_tr = O.forward(cfg, w64(w), toks, want_layers=True)
    assert compute == "float32" or min_margin(O, cfg, w, toks) > 0.2
    plan = make_plan(pkg, cfg, w, batch=32, compute=compute)
    try:
        assert plan.layered_info()[0] == len(ref_tr)
        lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
        for r in range(len(ref_tr)):
            assert rel_rms(tr[r], ref_tr[r]) <= TOL[compute], f"layer {r}"
        assert_rows(lg, ref_lg, TOL[compute], "logits")
    finally:
        plan.free()


def test_each_mechanism_alone(pkg):
    """One-layer models in which one mechanism is the only thing between the embedding and the logits: (1) no feed-forward, so
    the mixer alone; (2) output projection zeroed, so the experts alone, with a router that separates tokens sharply and a
    weight far from 1 (scaling the expert's input is not scaling its output: the activation sits between); (3) rotation over a
    part of the rotated entries with and without frequency blending, at positions far beyond the blending's original length."""
    S, O = pkg.synth, oracle()
    A, B = "latent_attention", "latent_attention_2"
    L = S.latusun_layer
    rng = np.random.default_rng(9)
    cases = {
        "mixer_gated": S.latusun_config(40, 60, [L(A, 2, 8, 8, 12, 10, experts=None)], residual_mult=1.0, logit_softcap=None),
        "mixer_plain": S.latusun_config(40, 60, [L(B, 3, 4, 6, 5, 7, experts=None)], residual_mult=1.0, logit_softcap=None),
        "experts": S.latusun_config(40, 60, [L(B, 1, 4, 4, 4, 4, experts=6, top=2, ff=12)], residual_mult=1.0, logit_softcap=None),
        "rotation_part": S.latusun_config(40, 60, [L(A, 2, 2, 12, 6, 6, experts=None, rope_dims=8, base=50.0,
                                                     scaling={"factor": 16.0, "original": 8, "fast": 2.0, "slow": 0.25})], logit_softcap=None),
        "rotation_all": S.latusun_config(40, 60, [L(B, 2, 2, 12, 6, 6, experts=None, base=30.0)], logit_softcap=None),
    }
    toks = rng.integers(0, 60, 90).tolist()
    for case, cfg in cases.items():
        w = S.latusun_weights(cfg, 15)
        if case == "experts":
            w["l0.mix.o"][:] = 0.0
            w["l0.mlp.router"] *= 3.0
        if case.startswith("rotation"):
            w["l0.mix.q"] *= 3.0  # sharp attention: a wrong angle moves the weights
        w = bf16_values(w)
        ref_lg, ref_tr = O.forward(cfg, w64(w), toks, want_layers=True)
        plan = make_plan(pkg, cfg, w, batch=128, compute="float32")
        try:
            lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
            assert rel_rms(tr[0], ref_tr[0]) <= TOL["float32"], case
            assert_rows(lg, ref_lg, TOL["float32"], case)
            step = np.stack([plan.forward_decode(t, p)[0] for p, t in enumerate(toks)])
            assert_rows(step, ref_lg, TOL_DECODE, case + " (decode)")
        finally:
            plan.free()


@pytest.mark.parametrize("name", ["mixed", "odd", "shared_first"])
def test_prefill_equals_token_by_token_decode(pkg, name):
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    toks = np.random.default_rng(6).integers(0, cfg["vocab"], 40).tolist()
    for compute in ("float32", "bfloat16"):
        w = weights(S, cfg, 12, compute)
        ref = O.forward(cfg, w64(w), toks)
        plan = make_plan(pkg, cfg, w, batch=64, compute=compute)
        try:
            whole = prefill_all(plan, toks, 64)
            plan.kv_reset()
            step = np.stack([plan.forward_decode(t, p)[0] for p, t in enumerate(toks)])
            assert_rows(step, ref, TOL_DECODE, "decode")
            assert_rows(whole, ref, TOL[compute], "prefill")
            assert_rows(whole, step, TOL[compute], "prefill vs decode")
        finally:
            plan.free()


@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_portions_of_every_size(pkg, compute):
    """The same prompt cut into portions of 2 .. 13 tokens, then decoded one by one; the chunk capacity (7) is below the portion
    sizes, so portions are cut again."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["mixed"]
    w = weights(S, cfg, 13, compute)
    toks = np.random.default_rng(7).integers(0, cfg["vocab"], 70).tolist()
    ref = O.forward(cfg, w64(w), toks)
    assert compute == "float32" or min_margin(O, cfg, w, toks) > 0.2
    plan = make_plan(pkg, cfg, w, ctx=80, batch=7, compute=compute)
    try:
        assert plan.layered_info()[1] == 80  # one cache slot per position
        for sizes in ([2, 3, 2, 13, 5, 2, 11, 2, 7], [9, 2, 2, 2, 12, 3], [50]):
            got, p = [], 0
            for m in sizes:
                got.append(prefill_all(plan, toks[p:p + m], 7, start=p))
                p += m
            while p < len(toks):
                got.append(plan.forward_decode(toks[p], p)[0][None])
                p += 1
            assert_rows(np.concatenate(got), ref, TOL[compute], f"portions {sizes}")
    finally:
        plan.free()


@pytest.mark.parametrize("name", ["tiles", "tiles128", "tiles192"])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_tensor_core_shapes(pkg, name, compute):
    """Widths and fused projections in whole tiles of the tcgen05 GEMMs, (key, value) sizes (64, 64), (128, 128), (192, 128) (in BF16 mode the prefill
    expands keys and values per head and runs the tensor-core attention): a prompt of several row and key tiles, whole and in
    ragged portions (one of them a single row), a portion AFTER decoded tokens (their cache rows come from the decode step),
    then decoded; experts that receive no row, one row, and more than a tile of rows."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)[name]
    w = weights(S, cfg, 21, compute)
    if name == "tiles":
        w["l1.mlp.router"][3] *= 0.0  # an expert whose score is always 1/2: next to never the largest
    toks = np.random.default_rng(12).integers(0, cfg["vocab"], 230).tolist()
    ref = O.forward(cfg, w64(w), toks)
    assert compute == "float32" or min_margin(O, cfg, w, toks) > 0.2
    plan = make_plan(pkg, cfg, w, ctx=256, batch=100, compute=compute)
    try:
        assert_rows(prefill_all(plan, toks, 100), ref, TOL[compute], "whole")
        got, p = [], 0
        for m in (65, 2, 100, 1, -3, 37):
            if m < 0:
                for _ in range(-m):
                    got.append(plan.forward_decode(toks[p], p)[0][None])
                    p += 1
                continue
            got.append(prefill_all(plan, toks[p:p + m], 100, start=p))
            p += m
        while p < len(toks):
            got.append(plan.forward_decode(toks[p], p)[0][None])
            p += 1
        assert_rows(np.concatenate(got), ref, TOL[compute], "portions")
    finally:
        plan.free()


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations(pkg, seed):
    """Random layer lists, sizes and constants: the whole prompt, random portions with a decoded tail, and decoding from the first
    token, in both compute modes."""
    S, O = pkg.synth, oracle()
    rng = np.random.default_rng(1000 + seed)
    cfg = random_config(S, rng)
    T = int(rng.integers(3, 120))
    toks = rng.integers(0, cfg["vocab"], T).tolist()
    for compute in ("float32", "bfloat16"):
        w = weights(S, cfg, seed, compute)
        ref = O.forward(cfg, w64(w), toks)
        if compute == "bfloat16" and min_margin(O, cfg, w, toks) < 0.1:
            continue
        batch = int(rng.choice([4, 16, 64, 256]))
        plan = make_plan(pkg, cfg, w, ctx=T + 3, batch=batch, compute=compute)
        try:
            assert_rows(prefill_all(plan, toks, batch), ref, TOL[compute], "whole")
            got, p = [], 0
            while p < T - min(T, 5):
                m = min(int(rng.integers(2, 40)), T - p)
                got.append(prefill_all(plan, toks[p:p + m], batch, start=p))
                p += m
            while p < T:
                got.append(plan.forward_decode(toks[p], p)[0][None])
                p += 1
            assert_rows(np.concatenate(got), ref, TOL[compute], "portions")
            step = np.stack([plan.forward_decode(t, q)[0] for q, t in enumerate(toks[:40])])
            assert_rows(step, ref[:40], TOL_DECODE, "decode")
        finally:
            plan.free()


def test_slots_are_reused_across_requests(pkg):
    """Request after request on one plan without clearing the cache (a short one after a long one reads nothing of the long
    one's rows; shared caches included); a request's logits do not depend on what ran before."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["shared_first"]
    w = S.latusun_weights(cfg, 14)
    plan = make_plan(pkg, cfg, w, ctx=48, batch=4, compute="float32")
    rng = np.random.default_rng(8)
    try:
        for n in (30, 3, 41, 1, 17, 48):
            toks = rng.integers(0, cfg["vocab"], n).tolist()
            ref = O.forward(cfg, w64(w), toks)
            cut = n // 2
            got = [prefill_all(plan, toks[:cut], 4)] if cut else []
            got += [plan.forward_decode(toks[p], p)[0][None] for p in range(cut, n)]
            assert_rows(np.concatenate(got), ref, TOL["float32"], f"request of {n}")
    finally:
        plan.free()


@pytest.mark.parametrize("kind", ["latent_attention", "latent_attention_2"])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_far_and_first_keys_with_a_planted_key(pkg, compute, kind):
    """A key that decides the output among hundreds of others: far back, at the very first position, right before the query,
    and the query's own position -- in a prompt (whole and across portion edges), and while decoding; a key AFTER the query
    changes nothing."""
    S, O = pkg.synth, oracle()
    cfg, w, A, B, fill = needle_model(S, kind)
    wd = w64(w)
    plan = make_plan(pkg, cfg, w, ctx=400, batch=64, compute=compute)

    def prompt(i, dist, extra=0):
        toks = [fill[(5 * t + 1) % len(fill)] for t in range(i + 1 + extra)]
        toks[i] = A
        if dist is not None:
            toks[i - dist] = B
        return toks

    try:
        for i, dist in [(300, 300), (300, 299), (300, 150), (300, 1), (63, 63), (64, 64), (65, 1), (128, 64), (3, 3), (1, 1), (0, None)]:
            toks = prompt(i, dist)
            ref = O.forward(cfg, wd, toks)
            got = prefill_all(plan, toks, 64)
            assert_rows(got[i:i + 1], ref[i:i + 1], TOL[compute], f"prompt, query {i}, key at distance {dist}")
            if i:  # everything before the query as a prompt, the query decoded (the key's row was written by the prefill kernels)
                prefill_all(plan, toks[:i], 64)
            lg = plan.forward_decode(toks[i], i)[0]
            assert rel_rms(lg, ref[i]) <= TOL[compute], f"decoded query {i}, key at distance {dist}"
            if i <= 128:  # everything decoded
                for p, t in enumerate(toks):
                    lg = plan.forward_decode(t, p)[0]
                assert rel_rms(lg, ref[i]) <= TOL_DECODE, f"all decoded, query {i}, key at distance {dist}"
        # teeth: with and without the planted key the row differs by far more than any tolerance; a later key is not seen
        with_key, without = prefill_all(plan, prompt(300, 300), 64)[300], prefill_all(plan, prompt(300, None), 64)[300]
        assert rel_rms(with_key, without) > 0.1
        later = prompt(300, None, extra=5)
        later[302] = B
        assert rel_rms(prefill_all(plan, later, 64)[300], without) <= (1e-6 if compute == "float32" else 1e-3)
    finally:
        plan.free()


def test_long_decoding_through_the_device_loop(pkg):
    """300 single-token steps in one call of the device-resident loop (teacher-forced): the argmax of every step equals the
    oracle's wherever the oracle's best two logits are not a near-tie, and the last logits agree."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["shared_first"]
    w = S.latusun_weights(cfg, 16)
    toks = np.random.default_rng(10).integers(0, cfg["vocab"], 300).tolist()
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=320, batch=1, compute="bfloat16")
    try:
        ids, ms = plan.decode_sequence(toks, len(toks), 0, feedback=False)
        srt = np.sort(ref, axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 1e-3 * np.abs(ref).max()
        assert clear.sum() > 250 and np.array_equal(ids[clear], ref.argmax(1)[clear])
        assert rel_rms(plan.read_buffer("logits", cfg["vocab"]), ref[-1]) <= TOL_DECODE
        assert ms > 0
    finally:
        plan.free()


def test_greedy_generation_through_the_engine(pkg):
    """engine.generate_tokens_layered (chunked prefill, then the decode step with the device-side argmax) reproduces the
    oracle's greedy continuation; the device loop with feedback gives the same ids; the device sampler at temperature 0 too."""
    S, O = pkg.synth, oracle()
    cfg = configs(S)["mixed"]
    w = S.latusun_weights(cfg, 17)
    wd = w64(w)
    prompt = np.random.default_rng(11).integers(0, cfg["vocab"], 19).tolist()
    seq, want = list(prompt), []
    for _ in range(12):
        lg = O.forward(cfg, wd, seq)[-1]
        top = np.sort(lg)
        assert top[-1] - top[-2] > 1e-4, "near-tie in the oracle: pick another seed"
        want.append(int(lg.argmax()))
        seq.append(want[-1])
    plan = make_plan(pkg, cfg, w, ctx=64, batch=5, compute="float32")
    try:
        got = pkg.engine.generate_tokens_layered(plan, prompt, stop_tokens=[], max_tokens=len(prompt) + 11, context_length=64, batch_size=5)
        assert got == want
        stop = want[4]
        got = pkg.engine.generate_tokens_layered(plan, prompt, stop_tokens=[stop], max_tokens=64, context_length=64, batch_size=5)
        assert got == want[:want.index(stop) + 1]
        for c in range(0, len(prompt) - 1, 5):
            plan.forward_batch_prefill(prompt[c:min(c + 5, len(prompt) - 1)], c)
        ids, _ = plan.decode_sequence([prompt[-1]], 12, len(prompt) - 1, feedback=True)
        assert ids.tolist() == want
        sampler = pkg.sampler.select_sampler(cfg["vocab"], 0.0, 0.9, 1)
        got = pkg.engine.generate_tokens_layered(plan, prompt, stop_tokens=[], max_tokens=len(prompt) + 3, context_length=64, batch_size=5, sampler=sampler)
        assert got == want[:4]
        # temperature / top-p on the capped logits row: a tight top-p picks the most likely token
        for c in range(0, len(prompt) - 1, 5):
            plan.forward_batch_prefill(prompt[c:min(c + 5, len(prompt) - 1)], c)
        assert plan.forward_decode_sample(prompt[-1], len(prompt) - 1, 0.7, 0.05, 0.0) == want[0]
    finally:
        plan.free()


def test_bad_arguments_are_refused(pkg):
    S = pkg.synth
    cfg = configs(S)["mixed"]
    w = S.latusun_weights(cfg, 19)
    plan = make_plan(pkg, cfg, w, ctx=16, batch=4)
    try:
        with pytest.raises(pkg.native.B200Error):
            plan.forward_batch_logits([1, 2, 3, 4, 5], 0, [0])        # longer than a chunk
        with pytest.raises(pkg.native.B200Error):
            plan.forward_batch_logits([1, 2], 15, [0])                # beyond the context
        with pytest.raises(pkg.native.B200Error):
            plan.forward_batch_logits([1, cfg["vocab"]], 0, [0])      # token out of range
        with pytest.raises(pkg.native.UnsupportedOperation):
            plan.set_decode_mode("persistent")
    finally:
        plan.free()
    bad = dict(w)
    del bad["l1.mix.dkv"]
    with pytest.raises(Exception):
        make_plan(pkg, cfg, bad)
    import copy
    c2 = copy.deepcopy(cfg)
    c2["layers"][2]["mixer"]["kv_from"] = 3  # a layer that runs later
    with pytest.raises(Exception):
        make_plan(pkg, c2, w)
    c3 = copy.deepcopy(cfg)
    c3["layers"][4]["mixer"]["kv_from"] = 2  # a layer without a cache of its own
    with pytest.raises(Exception):
        make_plan(pkg, c3, w)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_replays_steps(pkg, tmp_path, dtype):
    """bin/trace_run on a Latusun model directory: the model class comes from config.json; steps longer than --chunk, of two
    tokens and of one, wanted places out of order, steps that want nothing, two requests one after the other."""
    import json
    import os
    import subprocess
    import sys

    S, O = pkg.synth, oracle()
    cfg = configs(S)["mixed"]
    w = weights(S, cfg, 23, dtype)
    mdir = str(tmp_path / "model")
    S.write_model_dir(mdir, cfg, w)
    rng = np.random.default_rng(13)
    reqs = {"a": rng.integers(0, cfg["vocab"], 61).tolist(), "b": rng.integers(0, cfg["vocab"], 9).tolist()}
    ref = {k: O.forward(cfg, w64(w), v) for k, v in reqs.items()}
    plan_steps = [("a", 37, [36, 0, 5]), ("a", 2, []), ("a", 20, [19, 18]), ("a", 1, [0]), ("a", 1, []), ("b", 1, [0]), ("b", 8, [7, 3])]
    lines, expect, at = [], {}, {"a": 0, "b": 0}
    for n, (rid, count, want) in enumerate(plan_steps):
        lo = at[rid]
        at[rid] = lo + count
        end = [rid] if at[rid] == len(reqs[rid]) else []
        lines.append(json.dumps({"step": n, "entries": [{"id": rid, "tokens": reqs[rid][lo:lo + count], "want": want}], "end": end}))
        if want:
            expect[n] = np.stack([ref[rid][lo + k] for k in want])
    out = str(tmp_path / "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", mdir, "--dtype", dtype, "--out", out, "--max-tokens", "64",
                        "--chunk", "16"], input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done %d" % n for n in range(len(plan_steps))]
    for n in range(len(plan_steps)):
        path = os.path.join(out, "%d.f32" % n)
        if n in expect:
            got = np.fromfile(path, dtype="<f4").reshape(expect[n].shape)
            assert_rows(got, expect[n], TOL[dtype], f"step {n}")
        else:
            assert not os.path.exists(path)
