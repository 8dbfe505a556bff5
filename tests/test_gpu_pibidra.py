"""GPU tests of the layered-plan path (csrc/layered.cuh, csrc/layered_plan.cuh) on small random Pibidra models, against the
float64 oracle (oracle/pibidra_oracle.py, which shares no code with the product).

Tolerances.  FP32 compute mode and the decode step (FP32 activations in either mode): relative RMS error of a logits row
<= 2e-5 (measured 1e-6 .. 4e-6: only the summation order differs).  BF16 compute mode, batched prefill: GEMM operands are
rounded to BF16, <= 2e-2 (measured 2e-3 .. 6e-3).  Where a test plants a key that decides the output, a window or cache slip
moves the row by more than 10 %."""
import numpy as np
import pytest

from pibidra_util import bf16_values, configs, needle_model, oracle, rel_rms, w64

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 2e-2}
TOL_DECODE = 2e-5


def make_plan(pkg, cfg, weights, ctx=256, batch=16, compute="float32"):
    model = pkg.synth.pibidra_model(cfg, weights, ctx)
    return pkg.B200MasterPlan.initialize_plan(model, prefill_batch_size=batch, compute=compute)


def prefill_all(plan, toks, batch, start=0):
    """All logits of a prompt through chunks of at most `batch` tokens."""
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
@pytest.mark.parametrize("name", ["plain", "loop_mid", "loop_start_odd", "loop_once_end", "window_one", "big_head", "tiles64", "tiles128"])
def test_every_layer_run_matches_oracle(pkg, name, compute):
    """Residual stream after every layer run and the logits: each mechanism, in the order the runs apply them."""
    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)[name]
    w = S.pibidra_weights(cfg, 11, bias_rows=rows)
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 21).tolist()
    ref_lg, ref_tr = O.forward(cfg, w64(w), toks, want_layers=True)
    plan = make_plan(pkg, cfg, w, batch=32, compute=compute)
    try:
        assert plan.layered_info()[0] == len(ref_tr)
        lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
        for r in range(len(ref_tr)):
            assert rel_rms(tr[r], ref_tr[r]) <= TOL[compute], f"layer run {r}"
        assert_rows(lg, ref_lg, TOL[compute], "logits")
    finally:
        plan.free()


@pytest.mark.parametrize("name", ["loop_mid", "loop_start_odd", "big_head"])
def test_prefill_equals_token_by_token_decode(pkg, name):
    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)[name]
    w = S.pibidra_weights(cfg, 12, bias_rows=rows)
    toks = np.random.default_rng(6).integers(0, cfg["vocab"], 40).tolist()
    ref = O.forward(cfg, w64(w), toks)
    for compute in ("float32", "bfloat16"):
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
    """The same prompt cut into portions of 2 .. 13 tokens (edges in the middle of windows), then decoded one by one; the
    chunk capacity (7) is below the portion sizes, so portions are cut again, and the ring (window - 1 + 7 slots) wraps."""
    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)["loop_mid"]
    w = S.pibidra_weights(cfg, 13, bias_rows=rows)
    toks = np.random.default_rng(7).integers(0, cfg["vocab"], 70).tolist()
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, batch=7, compute=compute)
    try:
        assert plan.layered_info()[1] == 9 - 1 + 7  # slots per run: widest window - 1 + rows of a step
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


@pytest.mark.parametrize("name", ["tiles64", "tiles128", "tiles192"])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_tensor_core_prefill_shapes(pkg, name, compute):
    """Head sizes and widths that take the tcgen05 GEMMs and the tensor-core attention in BF16 mode: a prompt longer than
    several key tiles, whole and in ragged portions (one of them a single row of a 64-row tile), then decoded."""
    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)[name]
    w = S.pibidra_weights(cfg, 21, bias_rows=rows)
    toks = np.random.default_rng(12).integers(0, cfg["vocab"], 230).tolist()
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=256, batch=100, compute=compute)
    try:
        assert_rows(prefill_all(plan, toks, 100), ref, TOL[compute], "whole")
        got, p = [], 0
        for m in (65, 2, 100, 1, 37):
            got.append(prefill_all(plan, toks[p:p + m], 100, start=p))
            p += m
        while p < len(toks):
            got.append(plan.forward_decode(toks[p], p)[0][None])
            p += 1
        assert_rows(np.concatenate(got), ref, TOL[compute], "portions")
    finally:
        plan.free()


def test_slots_are_reused_across_requests_and_wraps(pkg):
    """Request after request on one plan without clearing the cache, each long enough to wrap the ring several times; a
    request's logits do not depend on what ran before."""
    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)["plain"]
    w = S.pibidra_weights(cfg, 14, bias_rows=rows)
    plan = make_plan(pkg, cfg, w, batch=4, compute="float32")
    rng = np.random.default_rng(8)
    try:
        assert plan.layered_info()[1] == 6 - 1 + 4
        for n in (30, 3, 41, 1, 17):
            toks = rng.integers(0, cfg["vocab"], n).tolist()
            ref = O.forward(cfg, w64(w), toks)
            cut = n // 2
            got = [prefill_all(plan, toks[:cut], 4)] if cut else []
            got += [plan.forward_decode(toks[p], p)[0][None] for p in range(cut, n)]
            assert_rows(np.concatenate(got), ref, TOL["float32"], f"request of {n}")
    finally:
        plan.free()


@pytest.mark.parametrize("kv_heads", [1, 2])
@pytest.mark.parametrize("compute", ["float32", "bfloat16"])
def test_window_edges_with_a_planted_key(pkg, compute, kv_heads):
    """A key that decides the output, placed just inside (distance window - 1) and just outside (distance window) the window,
    at a far distance, and at the first positions of the sequence -- in a prompt, across a portion edge, and while decoding."""
    S, O = pkg.synth, oracle()
    W = 12
    cfg, w, A, B, fill = needle_model(S, W, kv_heads=kv_heads)
    wd = w64(w)
    plan = make_plan(pkg, cfg, w, batch=8, compute=compute)
    try:
        for i, dist in [(40, W - 1), (40, W), (40, W - 2), (40, 1), (40, 0), (W - 1, W - 1), (W, W), (3, 3), (0, 0), (57, 37)]:
            toks = [fill[(5 * t + 1) % len(fill)] for t in range(i + 1)]
            toks[i] = A
            if dist:
                toks[i - dist] = B
            ref = O.forward(cfg, wd, toks)
            # whole prompt, portions
            got = prefill_all(plan, toks, 8)
            assert_rows(got[i:i + 1], ref[i:i + 1], TOL[compute], f"prompt, query {i}, key at distance {dist}")
            # everything before the query as a prompt, the query decoded (slot of the key written by the prefill kernels)
            if i:
                prefill_all(plan, toks[:i], 8)
            lg = plan.forward_decode(toks[i], i)[0]
            assert rel_rms(lg, ref[i]) <= TOL[compute], f"decoded query {i}, key at distance {dist}"  # the keys came from the prefill kernels
            # everything decoded
            for p, t in enumerate(toks):
                lg = plan.forward_decode(t, p)[0]
            assert rel_rms(lg, ref[i]) <= TOL_DECODE, f"all decoded, query {i}, key at distance {dist}"
        # the planted key has teeth: inside and outside differ by far more than any tolerance
        def row(dist):
            toks = [fill[(5 * t + 1) % len(fill)] for t in range(41)]
            toks[40], toks[40 - dist] = A, B
            return prefill_all(plan, toks, 8)[40]
        assert rel_rms(row(W - 1), row(W)) > 0.1
    finally:
        plan.free()


def test_distance_rows_sink_and_cap_alone(pkg):
    """Weights that isolate one mechanism each: (1) zero query weights leave only the distance table to shape the attention
    (large, distinct rows: a wrong row shows); (2) a table of -30 leaves the mass on the sink, so the mixer adds nothing; (3) a
    cap far below the raw scores."""
    S, O = pkg.synth, oracle()
    L = S.pibidra_layer
    rng = np.random.default_rng(9)
    toks = rng.integers(0, 60, 50).tolist()
    for case in ("rows", "sink", "cap"):
        cfg = S.pibidra_config(40, 60, [L(2, 1, 8, 8, 33, 48, softcap=(0.5 if case == "cap" else 30.0), bias_max=29.0)])
        w = S.pibidra_weights(cfg, 15, bias_rows=10)
        if case == "rows":
            w["l0.mix.q"][:] = 0.0
            w["l0.mix.q.b"][:] = 0.0
            w["l0.mix.rel"] = (3.0 * rng.permutation(10)[:, None] * np.array([1.0, -1.0])[None, :] / 4).astype(np.float32)
        if case == "sink":
            w["l0.mix.rel"][:] = -30.0
        if case == "cap":
            w["l0.mix.q.norm"][:] = 6.0
        w = bf16_values(w)
        ref_lg, ref_tr = O.forward(cfg, w64(w), toks, want_layers=True)
        plan = make_plan(pkg, cfg, w, batch=64, compute="float32")
        try:
            lg, tr = plan.forward_batch_logits(toks, 0, list(range(len(toks))), want_trace=True)
            assert_rows(lg, ref_lg, TOL["float32"], case)
            assert rel_rms(tr[0], ref_tr[0]) <= TOL["float32"], case
            plan.kv_reset()
            step = np.stack([plan.forward_decode(t, p)[0] for p, t in enumerate(toks)])
            assert_rows(step, ref_lg, TOL_DECODE, case + " (decode)")
        finally:
            plan.free()


def test_long_decoding_through_the_device_loop(pkg):
    """300 single-token steps in one call of the device-resident loop (teacher-forced), ring of 9 slots: the argmax of every
    step equals the oracle's wherever the oracle's best two logits are not a near-tie, and the last logits agree."""
    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)["loop_once_end"]
    w = S.pibidra_weights(cfg, 16, bias_rows=rows)
    toks = np.random.default_rng(10).integers(0, cfg["vocab"], 300).tolist()
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, ctx=320, batch=1, compute="bfloat16")
    try:
        assert plan.layered_info()[1] == 11
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
    cfg, rows = configs(S)["loop_mid"]
    w = S.pibidra_weights(cfg, 17, bias_rows=rows)
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
    finally:
        plan.free()


def test_device_sampler_on_a_layered_plan(pkg):
    """Temperature / top-p sampling runs on the plan's logits row: a uniform number near 0 picks the most likely token under a
    tight top-p, and the sampled id is always a valid token."""
    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)["plain"]
    w = S.pibidra_weights(cfg, 18, bias_rows=rows)
    toks = [7, 3, 9, 1]
    ref = O.forward(cfg, w64(w), toks)
    plan = make_plan(pkg, cfg, w, batch=4, compute="bfloat16")
    try:
        plan.forward_batch_prefill(toks[:-1], 0)
        assert plan.forward_decode_sample(toks[-1], 3, 0.7, 0.05, 0.0) == int(ref[-1].argmax())
        for u in (0.1, 0.5, 0.95):
            t = plan.forward_decode_sample(toks[-1], 3, 1.3, 0.9, u)
            assert 0 <= t < cfg["vocab"]
    finally:
        plan.free()


def test_bad_arguments_are_refused(pkg):
    S = pkg.synth
    cfg, rows = configs(S)["plain"]
    w = S.pibidra_weights(cfg, 19, bias_rows=rows)
    plan = make_plan(pkg, cfg, w, ctx=16, batch=4)
    try:
        with pytest.raises(pkg.native.B200Error):
            plan.forward_batch_logits([1, 2, 3, 4, 5], 0, [0])        # longer than a chunk
        with pytest.raises(pkg.native.B200Error):
            plan.forward_batch_logits([1, 2], 15, [0])                # beyond the context
        with pytest.raises(pkg.native.B200Error):
            plan.forward_batch_logits([1, cfg["vocab"]], 0, [0])      # token out of range
        with pytest.raises(pkg.native.B200Error):
            plan.forward_batch_logits([1, 2], 0, [2])                 # row outside the chunk
        with pytest.raises(pkg.native.UnsupportedOperation):
            plan.set_decode_mode("persistent")
        with pytest.raises(pkg.native.UnsupportedOperation):
            plan.set_prefill_mode("tensor_core")
    finally:
        plan.free()
    del w["l0.mix.rel"]
    with pytest.raises(Exception):
        make_plan(pkg, cfg, w)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_replays_steps(pkg, tmp_path, dtype):
    """bin/trace_run on a model directory: steps of many tokens (longer than --chunk, so the runner cuts them), of two tokens
    and of one token, wanted places out of order, steps that want nothing, two requests one after the other on one plan; the
    files hold the wanted rows in the order asked, and every step is acknowledged."""
    import json
    import os
    import subprocess
    import sys

    S, O = pkg.synth, oracle()
    cfg, rows = configs(S)["tiles64"]
    w = S.pibidra_weights(cfg, 23, bias_rows=rows)
    mdir = str(tmp_path / "model")
    S.write_pibidra_dir(mdir, cfg, w)
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
