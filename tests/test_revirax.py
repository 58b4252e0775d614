"""Revirax through the library's own step function, cache and generation loop, against the plain float64 implementation
of `plain_revirax.py`, on small configurations made here (`revirax_cases.py`); then every mechanism alone, with inputs
made so that a fault shows (a far key that one head must find, keys at both sides of a window's edge and of a page's, a
sink that takes a known share, a state that must remember one token over hundreds).

32-bit runs: every schedule of a sequence (whole, cut into portions, token by token, inside a batch, in pages and slots
that were used before) must give the same bits, and those must lie within 32-bit rounding of the plain result.
bfloat16 runs are judged position by position (`check`): every sublayer's result is normed before it is added, so the
relative error of a chain of roundings to 8 bits enters the stream undamped, layer after layer."""

import numpy as np
import pytest
import torch

import plain_revirax as pr
from helpers import check_logits
from revirax_cases import CONFIGS, as_float64, random_weights, write_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, folder, float64 weights)."""
    out = {}
    for i, (name, make) in enumerate(CONFIGS.items()):
        cfg = make()
        w = random_weights(cfg, seed=21 + i)
        out[name] = (cfg, write_model(tmp_path_factory.mktemp(f"rev_{name}"), cfg, w), as_float64(w))
    return out


def check(got, ref, dtype, what=""):
    if dtype == "float32":
        return check_logits(got, ref, dtype, what)
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
    assert np.median(err) <= 2.5e-2, f"{what}: median error {np.median(err):.3f} of the range"
    if len(err) >= 10:
        assert np.quantile(err, 0.9) <= 6e-2, f"{what}: 90 % of the positions within {np.quantile(err, 0.9):.3f} of the range"
        assert (err > 0.15).mean() <= 0.05, f"{what}: {(err > 0.15).sum()} of {len(err)} positions differ by more than 0.15 of the range"
    else:
        assert (err > 0.15).sum() <= 1, f"{what}: errors {np.round(err, 3)} of the range"


def tokens(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def load(folder, dtype, max_tokens=64 * 12, max_seqs=4, **kw):
    import rusty_llama_b200 as rl

    return rl.load(folder, dtype=dtype, max_tokens=max_tokens, max_seqs=max_seqs, **kw)


def run_cut(llm, toks, cuts):
    """One sequence fed in portions of the given sizes (the rest one by one); logits of every position."""
    from rusty_llama_b200 import StepEntry

    s = llm.open_sequence()
    out, at = [], 0
    sizes = list(cuts) + [1] * (len(toks) - sum(cuts))
    for n in sizes:
        out.append(llm.step([StepEntry(s, toks[at : at + n], list(range(n)))]).cpu().numpy())
        at += n
    llm.close_sequence(s)
    llm.engine.check_device_status()
    return np.concatenate(out, axis=0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_against_the_plain_model(models, name, dtype):
    cfg, folder, w = models[name]
    llm = load(folder, dtype)
    for n, seed in ((1, 0), (5, 1), (150, 2)):
        toks = tokens(cfg, n, seed)
        check(run_cut(llm, toks, [n]), pr.forward(cfg, w, toks), dtype, f"{name}: prompt of {n}")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_of_a_sequence_gives_the_same_bits_in_32_bit(models, name):
    """Whole, token by token from the first token on, and portions of 2, 3, 61, 64 and 7 tokens across page borders."""
    cfg, folder, w = models[name]
    toks = tokens(cfg, 140, 5)
    llm = load(folder, "float32")
    whole = run_cut(llm, toks, [140])
    check_logits(whole, pr.forward(cfg, w, toks), "float32", name)
    for cuts in ([], [2, 3, 61, 64, 7], [63, 2, 64], [1, 1, 126, 2], [16, 17, 15, 32]):
        got = run_cut(llm, toks, cuts)
        assert np.array_equal(got, whole), f"{name}: cut {cuts} changes bits, first at row {np.nonzero((got != whole).any(1))[0][:3]}"
    llm.engine.cache.check_consistent()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_decoding_in_bfloat16(models, name):
    cfg, folder, w = models[name]
    toks = tokens(cfg, 100, 6)
    ref = pr.forward(cfg, w, toks)
    llm = load(folder, "bfloat16")
    for cuts in ([], [2, 62, 2, 30], [90]):
        check(run_cut(llm, toks, cuts), ref, "bfloat16", f"{name}: cut {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_with_leavers_and_reused_slots(models, name, dtype):
    """Three requests of unequal lengths start together and decode together; the shortest leaves first, a fourth starts in
    its slot (whose states must read zero again) and pages; each against itself alone (same bits in 32-bit) and against the
    plain model."""
    from rusty_llama_b200 import StepEntry

    cfg, folder, w = models[name]
    reqs = {"a": tokens(cfg, 131, 7), "b": tokens(cfg, 70, 8), "c": tokens(cfg, 3, 9), "d": tokens(cfg, 66, 10)}
    refs = {k: pr.forward(cfg, w, v) for k, v in reqs.items()}
    llm = load(folder, dtype, max_tokens=64 * 6, max_seqs=3)
    got = {k: [] for k in reqs}
    prompt = {"a": 120, "b": 64, "c": 1}
    slots = {k: llm.open_sequence() for k in prompt}
    out = llm.step([StepEntry(slots[k], reqs[k][: prompt[k]], list(range(prompt[k]))) for k in prompt]).cpu().numpy()
    at = 0
    for k in prompt:
        got[k].append(out[at : at + prompt[k]])
        at += prompt[k]
    pos = dict(prompt)
    live = list(prompt)
    while live:
        out = llm.step([StepEntry(slots[k], [reqs[k][pos[k]]], [0]) for k in live]).cpu().numpy()
        for i, k in enumerate(live):
            got[k].append(out[i : i + 1])
            pos[k] += 1
        for k in [k for k in live if pos[k] == len(reqs[k])]:
            llm.close_sequence(slots[k])
            live.remove(k)
            if k == "c":  # the freed slot and pages are taken at once by a new request, alone in its prompt step
                slots["d"] = llm.open_sequence()
                assert slots["d"] == slots["c"]
                got["d"].append(llm.step([StepEntry(slots["d"], reqs["d"][:60], list(range(60)))]).cpu().numpy())
                pos["d"] = 60
                live.append("d")
    llm.engine.cache.check_consistent()
    llm.engine.check_device_status()
    alone = load(folder, dtype, max_tokens=64 * 3, max_seqs=1)
    for k in reqs:
        mine = np.concatenate(got[k], axis=0)
        check(mine, refs[k], dtype, f"{name}: request {k} in the batch")
        if dtype == "float32":
            assert np.array_equal(mine, run_cut(alone, reqs[k], [len(reqs[k])])), f"{name}: request {k} depends on its batch"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_across_pages_and_graph_buckets(models, dtype):
    """300 tokens one by one after a prompt of 10: page borders at 64, 128, 192, 256, the step from a page table of 4 to one
    of 8, windows of 5, 64 and 70 that pass over decoded tokens and give pages back; with and without CUDA graphs the 32-bit
    bits are equal."""
    cfg, folder, w = models["a"]
    toks = tokens(cfg, 310, 12)
    ref = pr.forward(cfg, w, toks)
    got = run_cut(load(folder, dtype), toks, [10])
    check(got, ref, dtype, "long decoding")
    if dtype == "float32":
        assert np.array_equal(got, run_cut(load(folder, dtype, use_graphs=False), toks, [10]))


def test_greedy_generation_through_the_generation_loop(models):
    """`LLM.generate` with temperature 0 (scheduler, batching, sampler) against greedy decoding of the plain model."""
    cfg, folder, w = models["a"]
    llm = load(folder, "float32", max_tokens=64 * 8, max_seqs=4)
    prompts = [tokens(cfg, 9, 20), tokens(cfg, 70, 21), tokens(cfg, 2, 22)]
    outs = llm.generate(prompts, max_new_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, o in zip(prompts, outs):
        seq = list(p)
        for t in o:
            logits = pr.forward(cfg, w, seq)[-1]
            best = np.sort(logits)[-2:]
            if best[1] - best[0] > 1e-3 * np.abs(logits).max():  # a clear winner must be the engine's token
                assert int(np.argmax(logits)) == t
            seq.append(t)
        assert len(o) == 12


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_and_command_line(models, dtype, tmp_path):
    """The two programs a user starts: `bin/trace_run` (a prompt whole, then cut, then two requests decoded together in a
    cache that the first run has used) and `bin/rusty_llama` (greedy ids)."""
    import os
    import subprocess
    import sys

    from helpers import REPO, TraceRun

    cfg, folder, w = models["b"]
    a, b = tokens(cfg, 90, 30), tokens(cfg, 7, 31)
    ref = {"a": pr.forward(cfg, w, a), "b": pr.forward(cfg, w, b)}
    run = TraceRun(folder, dtype, str(tmp_path / "out"), 64 * 3, cfg["vocab"])
    try:
        check(run.step([("w", a, range(90))], end=["w"]), ref["a"], dtype, "whole")
        rows = [run.step([("x", a[:80], range(80)), ("y", b[:3], range(3))])]
        got = {"x": [rows[0][:80]], "y": [rows[0][80:]]}
        for t in range(10):
            live = [("x", [a[80 + t]], [0])] + ([("y", [b[3 + t]], [0])] if t < 4 else [])
            end = (["x"] if t == 9 else []) + (["y"] if t == 3 else [])
            out = run.step(live, end=end)
            got["x"].append(out[:1])
            if t < 4:
                got["y"].append(out[1:2])
        check(np.concatenate(got["x"]), ref["a"], dtype, "cut and batched")
        check(np.concatenate(got["y"]), ref["b"], dtype, "the short one")
    finally:
        run.close()
    if dtype == "float32":
        out = subprocess.run(
            [sys.executable, os.path.join(REPO, "bin", "rusty_llama"), folder, "-t", "0", "-n", "12", "-i", " ".join(map(str, b)), "--dtype", "float32"],
            capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        ids = [int(t) for t in out.stdout.split()]
        new = ids[-(12 - len(b)):]
        seq = list(b)
        for t in new:
            logits = pr.forward(cfg, w, seq)[-1]
            best = np.sort(logits)[-2:]
            if best[1] - best[0] > 1e-3 * np.abs(logits).max():
                assert int(np.argmax(logits)) == t
            seq.append(t)


# ------------------------------------------------------------------ mechanisms alone
DTYPES = [torch.float32, torch.bfloat16]


def _dev(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to("cuda", dtype)


def _rounded(a, dtype):
    return _dev(a, dtype).to(torch.float64).cpu().numpy()


def _i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device="cuda")


def _tol(dtype, f32=2e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def _paged_kv(k, v, dtype, n_pages, order):
    """k [L, G, kdim], v [L, G, vdim] laid into pages in the given order of page ids; unused places hold finite junk."""
    L, G, kd = k.shape
    vd = v.shape[2]
    kp = torch.full((n_pages, G, 64, kd), 5.0, dtype=dtype, device="cuda")
    vp = torch.full((n_pages, G, 64, vd), -3.0, dtype=dtype, device="cuda")
    width = (L + 63) // 64
    for i in range(width):
        n = min(64, L - 64 * i)
        kp[order[i], :, :n] = _dev(k[64 * i : 64 * i + n], dtype).transpose(0, 1)
        vp[order[i], :, :n] = _dev(v[64 * i : 64 * i + n], dtype).transpose(0, 1)
    return kp, vp, _i32([order[:width]])


def _plain_rows(q, k, v, positions, scale, window, sink, talk):
    """The plain attention's rows at the given positions: q [n, H, kdim] are the queries AT those positions."""
    out = []
    for i, p in enumerate(positions):
        qq = np.zeros((p + 1,) + q.shape[1:])
        qq[p] = q[i]
        out.append(pr.softmax_attention(qq, k[: p + 1], v[: p + 1], scale, window, sink, talk)[p])
    return np.stack(out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, kd, vd, talk", [(3, 1, 40, 24, False), (4, 2, 16, 48, True), (8, 8, 64, 64, True), (1, 1, 8, 200, False)])
def test_attention_finds_one_far_key_among_hundreds(dtype, H, G, kd, vd, talk):
    """One cached key far back is made to fit one head's query: that head's result must be that key's value (almost all of
    the probability, whatever the sink), the other heads' must not be; pages lie in shuffled order; queries stand around the
    page borders; key and value sizes differ; with mixed scores the mixing matrix is far from the identity."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(H * 100 + kd)
    L = 64 * 5
    k = _rounded(rng.standard_normal((L, G, kd)), dtype)
    v = _rounded(rng.standard_normal((L, G, vd)), dtype)
    sink = rng.standard_normal(H) if not talk else None
    mix = (np.eye(H) + 0.3 * rng.standard_normal((H, H))).astype(np.float32).astype(np.float64) if talk else None
    order = [4, 0, 3, 1, 2]
    hot = H - 1
    for far, positions in ((2, (255, 256, 319)), (63, (63, 64, 65, 128)), (64, (64, 127, 191, 192)), (0, (0, 1, 300))):
        q = _rounded(0.05 * rng.standard_normal((len(positions), H, kd)), dtype)
        kf = k[far, hot // (H // G)]
        q[:, hot] = _rounded(kf * (60.0 / float(kf @ kf)), dtype)  # its score with the far key is 60
        kp, vp, table = _paged_kv(k, v, dtype, 6, order)
        out = ops.attn_ext(
            _dev(q.reshape(len(positions), H * kd), dtype), kp, vp, table, _i32(np.zeros(len(positions))), _i32(positions), H, G, kd, vd, 1.0,
            sink=None if sink is None else _dev(sink, torch.float32), mix=None if mix is None else _dev(mix, torch.float32),
        ).to(torch.float64).cpu().numpy().reshape(len(positions), H, vd)
        ref = _plain_rows(q, k, v, positions, 1.0, 0, sink, mix).reshape(len(positions), H, vd)
        assert np.abs(out - ref).max() <= _tol(dtype) * max(1.0, np.abs(ref).max()), (far, positions)
        if not talk and kd >= 16:  # (among hundreds of keys of 8 numbers another one may point the same way)
            for i, p in enumerate(positions):
                if p >= far:
                    assert np.abs(out[i, hot] - v[far, hot // (H // G)]).max() < 0.05, (far, p)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 2, 40, 64, 65, 100])
def test_window_edges_in_prompts_and_decoding(dtype, window):
    """The key just inside the window (position p - window + 1) and the one just outside (p - window) are each made to fit
    the query in turn: the first must take the result over, the second must leave no trace; p stands before, at and after
    page borders and before the window is full."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(window)
    H, G, kd, vd, L = 2, 1, 16, 8, 64 * 4
    k = _rounded(0.1 * rng.standard_normal((L, G, kd)), dtype)
    v = _rounded(rng.standard_normal((L, G, vd)), dtype)
    positions = [p for p in (0, 1, window - 1, window, window + 1, 63, 64, 65, 127, 128, 129, 200, 255) if 0 <= p < L]
    for edge in ("inside", "outside"):
        for p in positions:
            j = p - window + 1 if edge == "inside" else p - window
            if j < 0:
                continue
            kk = k.copy()
            kk[j, 0] = _rounded(np.full(kd, 2.0), dtype)
            q = np.zeros((1, H, kd))
            q[0, :] = _rounded(np.full(kd, 2.0), dtype)  # score 4 kd = 64 with key j, about 0 with the others
            kp, vp, table = _paged_kv(kk, v, dtype, 5, [3, 1, 4, 0])
            out = ops.attn_ext(_dev(q.reshape(1, H * kd), dtype), kp, vp, table, _i32([0]), _i32([p]), H, G, kd, vd, 1.0, window=window)
            out = out.to(torch.float64).cpu().numpy().reshape(H, vd)
            ref = _plain_rows(q, kk, v, [p], 1.0, window, None, None).reshape(H, vd)
            assert np.abs(out - ref).max() <= _tol(dtype), (edge, p, j)
            if edge == "inside":
                assert np.abs(out[0] - v[j, 0]).max() < 0.02, (p, j)
            elif window > 1:
                assert np.abs(out[0] - v[j, 0]).max() > 0.2, (p, j)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_takes_its_share_and_gate_and_scale_apply(dtype):
    """All scores equal zero: n keys and a sink of ln(n) share the probability half and half, so the result is half the mean
    value; a sink of -100 changes nothing, one of +100 leaves nothing.  Then the gate and the constant factor."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(1)
    H, G, kd, vd, n = 3, 3, 8, 16, 70
    k = np.zeros((n, G, kd))
    v = _rounded(rng.standard_normal((n, G, vd)), dtype)
    q = _rounded(rng.standard_normal((1, H * kd)), dtype)
    kp, vp, table = _paged_kv(k, v, dtype, 3, [2, 0])
    sink = np.array([np.log(n), -100.0, 100.0])
    gate = _rounded(rng.standard_normal((1, H * vd)), dtype)
    mean = v.mean(axis=0)
    args = (_dev(q, dtype), kp, vp, table, _i32([0]), _i32([n - 1]), H, G, kd, vd, 0.7)
    out = ops.attn_ext(*args, sink=_dev(sink, torch.float32)).to(torch.float64).cpu().numpy().reshape(H, vd)
    tol = _tol(dtype, 1e-5, 1e-2)
    assert np.abs(out[0] - 0.5 * mean[0]).max() <= tol and np.abs(out[1] - mean[1]).max() <= tol and np.abs(out[2]).max() <= tol
    out = ops.attn_ext(*args, sink=_dev(sink, torch.float32), gate=_dev(gate, dtype), out_scale=1.7).to(torch.float64).cpu().numpy().reshape(H, vd)
    ref = np.stack([0.5 * mean[0], mean[1], 0 * mean[2]]) * pr.sigmoid(gate.reshape(H, vd)) * 1.7
    assert np.abs(out - ref).max() <= 2 * tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, kd, vd, rot, interleaved, magnitude", [(3, 1, 12, 20, 8, False, 1.0), (2, 2, 16, 8, 16, False, 1.3), (4, 2, 10, 10, 4, True, 0.9), (1, 1, 8, 8, 0, False, 1.0)])
def test_biases_rotation_and_cache_write(dtype, H, G, kd, vd, rot, interleaved, magnitude):
    """q in place, k and v at their places in shuffled pages; positions around a page border; two sequences."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(kd)
    pos = np.array([62, 63, 64, 65, 0, 1], dtype=np.int32)
    seq = np.array([0, 0, 0, 0, 1, 1], dtype=np.int32)
    T, cols = len(pos), (H + G) * kd + G * vd
    x = _rounded(rng.standard_normal((T, cols + 5)), dtype)  # rows longer than what is used
    bias = rng.standard_normal(cols).astype(np.float32).astype(np.float64)
    f = (100.0 ** (-2.0 * np.arange(rot // 2) / max(rot, 1))).astype(np.float32)
    table = np.array([[3, 1], [2, 0]], dtype=np.int32)
    kp = torch.zeros((4, G, 64, kd), dtype=dtype, device="cuda")
    vp = torch.zeros((4, G, 64, vd), dtype=dtype, device="cuda")
    xt = _dev(x, dtype)
    ops.qkv_prep(xt, _dev(bias, torch.float32), _i32(pos), _i32(seq), _i32(table), kp, vp, _dev(f, torch.float32) if rot else None, magnitude, H, G, kd, vd, rot, interleaved)
    y = x[:, :cols] + bias

    def turn(heads):  # [T, n, kd]
        if not rot:
            return heads
        if interleaved:
            n = rot // 2
            a = pos[:, None].astype(np.float64) * f.astype(np.float64)[None, :]
            c, s = (np.cos(a) * magnitude)[:, None, :], (np.sin(a) * magnitude)[:, None, :]
            out = heads.copy()
            u, w = heads[..., 0:rot:2], heads[..., 1:rot:2]
            out[..., 0:rot:2], out[..., 1:rot:2] = u * c - w * s, w * c + u * s
            return out
        return pr.rotate_halves(heads, pos, f.astype(np.float64), magnitude)

    q_ref = turn(y[:, : H * kd].reshape(T, H, kd))
    k_ref = turn(y[:, H * kd : (H + G) * kd].reshape(T, G, kd))
    v_ref = y[:, (H + G) * kd :].reshape(T, G, vd)
    tol = _tol(dtype, 1e-5, 3e-2)
    got = xt.to(torch.float64).cpu().numpy()
    assert np.abs(got[:, : H * kd].reshape(T, H, kd) - q_ref).max() <= tol
    assert np.array_equal(got[:, cols:], x[:, cols:])
    for t in range(T):
        page = table[seq[t], pos[t] // 64]
        assert np.abs(kp[page, :, pos[t] % 64].to(torch.float64).cpu().numpy() - k_ref[t]).max() <= tol, t
        assert np.abs(vp[page, :, pos[t] % 64].to(torch.float64).cpu().numpy() - v_ref[t]).max() <= tol, t
    assert int((kp != 0).any(dim=-1).sum()) == T * G  # nothing else was written


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, dim, vdim", [(2, 24, 40), (1, 72, 8), (3, 32, 32), (2, 128, 64)])
def test_decayed_linear_attention_through_states_and_portions(dtype, H, dim, vdim):
    """Two sequences in slots 2 and 0 of a state that holds junk in slot 1; the first is fed in portions of 15, 1, 16, 17
    and 33 tokens (the kernel takes 16 at a time), the second whole beside it; against the plain recurrence.  Then slot 2 is
    zeroed as the cache does when it opens and must forget."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(dim)
    decay = np.array([0.5, 0.97, 1.0][:H], dtype=np.float32).astype(np.float64)
    La, Lb = 82, 33
    raw = {n: _rounded(rng.standard_normal((L, H * (2 * dim + vdim))), dtype) for n, L in (("a", La), ("b", Lb))}

    def split(x):
        return x[:, : H * dim], x[:, H * dim : 2 * H * dim], x[:, 2 * H * dim :]

    ref = {}
    for n, x in raw.items():
        q, k, v = (pr.silu(t) for t in split(x))
        ref[n] = pr.decayed_linear_attention(q.reshape(-1, H, dim), k.reshape(-1, H, dim), v.reshape(-1, H, vdim), decay).reshape(-1, H * vdim)
    state = torch.zeros((3, H, dim, vdim), dtype=torch.float32, device="cuda")
    state[1] = 9.0
    got = {"a": [], "b": []}
    at = 0
    for i, n in enumerate((15, 1, 16, 17, 33)):
        rows = [raw["a"][at : at + n]] + ([raw["b"]] if i == 0 else [])
        x = _dev(np.concatenate(rows), dtype)
        q, k, v = split(x)
        starts = [0, n] + ([n + Lb] if i == 0 else [])
        out = ops.decay_attn(q, k, v, _dev(decay, torch.float32), state, _i32([2, 0][: len(rows)]), _i32(starts), H, dim, vdim, silu=True)
        out = out.to(torch.float64).cpu().numpy()
        got["a"].append(out[:n])
        if i == 0:
            got["b"].append(out[n:])
        at += n
    tol = _tol(dtype, 2e-5, 2e-5)  # the inputs are exact in both types and the kernel computes in 32-bit
    for n in ("a", "b"):
        g = np.concatenate(got[n])
        assert np.abs(g - ref[n]).max() <= tol * max(1.0, np.abs(ref[n]).max()), n
    assert float((state[1] - 9.0).abs().max()) == 0.0
    state[2].zero_()
    x = _dev(raw["a"][:5], dtype)
    q, k, v = split(x)
    out = ops.decay_attn(q, k, v, _dev(decay, torch.float32), state, _i32([2]), _i32([0, 5]), H, dim, vdim, silu=True).to(torch.float64).cpu().numpy()
    assert np.abs(out - ref["a"][:5]).max() <= tol * max(1.0, np.abs(ref["a"]).max())


def test_decayed_state_remembers_one_token_over_hundreds():
    """With decay 1 and keys that are unit vectors, the value stored with key e_3 at position 7 comes back unchanged 400
    tokens later for the query e_3, in a step of its own, whatever was stored under the other keys since."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(5)
    H, dim, vdim, L = 1, 8, 12, 408
    k = np.zeros((L, dim))
    k[np.arange(L), rng.integers(0, 3, L)] = 1.0  # keys e_0 .. e_2
    k[7] = 0.0
    k[7, 3] = 1.0
    v = rng.standard_normal((L, vdim))
    q = np.zeros((L, dim))
    q[-1, 3] = 1.0
    x = _dev(np.concatenate([q, k, v], axis=1), torch.float32)
    state = torch.zeros((1, H, dim, vdim), dtype=torch.float32, device="cuda")
    one = _dev([1.0], torch.float32)
    ops.decay_attn(x[: L - 1, :dim], x[: L - 1, dim : 2 * dim], x[: L - 1, 2 * dim :], one, state, _i32([0]), _i32([0, L - 1]), H, dim, vdim)
    out = ops.decay_attn(x[L - 1 :, :dim], x[L - 1 :, dim : 2 * dim], x[L - 1 :, 2 * dim :], one, state, _i32([0]), _i32([0, 1]), H, dim, vdim)
    assert np.abs(out.cpu().numpy()[0] - v[7]).max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [7, 50, 224, 300])
def test_min_gru_through_states_and_portions(dtype, width):
    """Portions of 1, 7, 8, 9 and 40 tokens (the kernel takes 8 at a time) of one sequence, another whole beside it in the first
    step; a channel whose gate is shut after the first token must keep that token's candidate to the end."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(width)
    La, Lb = 65, 12
    raw = {n: _rounded(2.0 * rng.standard_normal((L, 3 * width)), dtype) for n, L in (("a", La), ("b", Lb))}
    raw["a"][0, 0], raw["a"][1:, 0] = _rounded(30.0, dtype), _rounded(-30.0, dtype)  # channel 0: z = 1, then 0
    bz = rng.standard_normal(width).astype(np.float32).astype(np.float64)
    bx = rng.standard_normal(width).astype(np.float32).astype(np.float64)
    bz[0] = 0.0
    ref = {}
    for n, x in raw.items():
        S = pr.min_gru(pr.sigmoid(x[:, :width] + bz), x[:, width : 2 * width] + bx)
        ref[n] = S * pr.silu(x[:, 2 * width :]) * 1.1
    state = torch.zeros((2, width), dtype=torch.float32, device="cuda")
    got = {"a": [], "b": []}
    at = 0
    for i, n in enumerate((1, 7, 8, 9, 40)):
        rows = [raw["a"][at : at + n]] + ([raw["b"]] if i == 0 else [])
        x = _dev(np.concatenate(rows), dtype)
        starts = [0, n] + ([n + Lb] if i == 0 else [])
        out = ops.min_gru(x[:, :width], x[:, width : 2 * width], x[:, 2 * width :], _dev(bz, torch.float32), _dev(bx, torch.float32), state,
                          _i32([1, 0][: len(rows)]), _i32(starts), out_scale=1.1).to(torch.float64).cpu().numpy()
        got["a"].append(out[:n])
        if i == 0:
            got["b"].append(out[n:])
        at += n
    for n in ("a", "b"):
        g = np.concatenate(got[n])
        assert np.abs(g - ref[n]).max() <= _tol(dtype, 1e-5, 1.5e-2) * max(1.0, np.abs(ref[n]).max()), n
    u0 = raw["a"][0, width] + bx[0]
    assert abs(float(state[1, 0]) - (u0 + 0.5 if u0 >= 0 else pr.sigmoid(u0))) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_row_kernels(dtype):
    """The norm of the linear attention's heads with its gate; the squared relu; the sandwich norm with a bias row and
    weights that were stored as distances from one."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(9)
    T, n = 5, 136
    x = rng.standard_normal((T, n)).astype(np.float32).astype(np.float64)
    w = rng.standard_normal(n).astype(np.float32).astype(np.float64)
    g = _rounded(rng.standard_normal((T, n + 3)), dtype)
    out = ops.rms_gate(_dev(x, torch.float32), _dev(w, torch.float32), 1e-5, _dev(g, dtype)[:, :n], dtype, out_scale=0.6)
    ref = pr.rms_unit(x, 1e-5) * w * pr.sigmoid(g[:, :n]) * 0.6
    assert np.abs(out.to(torch.float64).cpu().numpy() - ref).max() <= _tol(dtype, 1e-5, 2e-2) * np.abs(ref).max()
    h = _rounded(rng.standard_normal((T, n)), dtype)
    out = ops.unary_act(_dev(h, dtype)).to(torch.float64).cpu().numpy()
    assert np.abs(out - np.maximum(h, 0) ** 2).max() <= _tol(dtype, 1e-6, 2e-2) * 4
    d = 96
    xs = rng.standard_normal((T, d)).astype(np.float32).astype(np.float64)
    delta = _rounded(rng.standard_normal((T, d)), dtype)
    bias = rng.standard_normal(d).astype(np.float32).astype(np.float64)
    wd = (1.0 + 0.3 * rng.standard_normal(d)).astype(np.float32).astype(np.float64)
    wn = (1.0 + 0.3 * rng.standard_normal(d)).astype(np.float32).astype(np.float64)
    xt = _dev(xs, torch.float32)
    out = ops.normed_add_rmsnorm(xt, _dev(delta, dtype), _dev(wd, torch.float32), 1e-5, _dev(wn, torch.float32), 1e-6, dtype, delta_bias=_dev(bias, torch.float32))
    x_ref = xs + pr.centred_norm(delta + bias, wd - 1.0, 1e-5)
    assert np.abs(xt.to(torch.float64).cpu().numpy() - x_ref).max() <= 2e-5
    ref = pr.centred_norm(x_ref, wn - 1.0, 1e-6)
    assert np.abs(out.to(torch.float64).cpu().numpy() - ref).max() <= _tol(dtype, 1e-5, 2e-2) * np.abs(ref).max()


@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("hd, H, G", [(64, 8, 2), (128, 4, 4), (48, 6, 3), (24, 2, 1)])
def test_sink_on_the_tensor_core_attention_kernels(hd, H, G, window):
    """The bfloat16 kernels of a plain attention with a sink: a prompt that goes on from position 70 with 90 tokens (both prompt
    kernels where the head size allows), then single tokens at positions around page borders with the key range in one part
    and in several (both decode kernels).  Sinks of the size of the scores, one very large, one very small."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(hd)
    dt, L = torch.bfloat16, 64 * 5
    k = _rounded(rng.standard_normal((L, G, hd)), dt)
    v = _rounded(rng.standard_normal((L, G, hd)), dt)
    sink = np.concatenate([[30.0, -30.0], 2.0 * rng.standard_normal(H)])[:H] if H > 2 else np.array([1.0, 30.0])
    scale = 0.9 / np.sqrt(hd)
    kp, vp, table = _paged_kv(k, v, dt, 7, [5, 0, 3, 6, 2])
    sink_t = _dev(sink, torch.float32)
    q_all = _rounded(rng.standard_normal((L, H, hd)), dt)
    ref = pr.softmax_attention(q_all, k, v, scale, window, sink, None)
    # prompt: rows 70 .. 159
    q = _dev(q_all[70:160].reshape(90, H * hd), dt)
    start, pos0 = _i32([0, 90]), _i32([70])
    outs = {"flash_prefill": ops.flash_prefill(q, kp, vp, table, start, pos0, 90, H, G, hd, scale=scale, sink=sink_t, window=window)}
    if hd in ops.FLASH_TC_HEAD_DIMS:
        outs["flash_prefill_tc"] = ops.flash_prefill_tc(q, kp, vp, table, start, pos0, 90, H, G, hd, scale=scale, sink=sink_t, window=window)
    for name, out in outs.items():
        err = np.abs(out.to(torch.float64).cpu().numpy() - ref[70:160]).max()
        assert err <= 2e-2 * max(1.0, np.abs(ref).max()), (name, err)
    # decoding
    for p in (0, 1, 63, 64, 65, 200, 319):
        qd = _dev(q_all[p : p + 1].reshape(1, H * hd), dt)
        for impl in ("warp",) + (("tma",) if hd in ops.ATTN_DECODE_TMA_HEAD_DIMS else ()):
            for n_splits in (1, 3):
                scratch = torch.empty(ops.attn_decode_scratch_floats(1, H, hd, n_splits), dtype=torch.float32, device="cuda")
                out = ops.attn_decode(qd, kp, vp, table, _i32([p + 1]), H, G, hd, n_splits, scratch, scale=scale, impl=impl, sink=sink_t, window=window)
                err = np.abs(out.to(torch.float64).cpu().numpy()[0] - ref[p]).max()
                assert err <= 2e-2 * max(1.0, np.abs(ref).max()), (impl, n_splits, p, err)
    ops.tc_status_check()


@pytest.mark.parametrize("H, G, kd, vd, window, talk, use_sink", [
    (4, 2, 32, 32, 40, True, False), (8, 4, 16, 24, 5, True, False), (2, 1, 96, 96, 64, True, False), (6, 2, 24, 8, 0, False, True),
    (4, 4, 128, 64, 65, True, True), (1, 1, 8, 200, 0, False, False), (16, 8, 64, 64, 100, True, False)])
def test_tensor_core_attention_with_options(H, G, kd, vd, window, talk, use_sink):
    """`flash_mix` on a ragged step (a sequence that goes on from position 70 with 100 tokens, one that starts with 3, one that
    brings a single token at position 200) and on single tokens around page borders and window edges, against the plain
    attention: folded queries for the mixed scores, unequal key and value sizes, window, sink, gate and factor."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(H * 7 + kd)
    dt = torch.bfloat16
    lens = [(70, 100), (0, 3), (200, 1)]
    n_pages, width = 12, 4
    perm = rng.permutation(n_pages)
    table = np.zeros((3, width), dtype=np.int32)
    kp = torch.full((n_pages, G, 64, kd), 2.0, dtype=dt, device="cuda")
    vp = torch.full((n_pages, G, 64, vd), -2.0, dtype=dt, device="cuda")
    mix = (np.eye(H) * 0.8 + 0.4 * rng.standard_normal((H, H))).astype(np.float32).astype(np.float64) if talk else None
    sink = 1.5 * rng.standard_normal(H) if use_sink else None
    scale = 1.3 / np.sqrt(kd)
    ks, vs, qs, refs, at = [], [], [], [], 0
    for s, (held, n) in enumerate(lens):
        L = held + n
        k = _rounded(rng.standard_normal((L, G, kd)), dt)
        v = _rounded(rng.standard_normal((L, G, vd)), dt)
        q = _rounded(rng.standard_normal((L, H, kd)), dt)
        for i in range((L + 63) // 64):
            table[s, i] = perm[at]
            m = min(64, L - 64 * i)
            kp[perm[at], :, :m] = _dev(k[64 * i : 64 * i + m], dt).transpose(0, 1)
            vp[perm[at], :, :m] = _dev(v[64 * i : 64 * i + m], dt).transpose(0, 1)
            at += 1
        refs.append(pr.softmax_attention(q, k, v, scale, window, sink, mix)[held:])
        qs.append(q[held:])
        ks.append(k)
        vs.append(v)
    T = sum(n for _, n in lens)
    q_t = _dev(np.concatenate(qs).reshape(T, H * kd), dt)
    gate = _rounded(rng.standard_normal((T, H * vd)), dt)
    ref = np.concatenate(refs) * pr.sigmoid(gate) * 0.6
    start = _i32(np.concatenate([[0], np.cumsum([n for _, n in lens])]))
    pos0 = _i32([h for h, _ in lens])
    qq = ops.fold_queries(q_t, _dev(mix, torch.float32), H, G, kd) if talk else q_t
    wide = torch.zeros((T, H * vd + 6), dtype=dt, device="cuda")
    out = ops.flash_mix(qq, kp, vp, torch.from_numpy(table).cuda(), start, pos0, 100, H, G, kd, vd, scale, window=window,
                        sink=None if sink is None else _dev(sink, torch.float32), folded=talk, gate=_dev(gate, dt), out_scale=0.6, out=wide[:, : H * vd])
    err = np.abs(out.to(torch.float64).cpu().numpy() - ref).max()
    assert err <= 2.5e-2 * max(1.0, np.abs(ref).max()), err
    assert float(wide[:, H * vd :].abs().max()) == 0.0
    # single tokens of the first sequence, as a decode step of one sequence each
    k, v = ks[0], vs[0]
    full = pr.softmax_attention(np.concatenate([np.zeros((70, H, kd)), qs[0]]), k, v, scale, window, sink, mix)
    for p in (70, 127, 128, 129, 169):
        q1 = _dev(qs[0][p - 70 : p - 69].reshape(1, H * kd), dt)
        qq = ops.fold_queries(q1, _dev(mix, torch.float32), H, G, kd) if talk else q1
        out = ops.flash_mix(qq, kp, vp, torch.from_numpy(table[:1]).cuda(), _i32([0, 1]), _i32([p]), 1, H, G, kd, vd, scale, window=window,
                            sink=None if sink is None else _dev(sink, torch.float32), folded=talk)
        err = np.abs(out.to(torch.float64).cpu().numpy()[0] - full[p]).max()
        assert err <= 2.5e-2 * max(1.0, np.abs(full).max()), (p, err)
        # the decode kernel whose rows are the heads, with the key range in one part, in three and in more parts than pages
        fold = _dev(mix if talk else np.eye(H), torch.float32)
        g1 = _rounded(rng.standard_normal((1, H * vd)), dt)
        for n_splits in (1, 3, 7):
            scratch = torch.full((ops.flash_mix_decode_scratch_floats(1, H, vd, n_splits),), float("nan"), device="cuda")
            out = ops.flash_mix_decode(ops.fold_queries(q1, fold, H, G, kd), kp, vp, torch.from_numpy(table[:1]).cuda(), _i32([p]), H, G, kd, vd, scale,
                                       n_splits, scratch, window=window, sink=None if sink is None else _dev(sink, torch.float32), gate=_dev(g1, dt), out_scale=1.4)
            want = full[p] * pr.sigmoid(g1[0]) * 1.4
            err = np.abs(out.to(torch.float64).cpu().numpy()[0] - want).max()
            assert err <= 2.5e-2 * max(1.0, np.abs(full).max()), (p, n_splits, err)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, dim, vdim", [(2, 24, 40), (1, 72, 8), (2, 128, 64), (1, 256, 200), (2, 16, 32), (2, 64, 128), (1, 100, 50)])
def test_chunked_decay_attention_on_a_ragged_step(dtype, H, dim, vdim):
    """The chunk-by-chunk kernels on a step of four sequences of 163 (going on from a state that 37 tokens have left), 64, 65
    and 1 tokens, against the plain recurrence; the states they leave must be those the token-by-token kernel leaves."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(dim + vdim)
    decay = np.array([0.6, 0.999][:H], dtype=np.float32).astype(np.float64)
    lens = [200, 64, 65, 1]
    raw = [_rounded(rng.standard_normal((L, H * (2 * dim + vdim))), dtype) for L in lens]

    def split(x):
        return x[:, : H * dim], x[:, H * dim : 2 * H * dim], x[:, 2 * H * dim :]

    ref = []
    for x in raw:
        q, k, v = (pr.silu(t) for t in split(x))
        ref.append(pr.decayed_linear_attention(q.reshape(-1, H, dim), k.reshape(-1, H, dim), v.reshape(-1, H, vdim), decay).reshape(-1, H * vdim))
    dec = _dev(decay, torch.float32)
    states = {}
    for how in ("chunked", "plain"):
        state = torch.zeros((5, H, dim, vdim), dtype=torch.float32, device="cuda")
        q, k, v = split(_dev(raw[0][:37], dtype))
        ops.decay_attn(q, k, v, dec, state, _i32([3]), _i32([0, 37]), H, dim, vdim, silu=True)
        x = _dev(np.concatenate([raw[0][37:], raw[1], raw[2], raw[3]]), dtype)
        q, k, v = split(x)
        starts = _i32(np.concatenate([[0], np.cumsum([163, 64, 65, 1])]))
        kw = {}
        if how == "chunked":
            kw = dict(max_q_len=163, scratch=torch.full((ops.decay_attn_chunked_scratch_floats(4, 163, H, dim, vdim),), float("nan"), device="cuda"))
        out = ops.decay_attn(q, k, v, dec, state, _i32([3, 0, 4, 1]), starts, H, dim, vdim, silu=True, **kw).to(torch.float64).cpu().numpy()
        want = np.concatenate([ref[0][37:], ref[1], ref[2], ref[3]])
        # (in bfloat16 and up to size 128 the chunked outputs come from the tensor cores: q, k, v rounded after their activation)
        tol = 1.5e-2 if (how == "chunked" and dtype == torch.bfloat16 and max(dim, vdim) <= 128) else 5e-5
        assert np.abs(out - want).max() <= tol * max(1.0, np.abs(want).max()), how
        states[how] = state.cpu().numpy()
    # (up to size 128 the chunked kernels of a bfloat16 run take the values as bfloat16 after their activation)
    tol = 1e-2 if (dtype == torch.bfloat16 and max(dim, vdim) <= 128) else 5e-5
    assert np.abs(states["chunked"] - states["plain"]).max() <= tol * max(1.0, np.abs(states["plain"]).max())
    assert np.abs(states["chunked"][2]).max() == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [7, 96, 300])
def test_min_gru_in_stretches(dtype, width):
    """Sequences of 263 (going on from a state that 37 tokens have left), 129 and 5 tokens in one step, cut into stretches that
    run side by side, against the plain recurrence."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(width + 1)
    lens = [300, 129, 5]
    raw = [_rounded(2.0 * rng.standard_normal((L, 3 * width)), dtype) for L in lens]
    bz = rng.standard_normal(width).astype(np.float32).astype(np.float64)
    bx = rng.standard_normal(width).astype(np.float32).astype(np.float64)
    ref = [pr.min_gru(pr.sigmoid(x[:, :width] + bz), x[:, width : 2 * width] + bx) * pr.silu(x[:, 2 * width :]) for x in raw]
    state = torch.zeros((4, width), dtype=torch.float32, device="cuda")
    args = (_dev(bz, torch.float32), _dev(bx, torch.float32), state)
    x = _dev(raw[0][:37], dtype)
    ops.min_gru(x[:, :width], x[:, width : 2 * width], x[:, 2 * width :], *args, _i32([2]), _i32([0, 37]))
    x = _dev(np.concatenate([raw[0][37:], raw[1], raw[2]]), dtype)
    out = ops.min_gru(x[:, :width], x[:, width : 2 * width], x[:, 2 * width :], *args, _i32([2, 0, 3]), _i32([0, 263, 392, 397]), max_q_len=263)
    want = np.concatenate([ref[0][37:], ref[1], ref[2]])
    assert np.abs(out.to(torch.float64).cpu().numpy() - want).max() <= _tol(dtype, 2e-5, 1.5e-2) * max(1.0, np.abs(want).max())
    assert float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("M, N, K", [(3, 200, 128), (8, 4096, 1024), (200, 520, 256), (2048, 1024, 512), (20, 96, 68), (5, 64, 100)])
def test_products_with_the_squared_relu_in_their_epilogue(M, N, K):
    """`linear(..., act="relu2")` on every route it takes (the streaming kernel, the tcgen05 kernel, and the kernels behind which
    the activation is a pass of its own): the activation must see the 32-bit sums, and rows and columns beside the result stay."""
    from rusty_llama_b200.kernels.linear import linear

    rng = np.random.default_rng(M + N)
    x = _rounded(rng.standard_normal((M, K)), torch.bfloat16)
    w = _rounded(rng.standard_normal((N, K)) / np.sqrt(K), torch.bfloat16)
    out = linear(_dev(x, torch.bfloat16), _dev(w, torch.bfloat16), act="relu2").to(torch.float64).cpu().numpy()
    ref = np.maximum(x @ w.T, 0.0) ** 2
    assert out.shape == ref.shape
    assert np.abs(out - ref).max() <= 1.2e-2 * max(1.0, np.abs(ref).max())
    x32 = _dev(x, torch.float32)
    out32 = linear(x32, _dev(w, torch.float32), act="relu2").to(torch.float64).cpu().numpy()
    assert np.abs(out32 - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())
    from rusty_llama_b200.kernels import ops
    ops.tc_status_check()
