"""Vezatar through the library's own step function, cache and generation loop, against the plain float64
implementation of `plain_vezatar.py`, on small configurations made here (`vezatar_cases.py`).

32-bit runs: every schedule of a sequence (whole, cut into portions, token by token, inside a batch, in pages and slots
that were used before) must give the same bits, and those must lie within 32-bit rounding of the plain result.

bfloat16 runs are judged position by position (`check`).  Two things make them looser than a bfloat16 Llama.  Every
sublayer's result is normed before it is added, so it enters the stream at the stream's own size whatever its size was:
the relative error of a chain of roundings to 8 bits (2^-9 each, a dozen per sublayer) is carried into the stream
undamped, layer after layer, a few percent at the end.  And a token whose last chosen and first unchosen expert score
closer than that error may go to another expert, which changes its own logits much and those of later tokens a little:
a few positions of a hundred are allowed to differ by any amount."""

import numpy as np
import pytest
import torch

import plain_vezatar as pv
from helpers import check_logits
from vezatar_cases import CONFIGS, as_float64, random_weights, write_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, folder, float64 weights)."""
    out = {}
    for i, (name, make) in enumerate(CONFIGS.items()):
        cfg = make()
        w = random_weights(cfg, seed=11 + i)
        out[name] = (cfg, write_model(tmp_path_factory.mktemp(f"vez_{name}"), cfg, w), as_float64(w))
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
        check(run_cut(llm, toks, [n]), pv.forward(cfg, w, toks), dtype, f"{name}: prompt of {n}")


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_of_a_sequence_gives_the_same_bits_in_32_bit(models, name):
    """Whole, token by token from the first token on, and portions of 2, 3, 61, 64 and 7 tokens across page borders."""
    cfg, folder, w = models[name]
    toks = tokens(cfg, 140, 5)
    llm = load(folder, "float32")
    whole = run_cut(llm, toks, [140])
    check_logits(whole, pv.forward(cfg, w, toks), "float32", name)
    for cuts in ([], [2, 3, 61, 64, 7], [63, 2, 64], [1, 1, 126, 2]):
        got = run_cut(llm, toks, cuts)
        assert np.array_equal(got, whole), f"{name}: cut {cuts} changes bits, first at row {np.nonzero((got != whole).any(1))[0][:3]}"
    llm.engine.cache.check_consistent()


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_decoding_in_bfloat16(models, name):
    cfg, folder, w = models[name]
    toks = tokens(cfg, 100, 6)
    ref = pv.forward(cfg, w, toks)
    llm = load(folder, "bfloat16")
    for cuts in ([], [2, 62, 2, 30], [90]):
        check(run_cut(llm, toks, cuts), ref, "bfloat16", f"{name}: cut {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batch_with_leavers_and_reused_slots(models, name, dtype):
    """Three requests of unequal lengths start together and decode together; the shortest leaves first, a fourth
    starts in its slot and pages; each against itself alone (same bits in 32-bit) and against the plain model."""
    from rusty_llama_b200 import StepEntry

    cfg, folder, w = models[name]
    reqs = {"a": tokens(cfg, 131, 7), "b": tokens(cfg, 70, 8), "c": tokens(cfg, 3, 9), "d": tokens(cfg, 66, 10)}
    refs = {k: pv.forward(cfg, w, v) for k, v in reqs.items()}
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
    """300 tokens one by one after a prompt of 10: page borders at 64, 128, 192, 256 and the step from a page table of 4
    to one of 8; with and without CUDA graphs the 32-bit bits are equal."""
    cfg, folder, w = models["a"]
    toks = tokens(cfg, 310, 12)
    ref = pv.forward(cfg, w, toks)
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
            logits = pv.forward(cfg, w, seq)[-1]
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
    ref = {"a": pv.forward(cfg, w, a), "b": pv.forward(cfg, w, b)}
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
        # forty requests of two tokens each: far fewer tokens than --max-tokens, but forty pages
        many = [tokens(cfg, 2, 100 + i) for i in range(40)]
        out = run.step([(f"m{i}", t, [1]) for i, t in enumerate(many)], end=[f"m{i}" for i in range(40)])
        for i, t in enumerate(many):
            check(out[i : i + 1], pv.forward(cfg, w, t)[1:], dtype, f"short request {i}")
    finally:
        run.close()
    if dtype == "float32":
        out = subprocess.run(
            [sys.executable, os.path.join(REPO, "bin", "rusty_llama"), folder, "-t", "0", "-n", "12", "-i", " ".join(map(str, b)), "--dtype", "float32"],
            capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        ids = [int(t) for t in out.stdout.split()]
        assert len(ids) == 12 - len(b) or ids[: len(b)] == b  # the new ids alone, or the prompt and the new ids
        new = ids[-(12 - len(b)):]
        seq = list(b)
        for t in new:
            logits = pv.forward(cfg, w, seq)[-1]
            best = np.sort(logits)[-2:]
            if best[1] - best[0] > 1e-3 * np.abs(logits).max():
                assert int(np.argmax(logits)) == t
            seq.append(t)


# ------------------------------------------------------------------ mechanisms alone
def _dev(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to("cuda", dtype)


def _rounded(a, dtype):
    return _dev(a, dtype).to(torch.float64).cpu().numpy()


def _paged(rows, dtype, n_pages, page_order):
    """rows [L, D] laid into pages in the given order of page ids; returns (pages [n_pages, 1, 64, D], table [1, width])."""
    L, D = rows.shape
    pages = torch.full((n_pages, 1, 64, D), 7.0, dtype=dtype, device="cuda")  # what lies in unused places is finite junk
    width = (L + 63) // 64
    for i in range(width):
        part = rows[i * 64 : (i + 1) * 64]
        pages[page_order[i], 0, : part.shape[0]] = _dev(part, dtype)
    return pages, torch.tensor([page_order[:width]], dtype=torch.int32, device="cuda")


def _plain_latent_attn(q, rows, pos, rank, sink, scale, window=0):
    """q [H, rank + rot], rows [L, rank + rot] -> [H, rank]: softmax with a sink over keys first..pos."""
    first = max(0, pos + 1 - window) if window else 0
    out = np.zeros((q.shape[0], rank))
    for h in range(q.shape[0]):
        s = rows[first : pos + 1] @ q[h] * scale
        top = max(s.max(), sink[h])
        e = np.exp(s - top)
        out[h] = (e / (e.sum() + np.exp(sink[h] - top))) @ rows[first : pos + 1, :rank]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_finds_one_far_key_among_hundreds(dtype):
    """One cached row far back is made to fit one head's query: that head's result must be that row's latent (almost
    all of the probability), the other heads' must not; pages are in shuffled order; queries stand at positions around
    the page borders."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(3)
    rank, rot, H, L = 40, 8, 3, 64 * 5
    rows = _rounded(rng.standard_normal((L, rank + rot)), dtype)
    sink = rng.standard_normal(H)
    order = [4, 0, 3, 1, 2]
    for far, positions in ((2, (255, 256, 319)), (63, (63, 64, 65, 128)), (64, (64, 127, 191, 192)), (0, (0, 1, 300))):
        q = _rounded(0.1 * rng.standard_normal((len(positions), H, rank + rot)), dtype)
        q[:, 1] = _rounded(rows[far] * 2.0, dtype)  # head 1 scores the far key with 2 |row|^2, about 100
        pages, table = _paged(rows, dtype, 6, order)
        pos_t = torch.tensor(positions, dtype=torch.int32, device="cuda")
        seq_t = torch.zeros(len(positions), dtype=torch.int32, device="cuda")
        out = ops.latent_attn(_dev(q, dtype), pages, table, seq_t, pos_t, _dev(sink, torch.float32), rank, rot, 1.0)
        out = out.to(torch.float64).cpu().numpy()
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for i, pos in enumerate(positions):
            ref = _plain_latent_attn(q[i], rows, pos, rank, sink, 1.0)
            assert np.abs(out[i] - ref).max() <= tol * max(1.0, np.abs(ref).max()), (far, pos)
            if pos >= far:
                assert np.abs(out[i, 1] - rows[far, :rank]).max() < 0.05, (far, pos)


@pytest.mark.parametrize("rank, rot, H", [(64, 16, 4), (128, 32, 16), (512, 64, 16), (256, 0, 3), (64, 48, 40)])
def test_tensor_core_latent_attention_prompts_decoding_and_splits(rank, rot, H):
    """The tensor-core kernel on a ragged step (a sequence that goes on from position 70 with 37 tokens, one that starts
    with 3, one that brings a single token at position 200), then on single tokens with the key range cut into parts;
    in every case one head's query is made to fit a far key, and the plain kernel must agree as well."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(rank + rot)
    dt, Dk = torch.bfloat16, rank + rot
    lens = [(70, 37), (0, 3), (200, 1)]  # (positions held, tokens brought)
    n_pages, width = 16, 4
    perm = rng.permutation(n_pages)
    table = np.zeros((3, width), dtype=np.int32)
    pages = torch.full((n_pages, 1, 64, Dk), 3.0, dtype=dt, device="cuda")
    rows_of, at = [], 0
    for s, (held, n) in enumerate(lens):
        L = held + n
        rows = _rounded(rng.standard_normal((L, Dk)), dt)
        rows_of.append(rows)
        for i in range((L + 63) // 64):
            table[s, i] = perm[at]
            part = rows[i * 64 : (i + 1) * 64]
            pages[perm[at], 0, : part.shape[0]] = _dev(part, dt)
            at += 1
    T = sum(n for _, n in lens)
    q = _rounded(0.1 * rng.standard_normal((T, H, Dk)), dt)
    far = [5, 0, 64]
    tok_seq = np.concatenate([np.full(n, s) for s, (_, n) in enumerate(lens)]).astype(np.int32)
    tok_pos = np.concatenate([np.arange(held, held + n) for held, n in lens]).astype(np.int32)
    for t in range(T):
        q[t, H - 1] = _rounded(rows_of[tok_seq[t]][far[tok_seq[t]]] * (60.0 / Dk), dt)
    sink = rng.standard_normal(H)
    start = np.concatenate([[0], np.cumsum([n for _, n in lens])]).astype(np.int32)
    args = (_dev(q, dt), pages, torch.from_numpy(table).cuda())
    sink_t = _dev(sink, torch.float32)
    out = ops.latent_attn_mma(*args, torch.from_numpy(start).cuda(), torch.tensor([h for h, _ in lens], dtype=torch.int32, device="cuda"),
                              max(n for _, n in lens), sink_t, rank, rot, 0.5).double().cpu().numpy()
    plain = ops.latent_attn(*args, torch.from_numpy(tok_seq).cuda(), torch.from_numpy(tok_pos).cuda(), sink_t, rank, rot, 0.5).double().cpu().numpy()
    for t in range(T):
        ref = _plain_latent_attn(q[t], rows_of[tok_seq[t]], tok_pos[t], rank, sink, 0.5)
        assert np.abs(out[t] - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max()), (t, np.abs(out[t] - ref).max())
        assert np.abs(plain[t] - ref).max() <= 2e-2 * max(1.0, np.abs(ref).max())
        assert np.abs(out[t, H - 1] - rows_of[tok_seq[t]][far[tok_seq[t]], :rank]).max() < 0.06
    # single tokens, key range in parts (more parts than pages included)
    last = np.array([start[1] - 1, start[2] - 1, start[3] - 1])
    qd = _dev(q[last], dt)
    pos_d = torch.tensor([lens[s][0] + lens[s][1] - 1 for s in range(3)], dtype=torch.int32, device="cuda")
    for n_splits in (1, 2, 3, 7):
        scratch = torch.full((ops.latent_attn_mma_scratch_floats(3 * H, rank, n_splits) + 1,), float("nan"), device="cuda")
        got = ops.latent_attn_mma(qd, pages, args[2], torch.arange(4, dtype=torch.int32, device="cuda"), pos_d, 1, sink_t, rank, rot, 0.5,
                                  n_splits=n_splits, scratch=scratch).double().cpu().numpy()
        assert np.abs(got - out[last]).max() <= 1e-2 * max(1.0, np.abs(out).max()), n_splits


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_sink_and_window_edges(dtype):
    """A sink far above every score takes all the probability (the result is near zero), one far below changes nothing;
    with a window, a standing-out key counts while it is the last one inside and no longer one position later."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(4)
    rank, rot, H, L = 24, 4, 2, 200
    rows = _rounded(rng.standard_normal((L, rank + rot)), dtype)
    pages, table = _paged(rows, dtype, 4, [1, 3, 0, 2])
    q = _rounded(0.2 * rng.standard_normal((1, H, rank + rot)), dtype)
    pos_t = torch.tensor([150], dtype=torch.int32, device="cuda")
    seq_t = torch.zeros(1, dtype=torch.int32, device="cuda")
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for sink in (np.array([40.0, -40.0]), np.array([0.3, -0.2])):
        out = ops.latent_attn(_dev(q, dtype), pages, table, seq_t, pos_t, _dev(sink, torch.float32), rank, rot, 0.7).to(torch.float64).cpu().numpy()
        ref = _plain_latent_attn(q[0], rows, 150, rank, sink, 0.7)
        assert np.abs(out[0] - ref).max() <= tol
        if sink[0] > 30:
            assert np.abs(out[0, 0]).max() < 1e-6 and np.abs(out[0, 1]).max() > 1e-2
    none = ops.latent_attn(_dev(q, dtype), pages, table, seq_t, pos_t, None, rank, rot, 0.7).to(torch.float64).cpu().numpy()
    assert np.abs(none[0] - _plain_latent_attn(q[0], rows, 150, rank, np.array([-1e30, -1e30]), 0.7)).max() <= tol
    window, key = 70, 90
    q[0, 0] = _rounded(rows[key] * 2.0, dtype)
    for pos in (key + window - 1, key + window):  # the key is the first inside, then the first outside
        pos_t = torch.tensor([pos], dtype=torch.int32, device="cuda")
        out = ops.latent_attn(_dev(q, dtype), pages, table, seq_t, pos_t, _dev(np.zeros(H), torch.float32), rank, rot, 1.0, window=window)
        out = out.to(torch.float64).cpu().numpy()
        ref = _plain_latent_attn(q[0], rows, pos, rank, np.zeros(H), 1.0, window=window)
        assert np.abs(out[0] - ref).max() <= tol * max(1.0, np.abs(ref).max())
        inside = np.abs(out[0, 0] - rows[key, :rank]).max() < 0.05
        assert inside == (pos == key + window - 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prep_norms_rotates_and_stores(dtype):
    """The latent's norm, the rotation (scaled frequencies, magnitude, pairs of neighbours, a rotated part longer than
    the rotated dimensions) and the place in the pages, for tokens of two sequences at scattered positions."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(5)
    H, dim, rot, rank, dims = 3, 12, 12, 20, 8
    scaling = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}
    f, mag = pv.yarn_frequencies(dims, 10000.0, scaling)
    pos = np.array([0, 1, 63, 64, 500, 129])
    seq = np.array([0, 0, 0, 1, 1, 0])
    T = len(pos)
    q = _rounded(rng.standard_normal((T, H * (dim + rot))), dtype)
    kv = _rounded(rng.standard_normal((T, rank + rot)), dtype)
    w = 1.0 + 0.3 * rng.standard_normal(rank)
    w32 = _dev(w, torch.float32)
    table = torch.tensor([[3, 5, 1, 0, 0, 0, 0, 0], [2, 4, 6, 7, 8, 9, 10, 11]], dtype=torch.int32, device="cuda")
    pages = torch.zeros((12, 1, 64, rank + rot), dtype=dtype, device="cuda")
    q_cat = torch.zeros((T, H, rank + rot), dtype=dtype, device="cuda")
    ops.latent_prep(_dev(q, dtype), _dev(kv, dtype), w32, 1e-5, _dev(f, torch.float32), dims // 2, mag,
                    torch.tensor(pos, dtype=torch.int32, device="cuda"), torch.tensor(seq, dtype=torch.int32, device="cuda"),
                    table, pages, q_cat, H, dim, rot, rank)
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    c = pv.rms_norm(kv[:, :rank], w32.double().cpu().numpy(), 1e-5)
    kr = pv.rotate_pairs(kv[:, rank:], pos, f, mag)
    qr = pv.rotate_pairs(q.reshape(T, H, dim + rot)[:, :, dim:], pos, f, mag)
    tab = table.cpu().numpy()
    for t in range(T):
        row = pages[tab[seq[t], pos[t] // 64], 0, pos[t] % 64].to(torch.float64).cpu().numpy()
        assert np.abs(row[:rank] - c[t]).max() <= tol * np.abs(c[t]).max()
        assert np.abs(row[rank:] - kr[t]).max() <= tol * np.abs(kr[t]).max()
        assert np.array_equal(row[rank + dims :], kv[t, rank + dims :])  # beyond the rotated dimensions: unchanged
    got = q_cat[:, :, rank:].to(torch.float64).cpu().numpy()
    assert np.abs(got - qr).max() <= tol * np.abs(qr).max()
    assert int((pages != 0).any(dim=-1).sum()) == T  # nothing else was written


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_linear_with_and_without_gate(dtype):
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(6)
    # (rows whose starts are 16-byte aligned go to the tensor cores in bfloat16, the others to the plain kernel)
    for M, H, N, K, pad in ((1, 3, 20, 12, 3), (70, 2, 65, 33, 3), (5, 5, 8, 64, 3), (5, 5, 8, 64, 0), (200, 3, 130, 72, 8), (33, 2, 64, 8, 0)):
        x = _rounded(rng.standard_normal((M, H * K + pad)), dtype)
        w = _rounded(rng.standard_normal((H, N, K)), dtype)
        g = _rounded(rng.standard_normal((M, H * N)), dtype)
        ref = np.einsum("mhk,hnk->mhn", x[:, : H * K].reshape(M, H, K), w)
        for gate in (None, g):
            out = torch.full((M, H * N + 2), float("nan"), dtype=dtype, device="cuda")
            ops.head_linear(_dev(x, dtype), K, _dev(w, dtype), out, N, gate=None if gate is None else _dev(gate, dtype), gate_head_stride=N)
            want = ref if gate is None else ref * pv.sigmoid(g.reshape(M, H, N))
            got = out[:, : H * N].to(torch.float64).cpu().numpy().reshape(M, H, N)
            tol = 1e-5 if dtype == torch.float32 else 1e-2
            assert np.abs(got - want).max() <= tol * np.abs(want).max()
            assert torch.isnan(out[:, H * N :]).all()


def test_router_choice_weights_and_gate():
    """The bias chooses and does not weigh; ties are not tested; one more row gives the shared expert's gate."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(7)
    for E, top, d, T in ((5, 2, 48, 9), (3, 3, 20, 4), (64, 6, 96, 33), (7, 1, 33, 2)):
        x = rng.standard_normal((T, d))
        W = {"router": 2.0 * rng.standard_normal((E, d)) / np.sqrt(d), "correction": 0.5 * rng.standard_normal(E)}
        sg = rng.standard_normal((1, d)) / np.sqrt(d)
        chosen, weights, s = pv.router(_rounded(x, torch.float32), {k: _rounded(v, torch.float32) for k, v in W.items()}, "", top)
        w_all = _dev(np.concatenate([W["router"], sg]), torch.float32)
        ids, wts, gate = ops.moe_router(_dev(x, torch.float32), w_all, _dev(W["correction"], torch.float32), E, top)
        assert np.array_equal(ids.cpu().numpy(), chosen)
        assert np.abs(wts.cpu().numpy() - weights).max() < 1e-6
        assert np.abs(gate.cpu().numpy() - pv.sigmoid(_rounded(x, torch.float32) @ _rounded(sg, torch.float32).T)[:, 0]).max() < 1e-6
        # without a bias the choice is by score alone, and the weights may be renormalised
        ids2, wts2, none = ops.moe_router(_dev(x, torch.float32), _dev(W["router"], torch.float32), None, E, top, renormalize=True)
        assert none is None
        assert np.array_equal(ids2.cpu().numpy(), np.argsort(-s, axis=-1, kind="stable")[:, :top])
        assert np.abs(wts2.cpu().numpy().sum(-1) - 1.0).max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_plan_products_and_sum(dtype):
    """Every (token, choice) pair lands in exactly one row of exactly one tile of its expert; experts nobody chose and
    experts everybody chose; the weighted sum in the order of the choices."""
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(8)
    for E, top, d, ff, T in ((6, 2, 40, 24, 100), (4, 4, 16, 8, 3), (9, 1, 24, 70, 1), (3, 2, 32, 16, 77)):
        x = _rounded(rng.standard_normal((T, d)), dtype)
        ids = np.stack([rng.permutation(E if E != 6 else 4)[:top] for _ in range(T)]).astype(np.int32)  # E = 6: experts 4 and 5 get nobody
        wts = rng.random((T, top))
        wg, wu = (_rounded(rng.standard_normal((E, ff, d)) / np.sqrt(d), dtype) for _ in range(2))
        wd = _rounded(rng.standard_normal((E, d, ff)) / np.sqrt(ff), dtype)
        ids_t = torch.from_numpy(ids).cuda()
        for tile_rows in ((0,) if dtype == torch.float32 else (0, 32, 128)):  # 0: the plain products' own height
            if tile_rows == 128 and (d % 8 or ff % 8):
                continue  # rows that cannot be moved in 16-byte pieces stay with the plain products and their height
            order, place, tiles, max_tiles = ops.moe_plan(ids_t, E, tile_rows)
            o, p, tl = order.cpu().numpy(), place.cpu().numpy(), tiles.cpu().numpy()
            assert sorted(o.tolist()) == list(range(T * top)) and np.array_equal(o[p], np.arange(T * top))
            assert np.array_equal(np.sort(ids.reshape(-1)[o]), ids.reshape(-1)[o])  # expert after expert
            covered = np.zeros(T * top, dtype=int)
            assert tl[0] <= max_tiles
            for i in range(tl[0]):
                e, r0, n = tl[1 + 3 * i : 4 + 3 * i]
                assert 0 < n <= (tile_rows or ops.moe_tile_rows()) and (ids.reshape(-1)[o[r0 : r0 + n]] == e).all()
                covered[r0 : r0 + n] += 1
            assert (covered == 1).all()
            h = ops.moe_gemm(_dev(x, dtype), _dev(wg, dtype), tiles, max_tiles, T * top, order=order, gather_div=top, w2=_dev(wu, dtype), tile_rows=tile_rows)
            y = ops.moe_gemm(h, _dev(wd, dtype), tiles, max_tiles, T * top, out_dtype=torch.float32, tile_rows=tile_rows)
            out = ops.moe_combine(y, place, _dev(wts, torch.float32), None, None).to(torch.float64).cpu().numpy()
            ref = np.zeros((T, d))
            for t in range(T):
                for j in range(top):
                    e = ids[t, j]
                    a = wg[e] @ x[t]
                    hh = a * pv.sigmoid(a) * (wu[e] @ x[t])
                    if dtype == torch.bfloat16:
                        hh = _rounded(hh, dtype)
                    ref[t] += np.float32(wts[t, j]) * (wd[e] @ hh)
            tol = 2e-5 if dtype == torch.float32 else 1e-2
            assert np.abs(out - ref).max() <= tol * max(1.0, np.abs(ref).max())


def test_gate_up_product_with_the_clamped_activation():
    """The activation with limits in the epilogue of every bfloat16 gate/up product: the streaming kernels of a decode
    step (3 rows), the tensor-core kernel of a prompt step (200 rows), and the plain kernel for a k that is no multiple of 8."""
    from rusty_llama_b200.kernels.linear import linear_swiglu

    rng = np.random.default_rng(10)
    dt = torch.bfloat16
    for M, K, ff in ((3, 256, 96), (3, 72, 40), (200, 256, 320), (40, 128, 64), (5, 100, 24)):
        x = _rounded(rng.standard_normal((M, K)), dt)
        wg, wu = (_rounded(2.0 * rng.standard_normal((ff, K)) / np.sqrt(K), dt) for _ in range(2))
        w = torch.stack([_dev(wg, dt), _dev(wu, dt)], dim=1).reshape(2 * ff, K).contiguous()  # rows alternate gate, up
        for alpha, limit in ((1.702, 1.0), (1.0, 0.5)):
            got = linear_swiglu(_dev(x, dt), w, act=(alpha, limit)).double().cpu().numpy()
            g, u = np.minimum(x @ wg.T, limit), np.clip(x @ wu.T, -limit, limit)
            ref = g * pv.sigmoid(alpha * g) * (u + 1.0)
            assert np.abs(got - ref).max() <= 1e-2 * max(1.0, np.abs(ref).max()), (M, K, ff, alpha)
        got = linear_swiglu(_dev(x, dt), w).double().cpu().numpy()
        g, u = x @ wg.T, x @ wu.T
        assert np.abs(got - g * pv.sigmoid(g) * u).max() <= 1.2e-2 * np.abs(g * u).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_normed_sum_and_clamped_gate(dtype):
    from rusty_llama_b200.kernels import ops

    rng = np.random.default_rng(9)
    for T, d in ((3, 68), (70, 256), (1, 1000)):
        x = rng.standard_normal((T, d)).astype(np.float32)
        delta = _rounded(3.0 * rng.standard_normal((2, T, d)), dtype)
        wd, w = (_rounded(1.0 + 0.2 * rng.standard_normal(d), dtype) for _ in range(2))
        xt = torch.from_numpy(x.copy()).cuda()
        out = ops.normed_add_rmsnorm(xt, _dev(delta, dtype), _dev(wd, dtype), 1e-5, _dev(w, dtype), 1e-6, dtype)
        v = x.astype(np.float64) + pv.rms_norm(delta.sum(0), wd, 1e-5)
        assert np.abs(xt.double().cpu().numpy() - v).max() <= 2e-6 * np.abs(v).max()
        ref = pv.rms_norm(v, w, 1e-6)
        tol = 2e-6 if dtype == torch.float32 else 8e-3
        assert np.abs(out.double().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
        rows = torch.tensor([T - 1], dtype=torch.int32, device="cuda")
        xt2 = torch.from_numpy(x.copy()).cuda()
        part = ops.normed_add_rmsnorm(xt2, _dev(delta, dtype), _dev(wd, dtype), 1e-5, _dev(w, dtype), 1e-6, dtype, rows=rows, write_x=False)
        assert torch.equal(part[0], out[T - 1]) and torch.equal(xt2, torch.from_numpy(x).cuda())
    gu = _rounded(2.0 * rng.standard_normal((5, 2 * 37)), dtype)
    for alpha, limit in ((1.702, 1.0), (1.0, 0.25)):
        got = ops.clamped_glu(_dev(gu, dtype), alpha, limit).double().cpu().numpy()
        g, u = np.minimum(gu[:, :37], limit), np.clip(gu[:, 37:], -limit, limit)
        ref = g * pv.sigmoid(alpha * g) * (u + 1.0)
        assert np.abs(got - ref).max() <= (1e-6 if dtype == torch.float32 else 8e-3) * max(1.0, np.abs(ref).max())
