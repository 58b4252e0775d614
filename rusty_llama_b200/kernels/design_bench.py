"""Vezatar beside Llama at equal sizes: prompt-step and decode-step throughput through the engine, and every kernel that
only Vezatar uses timed alone beside the Llama kernel that does the like work.

    python bench.py --design vezatar [--design-sizes small,lite,wide]

Sizes resemble real models' layers (random weights, a few layers, the whole vocabulary): the width, head count, layer count
and vocabulary of the two models are equal; Llama's feed-forward has the size of Vezatar's dense one.  Every kernel's
fraction is what it must move (bytes, against the measured copy rate) or compute (flops, against the measured bfloat16
matrix rate), whichever bound is the tighter one, divided by the time it took.
"""

from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Dict

import torch

from . import microbench as mb
from . import ops

SIZES = {
    # width, heads, dim, rot, vdim, rank, dense ff, experts, top, expert ff, shared ff, vocabulary
    "small": dict(width=1024, heads=8, dim=64, rot=32, vdim=64, rank=256, ff=4096, experts=16, top=2, eff=1024, sff=1024, vocab=32000),
    "lite": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, rank=512, ff=8192, experts=64, top=6, eff=1408, sff=2816, vocab=32000),
    "wide": dict(width=4096, heads=32, dim=128, rot=64, vdim=128, rank=512, ff=12288, experts=32, top=4, eff=2048, sff=2048, vocab=32000),
}
LAYERS = 4


def vezatar_config(z: dict) -> dict:
    rot = {"base": 10000.0, "dims": z["rot"], "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}

    def mixer(kv_from=None):
        m = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["rank"], "rot": rot,
             "scale": 1.0 / math.sqrt(z["dim"] + z["rot"])}
        if kv_from is not None:
            m["kv_from"] = kv_from
        return m

    dense = {"kind": "dense", "ff": z["ff"], "limit": 7.0}
    moe = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["eff"]}, "shared": {"ff": z["sff"]}}
    layers = []
    for i in range(LAYERS):  # a layer with a latent of its own and a dense feed-forward, then one that reads its cache and routes
        layers.append({"type": "latent_attention", "mixer": mixer(None if i % 2 == 0 else i - 1), "mlp": dense if i % 2 == 0 else moe})
    return {"architecture": "Vezatar", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "layers": layers}


def llama_config(z: dict) -> dict:
    return {
        "architectures": ["LlamaForCausalLM"], "tie_word_embeddings": False, "torch_dtype": "bfloat16", "hidden_size": z["width"],
        "intermediate_size": z["ff"], "num_hidden_layers": LAYERS, "num_attention_heads": z["heads"], "num_key_value_heads": z["heads"],
        "head_dim": z["vdim"], "vocab_size": z["vocab"], "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "rope_scaling": None,
    }


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def step_times(cfg: dict, T: int, batch: int, ctx: int, steps: int, warmup: int) -> Dict[str, float]:
    """Milliseconds of a prompt step of T tokens (one sequence) and of a decode step of `batch` sequences near position ctx."""
    from .. import StepEntry, load_random

    llm = load_random(cfg, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=batch * (ctx + 64 * 4) + T + 64, max_seqs=batch + 1)
    V = cfg.get("vocab", cfg.get("vocab_size"))
    gen = torch.Generator().manual_seed(0)
    toks = lambda n: torch.randint(0, V, (n,), generator=gen).tolist()  # noqa: E731
    prefill = []
    for i in range(warmup + 3):
        s = llm.open_sequence()
        e0, e1 = _events()
        torch.cuda.synchronize()
        e0.record()
        llm.step([StepEntry(s, toks(T), [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        llm.close_sequence(s)
        if i >= warmup:
            prefill.append(e0.elapsed_time(e1))
    slots = [llm.open_sequence() for _ in range(batch)]
    for s in slots:  # fill the context sequence by sequence, in pieces that bound the activations
        left = ctx - steps - warmup - 2
        while left > 0:
            n = min(left, 4096)
            llm.step([StepEntry(s, toks(n), [])])
            left -= n
    for _ in range(warmup + 2):  # the plain run and the capture come first
        llm.step([StepEntry(s, toks(1), [0]) for s in slots], borrow=True)
    e0, e1 = _events()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        llm.step([StepEntry(s, toks(1), [0]) for s in slots], borrow=True)
    e1.record()
    torch.cuda.synchronize()
    llm.engine.check_device_status()
    out = {"prefill_ms": sorted(prefill)[len(prefill) // 2], "decode_ms": e0.elapsed_time(e1) / steps}
    del llm
    torch.cuda.empty_cache()
    return out


def _frac(us: float, nbytes: float, flops: float, peaks: dict) -> float:
    """The tighter of the two bounds over the time taken."""
    bound_us = max(nbytes / (peaks["hbm_gbs"] * 1e3), flops / (peaks["bf16_tflops"] * 1e6))
    return round(bound_us / us, 3)


def kernel_table(z: dict, T: int, batch: int, ctx: int, peaks: dict) -> Dict[str, dict]:
    """Each kernel of the design alone, at a prompt step of T tokens and a decode step of `batch` sequences at `ctx`."""
    dev, bf = "cuda:0", torch.bfloat16
    H, dim, rot, vdim, rank, d = z["heads"], z["dim"], z["rot"], z["vdim"], z["rank"], z["width"]
    Dk = rank + rot
    out: Dict[str, dict] = {}
    it = dict(iters=10, warmup=2)

    def note(name, us, nbytes, flops, like=None):
        out[name] = {"us": round(us, 1), "frac": _frac(us, nbytes, flops, peaks)}
        if like:
            out[name]["like"] = like

    # ---- attention: prompt
    pages_n = (T + 63) // 64
    pages = torch.randn(pages_n, 1, 64, Dk, device=dev, dtype=bf)
    table = torch.randperm(pages_n, device=dev).to(torch.int32).view(1, -1).contiguous()
    q_cat = torch.randn(T, H, Dk, device=dev, dtype=bf)
    sink = torch.zeros(H, device=dev)
    start = torch.tensor([0, T], dtype=torch.int32, device=dev)
    pos0 = torch.zeros(1, dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(dim + rot)
    us = mb._time(lambda i: ops.latent_attn_mma(q_cat, pages, table, start, pos0, T, sink, rank, rot, scale), 1, **it)
    flops = 2.0 * T * T / 2 * H * (Dk + rank)
    r = mb.bench_flash_prefill(SimpleNamespace(tokens=T, impl="auto", heads=H, kv_heads=H, head_dim=vdim, splits=0, **it))
    note("prefill_latent_attention", us, 0, flops, like={"kernel": r["kernel"], "us": r["us"], "frac": round(r["causal_TFLOPs"] / peaks["bf16_tflops"], 3)})
    out["prefill_latent_attention"]["TFLOPs"] = round(flops / us / 1e6, 1)
    # ---- attention: decode
    per_seq = (ctx + 63) // 64
    nv = min(mb._copies(batch * ctx * Dk * 2), 16)
    pools = [torch.randn(batch * per_seq, 1, 64, Dk, device=dev, dtype=bf) for _ in range(nv)]
    table = torch.randperm(batch * per_seq, device=dev).to(torch.int32).view(batch, per_seq).contiguous()
    qd = torch.randn(batch, H, Dk, device=dev, dtype=bf)
    startd = torch.arange(batch + 1, dtype=torch.int32, device=dev)
    posd = torch.full((batch,), ctx - 1, dtype=torch.int32, device=dev)
    blocks = batch * ((H + 31) // 32 if H > 16 else 1)
    n_splits = max(1, min(148 // blocks, per_seq // 2, 64))
    scratch = torch.empty(max(1, ops.latent_attn_mma_scratch_floats(batch * H, rank, n_splits)), device=dev)
    us = mb._time(lambda i: ops.latent_attn_mma(qd, pools[i], table, startd, posd, 1, sink, rank, rot, scale, n_splits=n_splits, scratch=scratch), nv, **it)
    r = mb.bench_attn_decode(SimpleNamespace(seqs=batch, ctx=ctx, impl="auto", heads=H, kv_heads=H, head_dim=vdim, splits=0, **it))
    note("decode_latent_attention", us, batch * ctx * Dk * 2, 2.0 * batch * ctx * H * (Dk + rank),
         like={"kernel": "attn_decode", "us": r["us"], "frac": round(r["GBps"] / peaks["hbm_gbs"], 3)})
    out["decode_latent_attention"]["cache_bytes_vs_like"] = round(Dk / (2.0 * H * vdim), 4)
    del pools
    # ---- the two per-head maps, norm + rotation + cache write
    for rows, tag in ((T, "prefill"), (batch, "decode")):
        qp = torch.randn(rows, H * (dim + rot) + H * vdim + Dk, device=dev, dtype=bf)
        w_uk = torch.randn(H, rank, dim, device=dev, dtype=bf)
        w_uv = torch.randn(H, vdim, rank, device=dev, dtype=bf)
        qc = torch.empty(rows, H * Dk, device=dev, dtype=bf)
        o_lat = torch.randn(rows, H * rank, device=dev, dtype=bf)
        a = torch.empty(rows, H * vdim, device=dev, dtype=bf)
        gate = qp[:, H * (dim + rot): H * (dim + rot) + H * vdim]
        us = mb._time(lambda i: ops.head_linear(qp, dim + rot, w_uk, qc, Dk), 1, **it)
        note(f"{tag}_query_to_latent", us, (w_uk.numel() + rows * H * (dim + rank)) * 2, 2.0 * rows * H * dim * rank)
        us = mb._time(lambda i: ops.head_linear(o_lat, rank, w_uv, a, vdim, gate=gate, gate_head_stride=vdim), 1, **it)
        note(f"{tag}_latent_to_value_gated", us, (w_uv.numel() + rows * H * (rank + 2 * vdim)) * 2, 2.0 * rows * H * vdim * rank)
        pg = torch.zeros(max(1, (rows + 63) // 64) + 1, 1, 64, Dk, device=dev, dtype=bf)
        tb = torch.arange(pg.shape[0], dtype=torch.int32, device=dev).view(1, -1)
        tp = torch.arange(rows, dtype=torch.int32, device=dev) if rows > batch else torch.zeros(rows, dtype=torch.int32, device=dev)
        ts = torch.zeros(rows, dtype=torch.int32, device=dev)
        freq = torch.rand(rot // 2, device=dev)
        nw = torch.ones(rank, device=dev)
        kv = qp[:, qp.shape[1] - Dk:]
        us = mb._time(lambda i: ops.latent_prep(qp, kv, nw, 1e-5, freq, rot // 2, 1.1, tp, ts, tb, pg, qc.view(rows, H, Dk), H, dim, rot, rank), 1, **it)
        note(f"{tag}_norm_rotate_store", us, rows * (2 * H * rot + 2 * Dk) * 2, 0)
    # ---- sandwich norm
    for rows, tag in ((T, "prefill"), (batch, "decode")):
        x = torch.randn(rows, d, device=dev)
        delta = torch.randn(rows, d, device=dev, dtype=bf)
        w1, w2 = torch.ones(d, device=dev, dtype=bf), torch.ones(d, device=dev, dtype=bf)
        us = mb._time(lambda i: ops.normed_add_rmsnorm(x, delta, w1, 1e-5, w2, 1e-5, bf), 1, **it)
        us_like = mb._time(lambda i: ops.add_rmsnorm(x, delta, w2, 1e-5, bf), 1, **it)
        nbytes = rows * d * (4 + 4 + 2 + 2)
        note(f"{tag}_normed_add_norm", us, nbytes, 0, like={"kernel": "add_rmsnorm", "us": round(us_like, 1), "frac": _frac(us_like, nbytes, 0, peaks)})
    # ---- dense feed-forward's activation (Llama's is fused into its product)
    for rows, tag in ((T, "prefill"), (batch, "decode")):
        gu = torch.randn(rows, 2 * z["ff"], device=dev, dtype=bf)
        us = mb._time(lambda i: ops.clamped_glu(gu, 1.702, 7.0), 1, **it)
        note(f"{tag}_clamped_gate", us, rows * 3 * z["ff"] * 2, 0)
    # ---- routed feed-forward
    E, top, eff = z["experts"], z["top"], z["eff"]
    wg, wu = (torch.randn(E, eff, d, device=dev, dtype=bf) * 0.02 for _ in range(2))
    wd = torch.randn(E, d, eff, device=dev, dtype=bf) * 0.02
    wr = torch.randn(E + 1, d, device=dev)
    bias = torch.zeros(E, device=dev)
    for rows, tag in ((T, "prefill"), (batch, "decode")):
        x = torch.randn(rows, d, device=dev, dtype=bf)
        us = mb._time(lambda i: ops.moe_router(x, wr, bias, E, top), 1, **it)
        note(f"{tag}_router", us, (E + 1) * d * 4 + rows * d * 2, 0)
        ids, wts, gate = ops.moe_router(x, wr, bias, E, top)
        us = mb._time(lambda i: ops.moe_plan(ids, E, 128 if rows * top >= 64 * E else 32), 1, **it)
        note(f"{tag}_plan", us, rows * top * 12, 0)
        tile_rows = 128 if rows * top >= 64 * E else 32  # as `RoutedExperts.forward` chooses
        order, place, tiles, max_tiles = ops.moe_plan(ids, E, tile_rows)
        used = int(torch.unique(ids).numel())
        us = mb._time(lambda i: ops.moe_gemm(x, wg, tiles, max_tiles, rows * top, order=order, gather_div=top, w2=wu, tile_rows=tile_rows), 1, **it)
        note(f"{tag}_experts_gate_up", us, (2 * used * eff * d + rows * d + rows * top * eff) * 2, 4.0 * rows * top * eff * d)
        h = ops.moe_gemm(x, wg, tiles, max_tiles, rows * top, order=order, gather_div=top, w2=wu, tile_rows=tile_rows)
        us = mb._time(lambda i: ops.moe_gemm(h, wd, tiles, max_tiles, rows * top, out_dtype=torch.float32, tile_rows=tile_rows), 1, **it)
        note(f"{tag}_experts_down", us, (used * eff * d + rows * top * eff) * 2 + rows * top * d * 4, 2.0 * rows * top * eff * d)
        y = ops.moe_gemm(h, wd, tiles, max_tiles, rows * top, out_dtype=torch.float32, tile_rows=tile_rows)
        shared = torch.randn(rows, d, device=dev, dtype=bf)
        us = mb._time(lambda i: ops.moe_combine(y, place, wts, shared, gate), 1, **it)
        note(f"{tag}_experts_sum", us, rows * top * d * 4 + rows * d * 6, 0)
        # the like work in Llama: its gate/up and down products at the dense size
        for nm, n, k, sw in (("gate_up", 2 * z["ff"], d, True), ("down", d, z["ff"], False)):
            r = mb.bench_linear(SimpleNamespace(rows=rows, n=n, k=k, swiglu=sw, to_stream=not sw, splits=0, heads=H, kv_heads=H, head_dim=vdim, **it))
            fr = r["TFLOPs"] / peaks["bf16_tflops"] if rows > 64 else r["GBps"] / peaks["hbm_gbs"]
            out[f"{tag}_llama_{nm}"] = {"us": r["us"], "frac": round(fr, 3)}
    ops.tc_status_check()
    return out


def run(sizes, T: int, batch: int, ctx: int, steps: int, warmup: int, peaks: dict, kernels: bool = True) -> dict:
    result = {"design": "Vezatar", "beside": "Llama at equal width, heads, layers and vocabulary", "layers": LAYERS, "dtype": "bf16",
              "prompt_tokens": T, "decode_batch": batch, "decode_context": ctx, "peaks": peaks, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        row = {"config": z}
        for who, cfg in (("vezatar", vezatar_config(z)), ("llama", llama_config(z))):
            t = step_times(cfg, T, batch, ctx, steps, warmup)
            row[who] = {
                "prefill_ms": round(t["prefill_ms"], 3), "prefill_tokens_per_s": round(T / t["prefill_ms"] * 1e3, 1),
                "decode_ms": round(t["decode_ms"], 4), "decode_tokens_per_s": round(batch / t["decode_ms"] * 1e3, 1),
            }
        if kernels:
            row["kernels"] = kernel_table(z, T, batch, ctx, peaks)
        result["sizes"][name] = row
    return result
