"""Revirax beside Llama at equal sizes: prompt-step and decode-step throughput through the engine, and every kernel that
only Revirax uses timed alone beside the Llama kernel that does the like work.

    python bench.py --design revirax [--design-sizes small,lite,wide]

Sizes resemble real models' layers (random weights, four layers: lightning, attention, parallel, attention; the whole
vocabulary).  Llama beside it has the same width, heads, kv heads, head size, layer count, feed-forward size and vocabulary.
Every kernel's fraction is what it must move (bytes, against the measured copy rate) or compute (flops, against the measured
bfloat16 matrix rate), whichever bound is the tighter one, divided by the time it took.
"""

from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Dict

import torch

from . import microbench as mb
from . import ops
from .design_bench import _frac, step_times

SIZES = {
    "small": dict(width=1024, heads=8, kv_heads=2, hd=128, window=512, gru=1024, ff=4096, vocab=32000),
    "lite": dict(width=2048, heads=16, kv_heads=4, hd=128, window=1024, gru=2048, ff=8192, vocab=32000),
    "wide": dict(width=4096, heads=32, kv_heads=8, hd=128, window=1024, gru=4096, ff=12288, vocab=32000),
}
LAYERS = 4


def revirax_config(z: dict) -> dict:
    H, G, hd = z["heads"], z["kv_heads"], z["hd"]
    banded = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}
    ramped = {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}
    attn = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": 1.0 / math.sqrt(hd), "rot": {"base": 500000.0, "dims": hd, "scaling": banded}}
    left = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": 1.0 / math.sqrt(hd), "mask": {"size": z["window"]},
            "rot": {"base": 10000.0, "dims": hd // 2, "scaling": ramped}}
    lightning = {"heads": H, "dim": hd, "vdim": hd, "decay": [1.0 - 2.0 ** (-3 - 5 * i / max(H - 1, 1)) for i in range(H)]}
    parallel = {"left": left, "right": {"width": z["gru"]}, "left_scale": 0.7, "right_scale": 0.7}
    mlp = {"kind": "dense", "ff": z["ff"]}
    kinds = [("lightning", lightning), ("attention", attn), ("parallel", parallel), ("attention", attn)]
    layers = [{"type": t, "mixer": m, "mlp": mlp} for t, m in (kinds[i % 4] for i in range(LAYERS))]
    return {"architecture": "Revirax", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "layers": layers}


def llama_config(z: dict) -> dict:
    return {
        "architectures": ["LlamaForCausalLM"], "tie_word_embeddings": False, "torch_dtype": "bfloat16", "hidden_size": z["width"],
        "intermediate_size": z["ff"], "num_hidden_layers": LAYERS, "num_attention_heads": z["heads"], "num_key_value_heads": z["kv_heads"],
        "head_dim": z["hd"], "vocab_size": z["vocab"], "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "rope_scaling": None,
    }


def kernel_table(z: dict, T: int, batch: int, ctx: int, peaks: dict) -> Dict[str, dict]:
    """Each kernel of the design alone, at a prompt step of T tokens (one sequence) and a decode step of `batch` sequences at `ctx`."""
    dev, bf = "cuda:0", torch.bfloat16
    H, G, hd, d, W, gw, ff = z["heads"], z["kv_heads"], z["hd"], z["width"], z["window"], z["gru"], z["ff"]
    out: Dict[str, dict] = {}
    it = dict(iters=10, warmup=2)
    scale = 1.0 / math.sqrt(hd)

    def note(name, us, nbytes, flops, like=None):
        out[name] = {"us": round(us, 1), "frac": _frac(us, nbytes, flops, peaks)}
        if like:
            out[name]["like"] = like

    like_prefill = mb.bench_flash_prefill(SimpleNamespace(tokens=T, impl="auto", heads=H, kv_heads=G, head_dim=hd, splits=0, **it))
    like_prefill = {"kernel": like_prefill["kernel"], "us": like_prefill["us"], "frac": round(like_prefill["causal_TFLOPs"] / peaks["bf16_tflops"], 3)}
    like_decode = mb.bench_attn_decode(SimpleNamespace(seqs=batch, ctx=ctx, impl="auto", heads=H, kv_heads=G, head_dim=hd, splits=0, **it))
    like_decode = {"kernel": "attn_decode", "us": like_decode["us"], "frac": round(like_decode["GBps"] / peaks["hbm_gbs"], 3)}

    # ---- softmax attention with a sink (all keys) and with mixed scores, a window and a gate: prompt and decode
    def attention(rows, n_seqs, pos0, tag):
        per_seq = (pos0 + rows // n_seqs + 63) // 64
        kp = torch.randn(n_seqs * per_seq, G, 64, hd, device=dev, dtype=bf)
        vp = torch.randn(n_seqs * per_seq, G, 64, hd, device=dev, dtype=bf)
        table = torch.randperm(n_seqs * per_seq, device=dev).to(torch.int32).view(n_seqs, per_seq).contiguous()
        q = torch.randn(rows, H * hd, device=dev, dtype=bf)
        gate = torch.randn(rows, H * hd, device=dev, dtype=bf)
        seq = torch.arange(n_seqs, dtype=torch.int32, device=dev).repeat_interleave(rows // n_seqs)
        pos = (pos0 + torch.arange(rows // n_seqs, dtype=torch.int32, device=dev)).repeat(n_seqs)
        sink = torch.zeros(H, device=dev)
        mix = torch.eye(H, device=dev)
        keys_all = sum(min(p + 1, 1 << 30) for p in range(pos0, pos0 + rows // n_seqs)) * n_seqs
        keys_win = sum(min(p + 1, W) for p in range(pos0, pos0 + rows // n_seqs)) * n_seqs
        cache_bytes = lambda keys_per_seq: n_seqs * keys_per_seq * G * 2 * hd * 2  # noqa: E731
        start = torch.arange(n_seqs + 1, dtype=torch.int32, device=dev) * (rows // n_seqs)
        p0 = torch.full((n_seqs,), pos0, dtype=torch.int32, device=dev)
        max_q = rows // n_seqs
        # a plain attention with a sink runs on the plain attention's own kernels
        if rows > batch:
            us = mb._time(lambda i: ops.flash_prefill_tc(q, kp, vp, table, start, p0, max_q, H, G, hd, scale=scale, sink=sink), 1, **it)
        else:
            from ..parts.attention import decode_splits
            n_splits = decode_splits(n_seqs, H, G, pos0 + 1, hd)
            scratch = torch.empty(ops.attn_decode_scratch_floats(n_seqs, H, hd, n_splits), device=dev)
            lens = torch.full((n_seqs,), pos0 + 1, dtype=torch.int32, device=dev)
            us = mb._time(lambda i: ops.attn_decode(q, kp, vp, table, lens, H, G, hd, n_splits, scratch, scale=scale, sink=sink), 1, **it)
        note(f"{tag}_attention_sink", us, cache_bytes(pos0 + rows // n_seqs) + rows * H * hd * 4, 4.0 * keys_all * H * hd,
             like=like_prefill if rows > batch else like_decode)
        if ops.flash_mix_takes(hd, hd, G):
            us_fold = mb._time(lambda i: ops.fold_queries(q, mix, H, G, hd), 1, **it)
            note(f"{tag}_fold_queries", us_fold, rows * H * hd * 2 * (1 + G), 2.0 * rows * H * H * hd)
            qf = ops.fold_queries(q, mix, H, G, hd)
            if rows > batch or not ops.flash_mix_decode_takes(H, G, hd, hd):
                us = mb._time(lambda i: ops.flash_mix(qf, kp, vp, table, start, p0, max_q, H, G, hd, hd, scale, window=W, folded=True, gate=gate), 1, **it)
            else:  # a decode step: the rows of a block are the heads (as `Attention` plans it)
                from .device import sm_count
                pages = (min(W, pos0 + 1) + 63) // 64 + 1
                n_splits = max(1, min(2 * sm_count() // n_seqs, pages, 64))
                sc = torch.empty(ops.flash_mix_decode_scratch_floats(n_seqs, H, hd, n_splits), device=dev)
                us = mb._time(lambda i: ops.flash_mix_decode(qf, kp, vp, table, p0, H, G, hd, hd, scale, n_splits, sc, window=W, gate=gate), 1, **it)
            # its products: the scores against the keys of all kv heads, and the values
            note(f"{tag}_attention_mixed_window_gate", us, cache_bytes(min(W, pos0 + rows // n_seqs)) + rows * H * hd * (2 * G + 4), 2.0 * keys_win * H * hd * (G + 1),
                 like=like_prefill if rows > batch else like_decode)
        # biases, rotation, cache write
        qkv = torch.randn(rows, (H + 2 * G) * hd, device=dev, dtype=bf)
        bias = torch.zeros((H + 2 * G) * hd, device=dev)
        freq = torch.rand(hd // 4, device=dev)
        us = mb._time(lambda i: ops.qkv_prep(qkv, bias, pos, seq, table, kp, vp, freq, 1.1, H, G, hd, hd, hd // 2, False), 1, **it)
        us_like = mb._time(lambda i: ops.rope_kv_write(qkv, pos, seq, table, kp, vp, freq, H, G, hd, hd // 2, False), 1, **it)
        nbytes = rows * ((H + G) * hd * 4 + G * hd * 4)
        note(f"{tag}_bias_rotate_store", us, nbytes, 0, like={"kernel": "rope_kv_write", "us": round(us_like, 1), "frac": _frac(us_like, nbytes, 0, peaks)})

    attention(T, 1, 0, "prefill")
    attention(batch, batch, ctx - 1, "decode")

    # ---- linear attention with decay, its norm and gate; the recurrent unit
    for rows, n_seqs, tag in ((T, 1, "prefill"), (batch, batch, "decode")):
        proj = torch.randn(rows, 4 * H * hd, device=dev, dtype=bf)
        q, k, v, g = (proj[:, i * H * hd: (i + 1) * H * hd] for i in range(4))
        decay = torch.full((H,), 0.99, device=dev)
        state = torch.zeros(n_seqs, H, hd, hd, device=dev)
        slots = torch.arange(n_seqs, dtype=torch.int32, device=dev)
        start = torch.arange(n_seqs + 1, dtype=torch.int32, device=dev) * (rows // n_seqs)
        kw = {}
        if rows > batch:  # a prompt step goes chunk by chunk
            kw = dict(max_q_len=rows // n_seqs, scratch=torch.empty(ops.decay_attn_chunked_scratch_floats(n_seqs, rows // n_seqs, H, hd, hd), device=dev))
        us = mb._time(lambda i: ops.decay_attn(q, k, v, decay, state, slots, start, H, hd, hd, silu=True, **kw), 1, **it)
        note(f"{tag}_decay_attention", us, rows * H * hd * (3 * 2 + 4) + 2 * state.numel() * 4, 4.0 * rows * H * hd * hd,
             like=like_prefill if rows > batch else like_decode)
        o = torch.randn(rows, H * hd, device=dev)
        w = torch.ones(H * hd, device=dev)
        us = mb._time(lambda i: ops.rms_gate(o, w, 1e-5, g, bf), 1, **it)
        note(f"{tag}_heads_norm_gate", us, rows * H * hd * (4 + 2 + 2), 0)
        zx = torch.randn(rows, 3 * gw, device=dev, dtype=bf)
        bz = torch.zeros(gw, device=dev)
        gstate = torch.zeros(n_seqs, gw, device=dev)
        us = mb._time(lambda i: ops.min_gru(zx[:, :gw], zx[:, gw: 2 * gw], zx[:, 2 * gw:], bz, bz, gstate, slots, start, max_q_len=rows // n_seqs), 1, **it)
        note(f"{tag}_min_gru", us, rows * gw * 8 + 2 * gstate.numel() * 4, 0)
        # the feed-forward's activation (Llama's is fused into its product), the sandwich norm beside Llama's
        hh = torch.randn(rows, ff, device=dev, dtype=bf)
        us = mb._time(lambda i: ops.unary_act(hh), 1, **it)
        note(f"{tag}_squared_relu", us, rows * ff * 4, 0)
        x = torch.randn(rows, d, device=dev)
        delta = torch.randn(rows, d, device=dev, dtype=bf)
        w1, w2, bias = torch.ones(d, device=dev), torch.ones(d, device=dev), torch.zeros(d, device=dev)
        us = mb._time(lambda i: ops.normed_add_rmsnorm(x, delta, w1, 1e-5, w2, 1e-5, bf, delta_bias=bias), 1, **it)
        us_like = mb._time(lambda i: ops.add_rmsnorm(x, delta, w2, 1e-5, bf), 1, **it)
        nbytes = rows * d * (4 + 4 + 2 + 2)
        note(f"{tag}_normed_add_norm", us, nbytes, 0, like={"kernel": "add_rmsnorm", "us": round(us_like, 1), "frac": _frac(us_like, nbytes, 0, peaks)})
    ops.tc_status_check()
    return out


def run(sizes, T: int, batch: int, ctx: int, steps: int, warmup: int, peaks: dict, kernels: bool = True) -> dict:
    result = {"design": "Revirax", "beside": "Llama at equal width, heads, kv heads, head size, layers, feed-forward size and vocabulary",
              "layers": LAYERS, "dtype": "bf16", "prompt_tokens": T, "decode_batch": batch, "decode_context": ctx, "peaks": peaks, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        row = {"config": z}
        for who, cfg in (("revirax", revirax_config(z)), ("llama", llama_config(z))):
            t = step_times(cfg, T, batch, ctx, steps, warmup)
            row[who] = {
                "prefill_ms": round(t["prefill_ms"], 3), "prefill_tokens_per_s": round(T / t["prefill_ms"] * 1e3, 1),
                "decode_ms": round(t["decode_ms"], 4), "decode_tokens_per_s": round(batch / t["decode_ms"] * 1e3, 1),
            }
        if kernels:
            row["kernels"] = kernel_table(z, T, batch, ctx, peaks)
        result["sizes"][name] = row
    return result
