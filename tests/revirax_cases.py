"""Small Revirax configurations and random weights for the tests, made without the library.

Weights are drawn so that every mechanism matters (activations of order one, sinks of the size of the scores they compete
with, a mixing matrix far from the identity, norm weights away from their neutral value), rounded to bfloat16 and written
with the third-party safetensors package."""

import json
import os

import numpy as np
import torch


def _rot(dims, base, scaling):
    return {"base": base, "dims": dims, "scaling": scaling}


def _attn(heads, kv_heads, dim, vdim, rot, scale=None, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale if scale is not None else 1.0 / float(np.sqrt(dim))}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _lightning(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def _parallel(left, width, left_scale, right_scale):
    return {"left": left, "right": {"width": width}, "left_scale": left_scale, "right_scale": right_scale}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def config_a():
    """Six layers that differ in everything: unequal key and value sizes that are no multiples of 8, 6 heads on 2 and 1 on 1,
    windows of 5 and of exactly one page, a window on a layer with a sink, a layer without feed-forward, both scalings and none,
    a state of 24 x 40 per head (neither a multiple of the kernels' 32)."""
    banded = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
    ramped = {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}
    return {
        "architecture": "Revirax", "vocab": 131, "width": 96, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "attention", "mixer": _attn(6, 2, 20, 12, _rot(8, 10000.0, banded), scale=0.3), "mlp": _dense(200)},
            {"type": "lightning", "mixer": _lightning(3, 24, 40, (0.5, 0.9, 0.999)), "mlp": None},
            {"type": "parallel", "mixer": _parallel(_attn(4, 4, 16, 24, _rot(16, 1000.0, ramped), window=5), 50, 1.3, 0.7), "mlp": _dense(72)},
            {"type": "attention", "mixer": _attn(1, 1, 32, 8, _rot(16, 500000.0, None), window=70), "mlp": _dense(56)},
            {"type": "parallel", "mixer": _parallel(_attn(2, 1, 24, 16, _rot(4, 100.0, None), scale=0.4, window=64), 9, 0.5, 2.0), "mlp": None},
            {"type": "lightning", "mixer": _lightning(1, 40, 8, (0.97,)), "mlp": _dense(40)},
        ],
    }


def config_b():
    """A width that no 16-byte-row kernel takes (68), a parallel layer first, a window of one (a query sees itself only), no
    rotation at all in one mixer, a recurrent unit of 7 channels."""
    return {
        "architecture": "Revirax", "vocab": 77, "width": 68, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "parallel", "mixer": _parallel(_attn(3, 1, 12, 12, _rot(0, 10000.0, None), window=1), 7, 1.0, 1.0), "mlp": _dense(50)},
            {"type": "lightning", "mixer": _lightning(2, 72, 8, (0.8, 1.0)), "mlp": _dense(36)},
            {"type": "attention", "mixer": _attn(4, 1, 8, 16, _rot(4, 1000.0, {"factor": 8.0, "low": 1.0, "high": 2.0, "original": 8})), "mlp": None},
            {"type": "parallel", "mixer": _parallel(_attn(2, 2, 8, 4, _rot(8, 50.0, {"factor": 1.5, "original": 32, "fast": 4.0, "slow": 1.0}), window=33), 20, 0.25, 1.5), "mlp": _dense(10)},
        ],
    }


def config_c():
    """Multiples of 8 everywhere, head sizes of 64 and 128, 8 heads on 2: the sizes that 16-byte-row and tensor-core kernels take."""
    banded = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}
    ramped = {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}
    return {
        "architecture": "Revirax", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "lightning", "mixer": _lightning(2, 128, 64, (0.9, 0.99)), "mlp": _dense(512)},
            {"type": "attention", "mixer": _attn(8, 2, 64, 64, _rot(32, 10000.0, banded)), "mlp": _dense(256)},
            {"type": "parallel", "mixer": _parallel(_attn(8, 4, 32, 32, _rot(32, 10000.0, ramped), window=128), 256, 0.8, 0.9), "mlp": _dense(512)},
            {"type": "attention", "mixer": _attn(2, 2, 128, 128, _rot(64, 500000.0, None), scale=0.05), "mlp": _dense(256)},
        ],
    }


CONFIGS = {"a": config_a, "b": config_b, "c": config_c}


def _attn_shapes(out, p, m, d, sink=False, extras=False):
    H, G = m["heads"], m["kv_heads"]
    out[p + "q"] = (H * m["dim"], d)
    out[p + "k"] = (G * m["dim"], d)
    out[p + "v"] = (G * m["vdim"], d)
    out[p + "o"] = (d, H * m["vdim"])
    if sink:
        out[p + "sink"] = (H,)
    if extras:
        out[p + "q.b"], out[p + "k.b"], out[p + "v.b"], out[p + "o.b"] = (H * m["dim"],), (G * m["dim"],), (G * m["vdim"],), (d,)
        out[p + "talk"] = (H, H)
        out[p + "g"] = (H * m["vdim"], d)


def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "head": (V, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = (d,)
        if layer["type"] == "lightning":
            H = m["heads"]
            out[p + "mix.q"] = out[p + "mix.k"] = (H * m["dim"], d)
            out[p + "mix.v"] = out[p + "mix.g"] = (H * m["vdim"], d)
            out[p + "mix.norm"] = (H * m["vdim"],)
            out[p + "mix.o"] = (d, H * m["vdim"])
        elif layer["type"] == "attention":
            _attn_shapes(out, p + "mix.", m, d, sink=True)
        else:
            _attn_shapes(out, p + "mix.left.", m["left"], d, extras=True)
            w = m["right"]["width"]
            out[p + "mix.right.z"] = out[p + "mix.right.x"] = out[p + "mix.right.g"] = (w, d)
            out[p + "mix.right.z.b"] = out[p + "mix.right.x.b"] = (w,)
            out[p + "mix.right.o"] = (d, w)
        if layer["mlp"] is not None:
            out[p + "norm2"] = out[p + "norm2b"] = (d,)
            out[p + "mlp.up"] = (layer["mlp"]["ff"], d)
            out[p + "mlp.down"] = (d, layer["mlp"]["ff"])
    return out


def random_weights(cfg, seed):
    """name -> torch.bfloat16 tensor."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            t = 0.3 * rng.standard_normal(shape)  # stored around zero
        elif name.endswith("mix.norm"):
            t = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last == "sink":
            t = 1.5 * rng.standard_normal(shape)
        elif last == "talk":
            t = np.eye(shape[0]) * 0.7 + 0.6 * rng.standard_normal(shape)
        elif last == "b":
            t = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            t = rng.standard_normal(shape)
        elif last in ("q", "k") and ".left." in name or (last in ("q", "k") and len(shape) == 2 and "mix" in name):
            t = 2.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])  # scores wide enough for a peaked softmax
        else:
            t = rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(t, dtype=np.float32)).to(torch.bfloat16)
    return out


def write_model(folder, cfg, weights):
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return str(folder)


def as_float64(weights):
    return {k: v.to(torch.float64).numpy() for k, v in weights.items()}
