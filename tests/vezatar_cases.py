"""Small Vezatar configurations and random weights for the tests, made without the library.

Weights are drawn so that every mechanism matters (activations of order one, sinks and router biases of the size of
the scores they compete with), rounded to bfloat16 and written with the third-party safetensors package."""

import json
import os

import numpy as np
import torch


def _rot(dims, base, scaling):
    return {"base": base, "dims": dims, "scaling": scaling}


def _mixer(heads, dim, rot_dim, vdim, rank, rot, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "rot": rot,
         "scale": scale if scale is not None else 1.0 / float(np.sqrt(dim + rot_dim))}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, shared_ff):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        d["shared"] = {"ff": shared_ff}
    return d


def config_a():
    """Five layers that differ in everything: unequal dim / vdim, a latent size that is no multiple of 32, three and two
    and one head, layers that read another layer's cache with other head sizes, a layer without feed-forward, all
    experts chosen, no shared expert, scaling present and absent."""
    rot_a = _rot(8, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0})
    rot_b = _rot(16, 500000.0, None)
    return {
        "architecture": "Vezatar", "vocab": 131, "width": 96, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "latent_attention", "mixer": _mixer(3, 24, 8, 40, 48, rot_a), "mlp": _moe(5, 2, 56, 72)},
            {"type": "latent_attention", "mixer": _mixer(2, 16, 8, 24, 48, rot_a, kv_from=0, scale=0.3), "mlp": {"kind": "dense", "ff": 200, "limit": 0.7}},
            {"type": "latent_attention", "mixer": _mixer(1, 32, 16, 8, 40, rot_b), "mlp": None},
            {"type": "latent_attention", "mixer": _mixer(4, 8, 8, 16, 48, rot_a, kv_from=0), "mlp": _moe(4, 4, 24, 0)},
            {"type": "latent_attention", "mixer": _mixer(2, 24, 16, 24, 40, rot_b, kv_from=2), "mlp": {"kind": "dense", "ff": 72, "limit": 2.5}},
        ],
    }


def config_b():
    """Sizes that no 16-byte-row kernel takes (a latent of 20, rotated part of 4, width 68), one expert per token of three,
    a routed layer first."""
    rot = _rot(4, 1000.0, {"factor": 1.5, "original": 32, "fast": 4.0, "slow": 1.0})
    return {
        "architecture": "Vezatar", "vocab": 77, "width": 68, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "latent_attention", "mixer": _mixer(4, 8, 4, 12, 20, rot), "mlp": _moe(3, 1, 36, 20)},
            {"type": "latent_attention", "mixer": _mixer(5, 4, 4, 4, 20, rot, kv_from=0), "mlp": {"kind": "dense", "ff": 50, "limit": 1.0}},
            {"type": "latent_attention", "mixer": _mixer(2, 16, 4, 20, 12, rot), "mlp": _moe(6, 3, 10, 10)},
        ],
    }


def config_c():
    """Multiples of 8 everywhere and 8 heads: the sizes that the 16-byte-row and tensor-core kernels take."""
    rot = _rot(32, 10000.0, {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0})
    return {
        "architecture": "Vezatar", "vocab": 512, "width": 256, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "latent_attention", "mixer": _mixer(8, 64, 32, 64, 128, rot), "mlp": {"kind": "dense", "ff": 512, "limit": 3.0}},
            {"type": "latent_attention", "mixer": _mixer(8, 64, 32, 64, 128, rot, kv_from=0), "mlp": _moe(8, 2, 128, 256)},
            {"type": "latent_attention", "mixer": _mixer(16, 32, 32, 48, 128, rot), "mlp": _moe(16, 4, 64, 0)},
        ],
    }


CONFIGS = {"a": config_a, "b": config_b, "c": config_c}


def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "head": (V, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H = m["heads"]
        out[p + "norm1"] = out[p + "norm1b"] = (d,)
        out[p + "mix.q"] = (H * (m["dim"] + m["rot_dim"]), d)
        if "kv_from" not in m:
            out[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], d)
            out[p + "mix.dkv.norm"] = (m["kv_rank"],)
        out[p + "mix.uk"] = (H * m["dim"], m["kv_rank"])
        out[p + "mix.uv"] = (H * m["vdim"], m["kv_rank"])
        out[p + "mix.sink"] = (H,)
        out[p + "mix.g"] = (H * m["vdim"], d)
        out[p + "mix.o"] = (d, H * m["vdim"])
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = out[p + "norm2b"] = (d,)
        if mlp["kind"] == "dense":
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (mlp["ff"], d)
            out[p + "mlp.down"] = (d, mlp["ff"])
        else:
            for e in range(mlp["router"]["experts"]):
                out[p + f"mlp.e{e}.gate"] = out[p + f"mlp.e{e}.up"] = (mlp["expert"]["ff"], d)
                out[p + f"mlp.e{e}.down"] = (d, mlp["expert"]["ff"])
            out[p + "mlp.router"] = (mlp["router"]["experts"], d)
            out[p + "mlp.correction"] = (mlp["router"]["experts"],)
            if mlp.get("shared"):
                out[p + "mlp.shared.gate"] = out[p + "mlp.shared.up"] = (mlp["shared"]["ff"], d)
                out[p + "mlp.shared.down"] = (d, mlp["shared"]["ff"])
                out[p + "mlp.shared.sg"] = (1, d)
    return out


def random_weights(cfg, seed):
    """name -> torch.bfloat16 tensor."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm1") or name.endswith("norm2") or name.endswith("norm1b") or name.endswith("norm2b") or name.endswith(".norm"):
            t = 1.0 + 0.2 * rng.standard_normal(shape)
        elif name.endswith("sink"):
            t = 1.5 * rng.standard_normal(shape)
        elif name.endswith("correction"):
            t = 0.3 * rng.standard_normal(shape)
        elif name.endswith("router"):
            t = 3.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])
        elif name in ("embed",):
            t = rng.standard_normal(shape)
        elif name.endswith("mix.q") or name.endswith("mix.uk"):
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
