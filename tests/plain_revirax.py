"""A plain, slow Revirax: whole sequences, no cache, float64, one function per mechanism.

It shares nothing with the package: tensors come as a dict of numpy arrays by
checkpoint name, the configuration as the dict that config.json holds.  The tests
compare the engine with it.

Notation: h is a sublayer's input [T, d]; rows are positions 0..T-1 of one sequence.
Recurrences are written as loops over positions, attention as a loop over queries.
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Tuple

import numpy as np


# --------------------------------------------------------------------------- small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def centred_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """The layer norm of this design: the weight is stored as its distance from one."""
    return rms_unit(x, eps) * (1.0 + w)


# --------------------------------------------------------------------------- rotary frequencies
def plain_frequencies(dims: int, base: float) -> np.ndarray:
    return base ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)


def banded_frequencies(dims: int, base: float, scaling: Optional[Mapping]) -> Tuple[np.ndarray, float]:
    """Scaling by wavelength bands (keys factor, low, high, original): short waves keep their frequency,
    long waves are slowed by `factor`, those between are blended.  Returns (f, 1)."""
    f = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < original / high:
            continue
        if wave > original / low:
            out[i] = fi / factor
        else:
            s = (original / wave - low) / (high - low)
            out[i] = (1.0 - s) * fi / factor + s * fi
    return out, 1.0


def ramped_frequencies(dims: int, base: float, scaling: Optional[Mapping]) -> Tuple[np.ndarray, float]:
    """Scaling by a ramp over the pair index (keys factor, original, fast, slow).  Returns (f, m): cosines and
    sines are multiplied by m = 0.1 ln(factor) + 1."""
    f = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    i = np.arange(dims // 2, dtype=np.float64)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotary_table(rot: Optional[Mapping]) -> Tuple[np.ndarray, float]:
    """(f, m) of a mixer's `rot` block; which scaling it is shows in the keys of `rot.scaling`."""
    if not rot or not rot.get("dims"):
        return np.zeros(0), 1.0
    scaling = rot.get("scaling")
    if scaling and "fast" in scaling:
        return ramped_frequencies(rot["dims"], rot["base"], scaling)
    return banded_frequencies(rot["dims"], rot["base"], scaling)


def rotate_halves(x: np.ndarray, pos: np.ndarray, f: np.ndarray, m: float) -> np.ndarray:
    """x[T, heads, size]: dimension i is paired with i + len(f); dimensions from 2 len(f) on stay."""
    n = len(f)
    if n == 0:
        return x.copy()
    a = pos.astype(np.float64)[:, None] * f[None, :]
    c, s = (np.cos(a) * m)[:, None, :], (np.sin(a) * m)[:, None, :]
    out = x.copy()
    u, v = x[..., :n], x[..., n : 2 * n]
    out[..., :n] = u * c - v * s
    out[..., n : 2 * n] = v * c + u * s
    return out


# --------------------------------------------------------------------------- mixers
def softmax_attention(
    q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int = 0,
    sink: Optional[np.ndarray] = None, talk: Optional[np.ndarray] = None,
) -> np.ndarray:
    """q[T, H, dim], k[T, G, dim], v[T, G, vdim] -> [T, H * vdim].

    Query head h reads key/value head h // (H / G).  talk[H, H]: the scaled scores of all heads are mixed,
    s_h <- sum_g talk[h, g] s_g, before the softmax.  window w > 0: query i sees keys j with 0 <= i - j < w.
    sink[H]: exp(sink_h) joins the softmax's denominator and nothing else."""
    T, H, _ = q.shape
    G, vdim = k.shape[1], v.shape[2]
    rep = H // G
    out = np.zeros((T, H, vdim))
    for i in range(T):
        j0 = max(0, i - window + 1) if window else 0
        s = np.stack([k[j0 : i + 1, h // rep] @ q[i, h] for h in range(H)]) * scale  # [H, keys]
        if talk is not None:
            s = talk @ s
        for h in range(H):
            top = s[h].max() if sink is None else max(s[h].max(), sink[h])
            e = np.exp(s[h] - top)
            den = e.sum() + (0.0 if sink is None else math.exp(sink[h] - top))
            out[i, h] = (e / den) @ v[j0 : i + 1, h // rep]
    return out.reshape(T, H * vdim)


def attention_mixer(h: np.ndarray, W: Mapping[str, np.ndarray], p: str, mix: Mapping, pos0: int = 0) -> np.ndarray:
    """Grouped-query attention with every option the design has; what a model lacks is absent from `mix` or W:
    biases (`<name>.b`), `talk`, `sink`, a gate `g`, `mask.size`."""
    T = h.shape[0]
    H, G, dim, vdim = mix["heads"], mix["kv_heads"], mix["dim"], mix["vdim"]

    def proj(name):
        y = h @ W[p + name].T
        return y + W[p + name + ".b"] if (p + name + ".b") in W else y

    pos = np.arange(pos0, pos0 + T)
    f, m = rotary_table(mix.get("rot"))
    q = rotate_halves(proj("q").reshape(T, H, dim), pos, f, m)
    k = rotate_halves(proj("k").reshape(T, G, dim), pos, f, m)
    v = proj("v").reshape(T, G, vdim)
    window = int((mix.get("mask") or {}).get("size", 0))
    a = softmax_attention(q, k, v, float(mix["scale"]), window, W.get(p + "sink"), W.get(p + "talk"))
    if (p + "g") in W:
        a = a * sigmoid(h @ W[p + "g"].T)
    return proj_out(a, W, p)


def proj_out(a, W, p):
    y = a @ W[p + "o"].T
    return y + W[p + "o.b"] if (p + "o.b") in W else y


def decayed_linear_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, decay: np.ndarray) -> np.ndarray:
    """Per head S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k [T, H, dim], v [T, H, vdim] -> [T, H, vdim]."""
    T, H, dim = q.shape
    vdim = v.shape[2]
    S = np.zeros((H, dim, vdim))
    out = np.zeros((T, H, vdim))
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + np.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out


def lightning_mixer(h: np.ndarray, W: Mapping[str, np.ndarray], p: str, mix: Mapping, eps: float) -> np.ndarray:
    T = h.shape[0]
    H, dim, vdim = mix["heads"], mix["dim"], mix["vdim"]
    q = silu(h @ W[p + "q"].T).reshape(T, H, dim)
    k = silu(h @ W[p + "k"].T).reshape(T, H, dim)
    v = silu(h @ W[p + "v"].T).reshape(T, H, vdim)
    o = decayed_linear_attention(q, k, v, np.asarray(mix["decay"], dtype=np.float64)).reshape(T, H * vdim)
    o = rms_unit(o, eps) * W[p + "norm"]  # all heads together, plain weight
    return (o * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def min_gru(z: np.ndarray, u: np.ndarray) -> np.ndarray:
    """S_t = (1 - z_t) S_(t-1) + z_t c_t element by element, S_(-1) = 0; c = u + 1/2 where u >= 0, else sigmoid(u)."""
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1])
    out = np.zeros_like(z)
    for t in range(z.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S
    return out


def gru_mixer(h: np.ndarray, W: Mapping[str, np.ndarray], p: str) -> np.ndarray:
    z = sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    return (min_gru(z, u) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h, W, p, mix, eps):
    left = attention_mixer(h, W, p + "left.", mix["left"])
    right = gru_mixer(h, W, p + "right.")
    return float(mix["left_scale"]) * left + float(mix["right_scale"]) * right


def mixer(kind: str, h, W, p, mix, eps):
    if kind == "lightning":
        return lightning_mixer(h, W, p, mix, eps)
    if kind == "attention":
        return attention_mixer(h, W, p, mix)
    if kind == "parallel":
        return parallel_mixer(h, W, p, mix, eps)
    raise ValueError(f"unknown mixer '{kind}'")


# --------------------------------------------------------------------------- feed-forward
def squared_relu_mlp(h, W, p):
    return (np.maximum(h @ W[p + "up"].T, 0.0) ** 2) @ W[p + "down"].T


# --------------------------------------------------------------------------- the model
def forward(cfg: Mapping, W: Mapping[str, np.ndarray], tokens, layers_out: Optional[List[np.ndarray]] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence.  layers_out: if a list, receives the stream after every layer."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][np.asarray(tokens, dtype=np.int64)]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = mixer(layer["type"], centred_norm(x, W[p + "norm1"], eps), W, p + "mix.", layer["mixer"], eps)
        x = x + centred_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"unknown feed-forward '{layer['mlp']['kind']}'")
            y = squared_relu_mlp(centred_norm(x, W[p + "norm2"], eps), W, p + "mlp.")
            x = x + centred_norm(y, W[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return centred_norm(x, W["final.norm"], eps) @ W["head"].T
