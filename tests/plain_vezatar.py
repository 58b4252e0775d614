"""A plain, slow Vezatar: whole sequences, no cache, float64, one function per mechanism.

It shares nothing with the package: tensors come as a dict of numpy arrays by
checkpoint name, the configuration as the dict that config.json holds.  The tests
compare the engine with it.

Notation: h is a sublayer's input [T, d]; rows are positions 0..T-1 of one sequence.
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional

import numpy as np


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    return rms_unit(x, eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def yarn_frequencies(dims: int, base: float, scaling: Optional[Mapping]) -> (np.ndarray, float):
    """(f[dims/2], m): pair i turns by position * f[i]; cos and sin are multiplied by m."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: np.ndarray, pos: np.ndarray, f: np.ndarray, m: float) -> np.ndarray:
    """x[T, ..., dims] with neighbours (2i, 2i+1) as a pair; only the first 2 len(f) dimensions turn."""
    n = 2 * len(f)
    a = pos.astype(np.float64)[:, None] * f[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (len(f),)
    c, s = (np.cos(a) * m).reshape(shape), (np.sin(a) * m).reshape(shape)
    out = x.copy()
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


def latent_kv(h: np.ndarray, W: Mapping[str, np.ndarray], p: str, mix: Mapping, eps: float):
    """(c[T, rank], kr[T, rot_dim]): the normed latent and the turned shared key part of positions 0..T-1."""
    rank, rot_dim = mix["kv_rank"], mix["rot_dim"]
    z = h @ W[p + "dkv"].T
    c = rms_norm(z[:, :rank], W[p + "dkv.norm"], eps)
    f, m = yarn_frequencies(mix["rot"]["dims"], mix["rot"]["base"], mix["rot"].get("scaling"))
    kr = rotate_pairs(z[:, rank : rank + rot_dim], np.arange(h.shape[0]), f, m)
    return c, kr


def latent_attention(h: np.ndarray, W: Mapping[str, np.ndarray], p: str, mix: Mapping, eps: float, c: np.ndarray, kr: np.ndarray) -> np.ndarray:
    """The mixer's output for input h, given the latents and shared key parts it attends to."""
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = mix["heads"], mix["dim"], mix["rot_dim"], mix["vdim"], mix["kv_rank"]
    q = (h @ W[p + "q"].T).reshape(T, H, dim + rot_dim)
    f, m = yarn_frequencies(mix["rot"]["dims"], mix["rot"]["base"], mix["rot"].get("scaling"))
    q_plain = q[:, :, :dim]
    q_rot = rotate_pairs(q[:, :, dim:], np.arange(T), f, m)
    k_plain = (c @ W[p + "uk"].T).reshape(T, H, dim)
    v = (c @ W[p + "uv"].T).reshape(T, H, vdim)
    sink = W[p + "sink"].astype(np.float64)
    out = np.zeros((T, H, vdim))
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ kr.T) * mix["scale"]
        for i in range(T):
            row = s[i, : i + 1]
            top = max(row.max(), sink[hd])
            e = np.exp(row - top)
            out[i, hd] = (e / (e.sum() + math.exp(sink[hd] - top))) @ v[: i + 1, hd]
    gate = sigmoid(h @ W[p + "g"].T)
    return (out.reshape(T, H * vdim) * gate) @ W[p + "o"].T


def dense_ff(h: np.ndarray, W: Mapping[str, np.ndarray], p: str, limit: float) -> np.ndarray:
    g = np.minimum(h @ W[p + "gate"].T, limit)
    u = np.clip(h @ W[p + "up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def silu_expert(h: np.ndarray, W: Mapping[str, np.ndarray], p: str) -> np.ndarray:
    a = h @ W[p + "gate"].T
    return ((a * sigmoid(a)) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def router(h: np.ndarray, W: Mapping[str, np.ndarray], p: str, top: int):
    """(chosen[T, top], weights[T, top], scores[T, E]).  Ties go to the lower index."""
    z = h @ W[p + "router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    choice = s + W[p + "correction"]
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1), s


def moe_ff(h: np.ndarray, W: Mapping[str, np.ndarray], p: str, mlp: Mapping) -> np.ndarray:
    top = mlp["router"]["top"]
    chosen, weights, _ = router(h, W, p, top)
    out = np.zeros((h.shape[0], W[p + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += weights[t, j] * silu_expert(h[t : t + 1], W, f"{p}e{int(chosen[t, j])}.")[0]
    if mlp.get("shared"):
        out += silu_expert(h, W, p + "shared.") * sigmoid(h @ W[p + "shared.sg"].T)
    return out


def forward(config: Mapping, W: Mapping[str, np.ndarray], tokens, keep_layers: Optional[List[np.ndarray]] = None) -> np.ndarray:
    """Logits [T, vocab] of one sequence; keep_layers, if a list, receives the stream after every layer."""
    W = {k: np.asarray(v, dtype=np.float64) for k, v in W.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    held: Dict[int, tuple] = {}
    for i, layer in enumerate(config["layers"]):
        p, mix = f"l{i}.", layer["mixer"]
        assert layer["type"] == "latent_attention"
        h = rms_norm(x, W[p + "norm1"], eps)
        src = mix.get("kv_from")
        if src is None:
            held[i] = latent_kv(h, W, p + "mix.", mix, eps)
            src = i
        c, kr = held[src]
        x = x + rms_norm(latent_attention(h, W, p + "mix.", mix, eps, c, kr), W[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = rms_norm(x, W[p + "norm2"], eps)
            y = dense_ff(h, W, p + "mlp.", mlp["limit"]) if mlp["kind"] == "dense" else moe_ff(h, W, p + "mlp.", mlp)
            x = x + rms_norm(y, W[p + "norm2b"], eps)
        if keep_layers is not None:
            keep_layers.append(x.copy())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T
