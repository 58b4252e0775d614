"""Attention whose keys and values are made from one cached latent vector per position."""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.device import sm_count
from ..kernels.linear import linear, linear_to_stream
from ..spec import PartSpec
from .base import MIXERS, POSITIONS, KVNeed, Mixer, ParamInfo

_NAMES = {"q": "q", "kv": "dkv", "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "sink": "sink", "gate": "g", "out": "o"}


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Causal attention over a cache that holds, per position, a latent c (`kv_rank` numbers, RMS-normed) and one
    rotated key part kr (`rot_dim` numbers) shared by all heads.

        q[t, h] = [q_plain (dim) | q_rot (rot_dim)] = rows of W_q xn[t];   [c_raw | kr_raw] = W_kv xn[t]
        c = rmsnorm(c_raw) * w_norm,  kr = rotate(kr_raw, pos),  q_rot = rotate(q_rot, pos)
        key of head h at j = [W_uk[h] c_j | kr_j],  value = W_uv[h] c_j
        score = (q_plain . W_uk[h] c_j + q_rot . kr_j) * scale,  softmax whose denominator also holds exp(sink[h])
        result = W_o ( concat_h(sum_j p_j W_uv[h] c_j) * sigmoid(W_g xn[t]) )

    The kernels never expand the cache into per-head keys and values: W_uk[h]^T is applied to the query
    (q_lat = W_uk[h]^T q_plain, so that the score is [q_lat | q_rot] . [c_j | kr_j]) and W_uv[h] to the
    probability-weighted sum of the latents, which is the same arithmetic in another order.

    params: hidden_size, num_heads, dim, rot_dim, vdim, kv_rank, scale, eps (of the latent's norm),
            sink (bool), gate (bool), own_kv (bool: False for a layer that only reads another layer's cache),
            window (0 = all keys), position (a PartSpec of kind "rotary" over the rotated part),
            names (optional: tensor names after the prefix, keys q kv kv_norm k_up v_up sink gate out).
    tensors: <prefix>q [H (dim + rot_dim), d], dkv [kv_rank + rot_dim, d], dkv.norm [kv_rank], uk [H dim, kv_rank],
             uv [H vdim, kv_rank], sink [H], g [H vdim, d], o [d, H vdim]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.H = int(self._param("num_heads"))
        self.dim = int(self._param("dim"))
        self.rot = int(self._param("rot_dim"))
        self.vdim = int(self._param("vdim"))
        self.rank = int(self._param("kv_rank"))
        self.scale = float(self._param("scale"))
        self.eps = float(self._param("eps"))
        self.has_sink = bool(spec.params.get("sink", True))
        self.has_gate = bool(spec.params.get("gate", True))
        self.own_kv = bool(spec.params.get("own_kv", True))
        self.window = int(spec.params.get("window", 0))
        self.names = dict(_NAMES, **dict(spec.params.get("names", {})))
        if min(self.H, self.rank, self.vdim) <= 0 or self.dim < 0 or self.rot < 0 or self.dim + self.rot == 0:
            raise ConfigError(f"latent_attention: sizes heads={self.H} dim={self.dim} rot_dim={self.rot} vdim={self.vdim} kv_rank={self.rank}")
        if self.rank > 1024:
            raise ConfigError(f"latent_attention: kv_rank {self.rank} is above 1024, the most the attention kernels built here take")
        pos_spec = self._param("position")
        if not isinstance(pos_spec, PartSpec):
            raise ConfigError("latent_attention: 'position' must be a PartSpec")
        self.position = POSITIONS.build(pos_spec, runtime)
        fusion = self.position.decode_fusion()
        if fusion is None and getattr(self.position, "rotary_dim", 0):
            fusion = (self.position.inv_freq, self.position.rotary_dim, self.position.interleaved)
        if fusion is None or (fusion[1] and not fusion[2]):
            raise ConfigError("latent_attention: the position encoding must be a rotation of neighbouring pairs (or none)")
        self.freq, rotary_dim = fusion[0], int(fusion[1])
        if rotary_dim > self.rot or rotary_dim % 2:
            raise ConfigError(f"latent_attention: {rotary_dim} rotated dimensions do not fit a rotated part of {self.rot}")
        self.n_pairs = rotary_dim // 2
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.qd, self.vd, self.kvd = self.H * (self.dim + self.rot), self.H * self.vdim, self.rank + self.rot
        self.w_in = self.w_o = self.w_ukT = self.w_uv = self.w_norm = self.sink = None

    def cache_need(self):
        return KVNeed(1, self.kvd, self.window, values=False) if self.own_kv else None

    def children(self):
        return (self.position,)

    def param_infos(self) -> Dict[str, ParamInfo]:
        p, n = self.prefix, self.names
        infos = {
            p + n["q"]: ParamInfo((self.qd, self.d)),
            p + n["k_up"]: ParamInfo((self.H * self.dim, self.rank)),
            p + n["v_up"]: ParamInfo((self.vd, self.rank)),
            p + n["out"]: ParamInfo((self.d, self.vd)),
        }
        if self.own_kv:
            infos[p + n["kv"]] = ParamInfo((self.kvd, self.d))
            infos[p + n["kv_norm"]] = ParamInfo((self.rank,), "scalars")
        if self.has_sink:
            infos[p + n["sink"]] = ParamInfo((self.H,), "scalars")
        if self.has_gate:
            infos[p + n["gate"]] = ParamInfo((self.vd, self.d))
        return infos

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = self.prefix, self.names
        # one product serves the queries, the gate and (in a layer with a cache of its own) the latent row
        parts = [tensors[p + n["q"]]]
        if self.has_gate:
            parts.append(tensors[p + n["gate"]])
        if self.own_kv:
            parts.append(tensors[p + n["kv"]])
            self.w_norm = tensors[p + n["kv_norm"]].contiguous()
        self.w_in = torch.cat(parts, dim=0).contiguous()
        # W_uk[h] as [rank, dim]: the map from a head's plain query part to the latent space
        self.w_ukT = tensors[p + n["k_up"]].view(self.H, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[p + n["v_up"]].view(self.H, self.vdim, self.rank).contiguous()
        self.w_o = tensors[p + n["out"]].contiguous()
        self.sink = tensors[p + n["sink"]].contiguous() if self.has_sink else None

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False):
        if shared_cache == self.own_kv:
            raise ConfigError("latent_attention: a layer with a latent projection of its own fills its own cache, one without reads another's")
        T = xn.shape[0]
        proj = linear(xn, self.w_in)
        q = proj[:, : self.qd]
        g = proj[:, self.qd : self.qd + self.vd] if self.has_gate else None
        kv = proj[:, proj.shape[1] - self.kvd :] if self.own_kv else None
        q_cat = torch.empty((T, self.H, self.kvd), dtype=xn.dtype, device=xn.device)
        ops.latent_prep(
            q, kv, self.w_norm, self.eps, self.freq, self.n_pairs, self.magnitude, step.tok_pos, step.tok_seq,
            cache.block_table, cache.k_pages, q_cat, self.H, self.dim, self.rot, self.rank,
        )
        if self.dim:
            ops.head_linear(q, self.dim + self.rot, self.w_ukT, q_cat.view(T, self.H * self.kvd), self.kvd)
        else:
            q_cat[:, :, : self.rank].zero_()
        if xn.dtype == torch.bfloat16 and ops.latent_attn_mma_takes(self.rank, self.rot):
            # tensor cores; a decode step cuts every sequence's keys into parts so that the GPU is filled once, none
            # shorter than two pages (planned from the step's page-table width, which a captured graph keeps)
            n_splits = 1
            if step.decode_only:
                blocks = step.n_seqs * ((self.H + 31) // 32 if self.H > 16 else 1)
                pages = max(1, (step.plan_kv_len + ops.PAGE_SIZE - 1) // ops.PAGE_SIZE)
                n_splits = max(1, min(sm_count(xn.device) // blocks, pages // 2, 64))
            scratch = None
            if n_splits > 1:
                scratch = self.rt.workspace.get("latent_attn", ops.latent_attn_mma_scratch_floats(T * self.H, self.rank, n_splits), torch.float32)
            o_lat = ops.latent_attn_mma(
                q_cat, cache.k_pages, cache.block_table, step.seq_start, step.seq_pos0, step.max_q_len, self.sink, self.rank, self.rot,
                self.scale, self.window, n_splits, scratch,
            )
        else:
            o_lat = ops.latent_attn(
                q_cat, cache.k_pages, cache.block_table, step.tok_seq, step.tok_pos, self.sink, self.rank, self.rot, self.scale, self.window,
            )
        a = torch.empty((T, self.vd), dtype=xn.dtype, device=xn.device)
        ops.head_linear(o_lat.view(T, self.H * self.rank), self.rank, self.w_uv, a, self.vdim, gate=g, gate_head_stride=self.vdim)
        return a, self.w_o
