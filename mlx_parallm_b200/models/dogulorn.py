"""Dogulorn: a decoder whose layers alternate a gated-delta-rule mixer with sliding-window latent attention.

config.json (``"architecture": "Dogulorn"``) lists the layers one by one -- ``type`` (``delta`` / ``latent_attention``), the
mixer's sizes and its feed-forward (or null) -- and gives every size and constant; tensors are named ``l<i>.<part>``.  Each
sublayer is wrapped in a norm on both sides, x <- x + norm_b(f(norm(x))), and after a layer's sublayers a per-layer token input
is added the same way.  The embedding adds a hashed bigram row.  The reference has no such graph; the blocks are in
models/_sequence.py and run on the ragged-batch kernels of the library.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ._sequence import (ClampedGLU, GatedDeltaMixer, HashedBigramEmbedding, LatentAttention, Linear, SequenceModel, Sublayer,
                        TokenSideInput)
from .base import BaseModelArgs


@dataclass
class ModelArgs(BaseModelArgs):
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    embedding: Dict[str, Any] = field(default_factory=dict)
    norm: Dict[str, Any] = field(default_factory=dict)
    token_side: Optional[Dict[str, Any]] = None
    architecture: str = "Dogulorn"
    model_type: str = "dogulorn"

    def __post_init__(self):
        if not self.layers:
            raise ValueError("config 'layers' is empty")
        kind = str(self.norm.get("kind", self.norm.get("type", "rms"))).lower().replace("_", "").replace("norm", "")
        extra = set(self.norm) - {"eps", "kind", "type"}
        if extra or kind != "rms":
            raise NotImplementedError(f"norm options {sorted(extra) or kind!r} are not part of this design (an rms norm with a weight)")
        for i, L in enumerate(self.layers):
            if L.get("type") not in ("delta", "latent_attention"):
                raise NotImplementedError(f"layer {i}: mixer type {L.get('type')!r} is not part of this design")
            mlp = L.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
            kv_from = L["mixer"].get("kv_from")
            if kv_from is not None:
                src = self.layers[kv_from] if 0 <= kv_from < i else None
                if src is None or src["type"] != "latent_attention" or src["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer with latents of its own")
                if src["mixer"]["kv_rank"] != L["mixer"]["kv_rank"]:
                    raise ValueError(f"layer {i}: kv_rank differs from layer {kv_from}, whose latents it reads")

    @property
    def vocab_size(self) -> int:
        return self.vocab


class Model(SequenceModel):
    def __init__(self, args: ModelArgs):
        super().__init__(args)
        W = args.width
        self.eps = float(args.norm.get("eps", 1e-6))
        emb = args.embedding or {}
        big = emb.get("bigram") or {}
        self.embed = HashedBigramEmbedding(args.vocab, W, float(emb.get("scale", 1.0)), int(big.get("buckets", 0)),
                                           int(big.get("mul_prev", 0)), int(big.get("mul_cur", 0)))
        side_dim = int(args.token_side["dim"]) if args.token_side else 0
        for i, L in enumerate(args.layers):
            m = L["mixer"]
            if L["type"] == "delta":
                mixer = GatedDeltaMixer(W, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m.get("conv", 1), self.eps)
            else:
                mask = m.get("mask") or {}
                mixer = LatentAttention(W, m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"],
                                        float(m.get("scale", m["dim"] ** -0.5)), int(mask.get("size") or 0), self.eps,
                                        m.get("kv_from"))
            self.mixers.append(mixer)
            self.sublayers.append(Sublayer("mixer", mixer, i, f"l{i}.norm1", f"l{i}.norm1b"))
            if L.get("mlp") is not None:
                self.sublayers.append(Sublayer("mlp", ClampedGLU(W, L["mlp"]["ff"], float(L["mlp"]["limit"])), i, f"l{i}.norm2",
                                               f"l{i}.norm2b"))
            if side_dim:
                self.sublayers.append(Sublayer("side", TokenSideInput(W, side_dim, i * side_dim), i, None, f"l{i}.side.norm"))
        self.lm_head = Linear(W, args.vocab)

    # -- parameters ------------------------------------------------------------------------------------------
    def parameter_names(self) -> List[str]:
        names = ["embed", "final.norm", "head"]
        if self.embed.buckets:
            names.append("bigram")
        if self.args.token_side:
            names.append("side.embed")
        for sl in self.sublayers:
            p = f"l{sl.layer}."
            names += [n for n in (sl.pre_w_name, sl.post_w_name) if n]
            if sl.kind == "mlp":
                names += [p + "mlp.gate", p + "mlp.up", p + "mlp.down"]
            elif sl.kind == "side":
                names += [p + "side.gate", p + "side.proj"]
            elif isinstance(sl.module, GatedDeltaMixer):
                names += [p + "mix." + n for n in ("q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "a", "A_log", "dt_bias", "g",
                                                   "norm", "o")]
            else:
                names += [p + "mix." + n for n in ("dq", "dq.norm", "uq", "uk", "uv", "o")]
                if sl.module.own_kv:
                    names += [p + "mix.dkv", p + "mix.dkv.norm"]
        return names

    def load_weights(self, weights: Dict[str, torch.Tensor], device="cuda", strict: bool = True, dtype=None):
        """Matrices go to the device in ``dtype`` (default: as stored); vectors (norm weights, convolution taps, decay
        parameters) as float32.  Projections that read the same input are stacked into one matrix; the per-head key
        up-projection is stored transposed for the folded attention."""
        device = torch.device(device)
        missing = [n for n in self.parameter_names() if n not in weights]
        if missing:
            raise KeyError(f"missing parameters: {missing[:4]}{'...' if len(missing) > 4 else ''}")
        if dtype is None:
            dtype = weights["embed"].dtype
        if dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise TypeError(f"unsupported storage dtype {dtype}")
        self.dtype, self.device = dtype, device

        def mat(*names):
            ts = [weights[n] for n in names]
            t = ts[0] if len(ts) == 1 else torch.cat(ts, 0)
            return t.to(device=device, dtype=dtype).contiguous()

        def vec(*names):
            ts = [weights[n].float() for n in names]
            return (ts[0] if len(ts) == 1 else torch.cat(ts, 0)).to(device).contiguous()

        def check(name, shape):
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(weights[name].shape)} does not match the config ({tuple(shape)})")

        a, W = self.args, self.args.width
        check("embed", (a.vocab, W))
        check("head", (a.vocab, W))
        self.embed.weight = mat("embed")
        if self.embed.buckets:
            check("bigram", (self.embed.buckets + 1, W))
            self.embed.bigram = mat("bigram")
        if a.token_side:
            check("side.embed", (a.vocab, len(a.layers) * int(a.token_side["dim"])))
            self.side_table = mat("side.embed")
        self.final_norm_w = vec("final.norm")
        self.lm_head.weight = mat("head")
        for sl in self.sublayers:
            p = f"l{sl.layer}."
            sl.pre_w = vec(sl.pre_w_name) if sl.pre_w_name else None
            sl.post_w = vec(sl.post_w_name)
            m = sl.module
            if sl.kind == "mlp":
                check(p + "mlp.gate", (m.ff, W))
                gu = torch.stack([weights[p + "mlp.gate"], weights[p + "mlp.up"]], 1).reshape(2 * m.ff, W)     # rows g0 u0 g1 u1 ..
                m.gate_up.weight = gu.to(device=device, dtype=dtype).contiguous()
                m.down.weight = mat(p + "mlp.down")
            elif sl.kind == "side":
                check(p + "side.gate", (m.dim, W))
                m.gate.weight, m.proj.weight = mat(p + "side.gate"), mat(p + "side.proj")
            elif isinstance(m, GatedDeltaMixer):
                q = p + "mix."
                check(q + "q", (m.c_qk, W))
                check(q + "v", (m.c_v, W))
                check(q + "q.conv", (m.c_qk, m.taps))
                m.in_proj.weight = mat(q + "q", q + "k", q + "v", q + "b", q + "g", q + "a")
                m.o_proj.weight = mat(q + "o")
                m.conv_w = vec(q + "q.conv", q + "k.conv", q + "v.conv")
                m.A_log, m.dt_bias, m.norm_w = vec(q + "A_log"), vec(q + "dt_bias"), vec(q + "norm")
            else:
                q = p + "mix."
                check(q + "dq", (m.q_rank, W))
                check(q + "uk", (m.heads * m.dim, m.kv_rank))
                check(q + "uv", (m.heads * m.vdim, m.kv_rank))
                m.down.weight = mat(q + "dq", q + "dkv") if m.own_kv else mat(q + "dq")
                m.q_norm_w = vec(q + "dq.norm")
                m.kv_norm_w = vec(q + "dkv.norm") if m.own_kv else None
                m.uq.weight = mat(q + "uq")
                uk = weights[q + "uk"].view(m.heads, m.dim, m.kv_rank).transpose(1, 2)
                m.uk_t = uk.to(device=device, dtype=dtype).contiguous()
                m.uv = mat(q + "uv")
                m.o_proj.weight = mat(q + "o")
        self._arenas.clear()
        return self
