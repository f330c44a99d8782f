"""Pupopel: a decoder whose layers add a mixer and a feed-forward that read ONE norm, with a span of layers that can run
several times on the same weights.

config.json (``"architecture": "Pupopel"``) lists the layers one by one -- ``type``, the mixer's sizes, its feed-forward (or
null) -- and gives every size and constant; tensors are named ``l<i>.<part>``.

    layer         x <- x + (mixer(n) + ff(n)), n = rms_norm(x) * (1 + w)             (the stored norm weights are offsets from one)
    loop          layers start .. stop-1 run ``times`` times; every pass has its own states and opens with
                  x <- W_in [x ; embedding]
    channel_delta gated delta rule with short convolutions, ONE DECAY PER KEY CHANNEL, decay and gate through low-rank pairs
                  of matrices (their inner size is read from the tensors), sigmoid gate
    parallel      two mixers side by side on the same input: attention with normed q / k, a logarithmic query temperature, a
                  distance bias 2^(-8 (h+1) / H) (i - j) and a sink in the softmax; and linear attention with constant decays
    feed-forward  dense (gelu_tanh gate) or routed experts (silu gate; softmax over the chosen logits) with a shared expert

The reference has no such graph; the blocks are in models/_sequence.py and run on the ragged-batch kernels of the library.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from ._sequence import (DecayLinearAttention, GatedDeltaMixer, GatedFF, HashedBigramEmbedding, LayerRun, Linear, RoutedExperts,
                        SequenceModel, SideBySideMixer, SinkAttention, unroll_layers)
from .base import BaseModelArgs

DISTANCE_SLOPE_LOG2 = -8.0        # head h of H: slope 2^(-8 (h + 1) / H)


@dataclass
class ModelArgs(BaseModelArgs):
    vocab: int
    width: int
    layers: List[Dict[str, Any]]
    norm: Dict[str, Any] = field(default_factory=dict)
    loop: Optional[Dict[str, Any]] = None
    architecture: str = "Pupopel"
    model_type: str = "pupopel"

    def __post_init__(self):
        if not self.layers:
            raise ValueError("config 'layers' is empty")
        for i, L in enumerate(self.layers):
            if L.get("type") not in ("channel_delta", "parallel"):
                raise NotImplementedError(f"layer {i}: mixer type {L.get('type')!r} is not part of this design")
            mlp = L.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not part of this design")
            m = L["mixer"]
            for part in ([m] if L["type"] == "channel_delta" else [m["left"]]):
                if part["heads"] % part.get("kv_heads", part["heads"]):
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
        if self.loop:
            a, b, n = int(self.loop["start"]), int(self.loop["stop"]), int(self.loop["times"])
            if not (0 <= a <= b <= len(self.layers)) or n < 1:
                raise ValueError("loop: 0 <= start <= stop <= number of layers and times >= 1")

    @property
    def vocab_size(self) -> int:
        return self.vocab


class Model(SequenceModel):
    block_style = "parallel"
    kernel_units = "sequence_moe"

    def __init__(self, args: ModelArgs):
        super().__init__(args)
        W = args.width
        self.eps = float(args.norm.get("eps", 1e-6))
        self.embed = HashedBigramEmbedding(args.vocab, W, 1.0)
        blocks = []
        for L in args.layers:
            m = L["mixer"]
            if L["type"] == "channel_delta":
                mixer = GatedDeltaMixer(W, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], int(m.get("conv", 1)), self.eps,
                                        channel_decay=True, decay_rank=None, gate_rank=None, gate_act="sigmoid")
            else:
                a, b = m["left"], m["right"]
                qt = a.get("q_temp") or {}
                left = SinkAttention(a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a["vdim"], float(a["scale"]), self.eps,
                                     qk_norm=True, temp_coef=float(qt.get("coef", 0.0)), temp_every=float(qt.get("every", 1)),
                                     slope_log2=DISTANCE_SLOPE_LOG2, sink=True)
                right = DecayLinearAttention(b["heads"], b["dim"], b["vdim"], b["decay"], self.eps)
                mixer = SideBySideMixer(W, [left, right], [float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))])
            mlp = L.get("mlp")
            if mlp is None:
                ff = None
            elif mlp["kind"] == "dense":
                ff = GatedFF(W, int(mlp["ff"]), "gelu_tanh")
            else:
                shared = mlp.get("shared") or {}
                ff = RoutedExperts(W, int(mlp["router"]["experts"]), int(mlp["router"]["top"]), int(mlp["expert"]["ff"]), "silu",
                                   shared_ff=int(shared.get("ff", 0)))
            blocks.append((mixer, ff))
        self.mixers = [b[0] for b in blocks]
        loop = args.loop or {}
        order = unroll_layers(len(blocks), int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1)))
        for slot, (i, opens) in enumerate(order):
            self.runs.append(LayerRun(i, slot, blocks[i][0], blocks[i][1], f"l{i}.norm1", opens))
        if any(r.opens for r in self.runs):
            self.loop_in = Linear(2 * W, W)
        self.lm_head = Linear(W, args.vocab)

    # -- parameters ------------------------------------------------------------------------------------------
    @staticmethod
    def _glu_names(prefix: str) -> List[str]:
        return [prefix + "gate", prefix + "up", prefix + "down"]

    def parameter_names(self) -> List[str]:
        names = ["embed", "final.norm", "head"]
        if self.loop_in is not None:
            names.append("loop.in")
        for i, L in enumerate(self.args.layers):
            p = f"l{i}."
            names.append(p + "norm1")
            if L["type"] == "channel_delta":
                names += [p + "mix." + n for n in ("q", "q.conv", "k", "k.conv", "v", "v.conv", "b", "A_log", "norm", "a1", "a2",
                                                   "dt_bias", "g1", "g2", "o")]
            else:
                names += [p + "mix.left." + n for n in ("q", "k", "v", "q.norm", "k.norm", "sink", "o")]
                names += [p + "mix.right." + n for n in ("q", "k", "v", "g", "o", "norm")]
            mlp = L.get("mlp")
            if mlp is None:
                continue
            if mlp["kind"] == "dense":
                names += self._glu_names(p + "mlp.")
            else:
                for e in range(int(mlp["router"]["experts"])):
                    names += self._glu_names(f"{p}mlp.e{e}.")
                names += [p + "mlp.router", p + "mlp.router.b"]
                if (mlp.get("shared") or {}).get("ff"):
                    names += self._glu_names(p + "mlp.shared.")
        return names

    def load_weights(self, weights: Dict[str, torch.Tensor], device="cuda", strict: bool = True, dtype=None):
        """Matrices go to the device in ``dtype`` (default: as stored); vectors (norm weights, convolution taps, decay
        parameters, sinks, router biases) as float32, the norm weights with their one added.  Projections that read the same
        input are stacked into one matrix, gate / up rows interleaved for the fused epilogue, the experts stacked per layer."""
        device = torch.device(device)
        missing = [n for n in self.parameter_names() if n not in weights]
        if missing:
            raise KeyError(f"missing parameters: {missing[:4]}{'...' if len(missing) > 4 else ''}")
        if dtype is None:
            dtype = weights["embed"].dtype
        if dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise TypeError(f"unsupported storage dtype {dtype}")
        self.dtype, self.device = dtype, device

        def put(t):
            return t.to(device=device, dtype=dtype).contiguous()

        def vec(name, shape=None, one_plus=False):
            t = weights[name].float()
            if shape is not None:
                check(name, shape)
            return ((1.0 + t) if one_plus else t).to(device).contiguous()

        def check(name, shape):
            if tuple(weights[name].shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(weights[name].shape)} does not match the config ({tuple(shape)})")

        def glu(ff: GatedFF, prefix: str):
            check(prefix + "gate", (ff.ff, W))
            check(prefix + "up", (ff.ff, W))
            check(prefix + "down", (W, ff.ff))
            ff.gate_up.weight = put(GatedFF.interleave(weights[prefix + "gate"], weights[prefix + "up"]))
            ff.down.weight = put(weights[prefix + "down"])

        a, W = self.args, self.args.width
        check("embed", (a.vocab, W))
        check("head", (a.vocab, W))
        self.embed.weight = put(weights["embed"])
        self.final_norm_w = vec("final.norm", (W,), one_plus=True)
        self.lm_head.weight = put(weights["head"])
        if self.loop_in is not None:
            check("loop.in", (W, 2 * W))
            self.loop_in.weight = put(weights["loop.in"])
        norm_w = {}
        for i, (L, m) in enumerate(zip(a.layers, self.mixers)):
            p = f"l{i}.mix."
            norm_w[i] = vec(f"l{i}.norm1", (W,), one_plus=True)
            if isinstance(m, GatedDeltaMixer):
                check(p + "q", (m.c_qk, W))
                check(p + "k", (m.c_qk, W))
                check(p + "v", (m.c_v, W))
                check(p + "b", (m.heads, W))
                r_a, r_g = weights[p + "a1"].shape[0], weights[p + "g1"].shape[0]
                check(p + "a1", (r_a, W))
                check(p + "a2", (m.n_decay, r_a))
                check(p + "g1", (r_g, W))
                check(p + "g2", (m.c_v, r_g))
                m.set_ranks(r_a, r_g)
                m.in_proj.weight = put(m.stack_in_proj(*(weights[p + n] for n in ("q", "k", "v", "b", "g1", "a1"))))
                m.decay_up.weight, m.gate_up.weight = put(weights[p + "a2"]), put(weights[p + "g2"])
                m.o_proj.weight = put(weights[p + "o"])
                for n, rows in (("q.conv", m.c_qk), ("k.conv", m.c_qk), ("v.conv", m.c_v)):
                    check(p + n, (rows, m.taps))
                m.conv_w = torch.cat([weights[p + n].float() for n in ("q.conv", "k.conv", "v.conv")], 0).to(device).contiguous()
                m.A_log, m.dt_bias = vec(p + "A_log", (m.heads,)), vec(p + "dt_bias", (m.n_decay,))
                m.norm_w = vec(p + "norm", (m.vdim,))
            else:
                left, right = m.branches
                lp, rp = p + "left.", p + "right."
                check(lp + "q", (left.heads * left.dim, W))
                check(lp + "k", (left.kv_heads * left.dim, W))
                check(lp + "v", (left.kv_heads * left.vdim, W))
                check(lp + "o", (W, left.n_mix))
                check(rp + "q", (right.c_qk, W))
                check(rp + "k", (right.c_qk, W))
                check(rp + "v", (right.c_v, W))
                check(rp + "g", (right.c_v, W))
                check(rp + "o", (W, right.n_mix))
                m.in_proj.weight = put(m.stack_in_proj([torch.cat([weights[lp + n] for n in ("q", "k", "v")], 0),
                                                        torch.cat([weights[rp + n] for n in ("q", "k", "v", "g")], 0)]))
                m.o_proj.weight = put(m.stack_o_proj([weights[lp + "o"], weights[rp + "o"]]))
                left.q_norm_w, left.k_norm_w = vec(lp + "q.norm", (left.dim,)), vec(lp + "k.norm", (left.dim,))
                left.sink = vec(lp + "sink", (left.heads,))
                right.norm_w = vec(rp + "norm", (right.c_v,))
                right.decay = torch.tensor(right.decay_values, dtype=torch.float32, device=device)
        seen = set()
        for r in self.runs:
            r.norm_w = norm_w[r.layer]
            ff = r.mlp
            if ff is None or r.layer in seen:
                continue
            seen.add(r.layer)
            q = f"l{r.layer}.mlp."
            if isinstance(ff, GatedFF):
                glu(ff, q)
            else:
                check(q + "router", (ff.experts, W))
                ff.router.weight = put(weights[q + "router"])
                ff.router_bias = vec(q + "router.b", (ff.experts,))
                for e in range(ff.experts):
                    check(f"{q}e{e}.gate", (ff.ff, W))
                    check(f"{q}e{e}.down", (W, ff.ff))
                ff.gate_up = put(torch.stack([GatedFF.interleave(weights[f"{q}e{e}.gate"], weights[f"{q}e{e}.up"])
                                              for e in range(ff.experts)], 0))
                ff.down = put(torch.stack([weights[f"{q}e{e}.down"] for e in range(ff.experts)], 0))
                if ff.shared is not None:
                    glu(ff.shared, q + "shared.")
        self._arenas.clear()
        return self
