"""Building blocks for decoder designs outside the Llama mould, and the ragged-batch model that runs them.

The reference has no counterpart (its graphs are models/llama.py and models/qwen3.py): these blocks carry designs whose
layers mix a recurrent state with windowed attention over a shared low-rank latent, with dense (unquantised) weights.

    Linear                  dense [out, in] weight                                 b200p_gemm
    HashedBigramEmbedding   token row * scale + a row picked by (previous, current)  b200p_embed_hashed
    GatedDeltaMixer         short convolutions + gated delta rule                   b200p_delta_prep / _conv_commit / _scan / _out
    LatentAttention         queries and keys/values through low-rank latents,       b200p_latent_prep / b200p_latent_attn
                            sliding window, optional sharing of another layer's latents
    ClampedGLU              g * sigmoid(1.702 g) * (u + 1) on clamped gate / up      b200p_gemm (fused epilogue)
    TokenSideInput          a small per-layer table indexed by the token, gated      b200p_token_gate
    SequenceModel           norm -> sublayer -> norm -> residual chain over a ragged batch (b200p_norm_add_norm)

A step is a ragged batch: entry e brings ``counts[e]`` tokens for cache row ``rows[e]``; prompts of different lengths are
packed back to back (no padding), decode steps bring one token per live row.  Every kernel works from the per-token plan
(row, position, offset in the portion), so the logits of a position do not depend on how the prompt was cut or on the
other rows.  Matrix products run in the model's storage type with fp32 accumulation; the residual stream, every norm,
softmax, the recurrence and what feeds it are fp32.  A float32 model runs true fp32 FMAs throughout.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .._lib import GEMM_GLU_CLAMP, GEMM_STORE, GEMM_STORE_F32
from .base import DeltaRuleState, LatentKVCache, RowState, TokenState

MAX_TOKENS_PER_FORWARD = 8192     # packed tokens of one pass through the layers


class Linear:
    """Dense linear layer, weight [out, in] in the model's storage type, applied as W x."""

    def __init__(self, in_features: int, out_features: int):
        self.in_features, self.out_features = in_features, out_features
        self.weight: Optional[torch.Tensor] = None

    def __call__(self, x, epilogue=GEMM_STORE, out=None, limit=0.0):
        return ops.gemm(x, self.weight, epilogue, out=out, limit=limit)


class Scratch:
    """Flat per-step buffers, sized for the largest layer, handed out as [M, n] views."""

    def __init__(self, device, rows: int):
        self.device, self.rows = device, rows
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self._need: Dict[tuple, int] = {}

    def reserve(self, name: str, dtype, cols: int):
        key = (name, dtype)
        self._need[key] = max(self._need.get(key, 0), cols)

    def allocate(self):
        for key, cols in self._need.items():
            self._bufs[key] = torch.empty((self.rows * cols,), dtype=key[1], device=self.device)

    def get(self, name: str, dtype, M: int, cols: int) -> torch.Tensor:
        return self._bufs[(name, dtype)][:M * cols].view(M, cols)


class GatedDeltaMixer:
    """Gated delta rule with short causal convolutions on q, k and v.

    q, k: ``kv_heads`` heads of ``dim``; v: ``heads`` heads of ``vdim``; head h reads q/k head h // (heads // kv_heads).
    Per head the fp32 state S [dim, vdim] goes S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with
    g = exp(-exp(A_log) softplus(a + dt_bias)) and beta = sigmoid(b).  o is rms-normed over vdim, weighted and gated by
    silu of a fifth projection before the output projection."""

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float):
        self.width, self.heads, self.kv_heads, self.dim, self.vdim, self.taps, self.eps = width, heads, kv_heads, dim, vdim, taps, eps
        self.c_qk = kv_heads * dim
        self.c_v = heads * vdim
        self.conv_channels = 2 * self.c_qk + self.c_v
        self.col_g = self.conv_channels
        self.col_b = self.col_g + self.c_v
        self.col_a = self.col_b + heads
        self.n_proj = self.col_a + heads
        self.in_proj = Linear(width, self.n_proj)            # rows [q | k | v | gate | b | a]
        self.o_proj = Linear(self.c_v, width)
        self.conv_w = self.A_log = self.dt_bias = self.norm_w = None     # fp32

    def new_state(self, batch_size: int) -> RowState:
        return DeltaRuleState(self.heads, self.dim, self.vdim, self.conv_channels, self.taps, batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.n_proj)
        s.reserve("qn", torch.float32, self.c_qk)
        s.reserve("kn", torch.float32, self.c_qk)
        s.reserve("v", torch.float32, self.c_v)
        s.reserve("beta", torch.float32, self.heads)
        s.reserve("decay", torch.float32, self.heads)
        s.reserve("o", torch.float32, self.c_v)
        s.reserve("mix", dt, self.c_v)

    def __call__(self, x, y_out, st: DeltaRuleState, plan: dict, s: Scratch, caches):
        M, dt, f32 = x.shape[0], x.dtype, torch.float32
        proj = self.in_proj(x, GEMM_STORE_F32, out=s.get("proj", f32, M, self.n_proj))
        qn, kn = s.get("qn", f32, M, self.c_qk), s.get("kn", f32, M, self.c_qk)
        v, o = s.get("v", f32, M, self.c_v), s.get("o", f32, M, self.c_v)
        beta, decay = s.get("beta", f32, M, self.heads), s.get("decay", f32, M, self.heads)
        ops.delta_prep(proj, self.col_b, self.col_a, self.conv_w, st.conv, self.A_log, self.dt_bias, plan["t_row"], plan["t_pos"],
                       plan["t_off"], qn, kn, v, beta, decay, self.heads, self.kv_heads, self.dim, self.vdim, self.taps)
        ops.delta_conv_commit(proj, st.conv, plan["cu"], plan["rows"], plan["nb"], self.conv_channels, self.taps)
        ops.delta_scan(qn, kn, v, beta, decay, st.state, plan["cu"], plan["rows"], plan["lengths"], o, plan["nb"], self.heads,
                       self.kv_heads, self.dim, self.vdim)
        mix = s.get("mix", dt, M, self.c_v)
        ops.delta_out(o, proj, self.col_g, self.norm_w, mix, self.heads, self.vdim, self.eps)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


class LatentAttention:
    """Attention whose queries and keys/values pass through low-rank latents; no positional rotation.

    c_q = rms_norm(W_dq x); q = W_uq c_q (``heads`` x ``dim``).  c = rms_norm(W_dkv x) (``kv_rank``) is the only thing cached;
    k = W_uk c, v = W_uv c per head.  Here the up-projections are folded around the attention: the query is carried into
    the latent space (W_uk^T q per head), the heads attend over c itself, and W_uv is applied to the attended latent.
    ``window`` > 0: position i sees j with 0 <= i - j < window.  ``kv_from``: index of the earlier layer whose latents this
    layer reads (it then has no W_dkv of its own)."""

    def __init__(self, width: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float, window: int,
                 eps: float, kv_from: Optional[int] = None):
        self.width, self.heads, self.dim, self.vdim = width, heads, dim, vdim
        self.q_rank, self.kv_rank, self.scale, self.window, self.eps, self.kv_from = q_rank, kv_rank, scale, window, eps, kv_from
        self.own_kv = kv_from is None
        self.down = Linear(width, q_rank + (kv_rank if self.own_kv else 0))      # rows [dq | dkv]
        self.uq = Linear(q_rank, heads * dim)
        self.uk_t: Optional[torch.Tensor] = None          # [heads, kv_rank, dim]: W_uk per head, transposed
        self.uv: Optional[torch.Tensor] = None            # [heads * vdim, kv_rank]
        self.o_proj = Linear(heads * vdim, width)
        self.q_norm_w = self.kv_norm_w = None             # fp32

    def new_state(self, batch_size: int) -> RowState:
        return LatentKVCache(self.kv_rank, batch_size) if self.own_kv else RowState(batch_size)

    def reserve(self, s: Scratch, dt):
        s.reserve("proj", torch.float32, self.down.out_features)
        s.reserve("cq", dt, self.q_rank)
        s.reserve("q", dt, self.heads * self.dim)
        s.reserve("qlat", torch.float32, self.heads * self.kv_rank)
        s.reserve("olat", dt, self.heads * self.kv_rank)
        s.reserve("mix", dt, self.heads * self.vdim)

    def __call__(self, x, y_out, st: RowState, plan: dict, s: Scratch, caches):
        M, dt, f32 = x.shape[0], x.dtype, torch.float32
        H, R, dk, dv = self.heads, self.kv_rank, self.dim, self.vdim
        proj = self.down(x, GEMM_STORE_F32, out=s.get("proj", f32, M, self.down.out_features))
        cq = s.get("cq", dt, M, self.q_rank)
        cache = st if self.own_kv else caches[self.kv_from]
        ops.latent_prep(proj, self.q_rank, R, self.q_norm_w, self.kv_norm_w, self.eps, cq, cache.latent if self.own_kv else None,
                        plan["t_row"], plan["t_pos"])
        q = self.uq(cq, GEMM_STORE, out=s.get("q", dt, M, H * dk))
        qlat = s.get("qlat", f32, M, H * R)
        ops.gemm(q, self.uk_t, GEMM_STORE_F32, out=qlat, batch=H, strides=(dk, R * dk, R), M=M, N=R, K=dk, ldx=H * dk, ldw=dk,
                 ldy=H * R)
        olat = s.get("olat", dt, M, H * R)
        ops.latent_attn(qlat, cache.latent, plan["t_row"], plan["t_pos"], olat, H, R, self.window, self.scale, cu=plan["cu"],
                        rows=plan["rows"], nb=plan["nb"], max_n=plan["max_n"])
        mix = s.get("mix", dt, M, H * dv)
        ops.gemm(olat, self.uv, GEMM_STORE, out=mix, batch=H, strides=(R, dv * R, dv), M=M, N=dv, K=R, ldx=H * R, ldw=R, ldy=H * dv)
        return self.o_proj(mix, GEMM_STORE_F32, out=y_out)


class ClampedGLU:
    """Feed-forward y = W_down (g * sigmoid(1.702 g) * (u + 1)), g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit).
    gate and up rows are interleaved in one matrix so that the GEMM epilogue holds both values of a hidden unit."""

    def __init__(self, width: int, ff: int, limit: float):
        self.width, self.ff, self.limit = width, ff, limit
        self.gate_up = Linear(width, 2 * ff)
        self.down = Linear(ff, width)

    def reserve(self, s: Scratch, dt):
        s.reserve("act", dt, self.ff)

    def __call__(self, x, y_out, s: Scratch):
        act = self.gate_up(x, GEMM_GLU_CLAMP, out=s.get("act", x.dtype, x.shape[0], self.ff), limit=self.limit)
        return self.down(act, GEMM_STORE_F32, out=y_out)


class TokenSideInput:
    """Per-layer token input: e = table[token, layer slice]; y = W_proj (gelu_tanh(W_gate x) * e), x the residual stream."""

    def __init__(self, width: int, dim: int, col0: int):
        self.width, self.dim, self.col0 = width, dim, col0
        self.gate = Linear(width, dim)
        self.proj = Linear(dim, width)

    def reserve(self, s: Scratch, dt):
        s.reserve("sgate", torch.float32, self.dim)
        s.reserve("sg", dt, self.dim)

    def __call__(self, x_raw, y_out, table, ids, s: Scratch):
        M = x_raw.shape[0]
        gate = self.gate(x_raw, GEMM_STORE_F32, out=s.get("sgate", torch.float32, M, self.dim))
        g = ops.token_gate(gate, table, ids, s.get("sg", x_raw.dtype, M, self.dim), self.col0)
        return self.proj(g, GEMM_STORE_F32, out=y_out)


class HashedBigramEmbedding:
    """x = embed[token] * scale + bigram[(prev * mul_prev + token * mul_cur) mod buckets]; the table's last row (index
    ``buckets``) serves a sequence's first token.  ``bigram`` may be absent."""

    def __init__(self, vocab: int, width: int, scale: float, buckets: int = 0, mul_prev: int = 0, mul_cur: int = 0):
        self.vocab, self.width, self.scale = vocab, width, scale
        self.buckets, self.mul_prev, self.mul_cur = buckets, mul_prev, mul_cur
        self.weight: Optional[torch.Tensor] = None
        self.bigram: Optional[torch.Tensor] = None


class Sublayer:
    """One residual branch: x <- x + post_norm(f(pre(x))); ``pre_w`` None means f reads the residual stream itself."""

    def __init__(self, kind: str, module, layer: int, pre_w_name: Optional[str], post_w_name: str):
        self.kind, self.module, self.layer = kind, module, layer
        self.pre_w_name, self.post_w_name = pre_w_name, post_w_name
        self.pre_w: Optional[torch.Tensor] = None
        self.post_w: Optional[torch.Tensor] = None


class SequenceModel:
    """callable(inputs [B, L], cache=None, last_only=False, prompt_lengths=None) -> float32 logits, like the other models,
    plus ``forward_ragged`` for prompts of unequal length and arbitrary logit positions.  Subclasses build ``self.embed``,
    ``self.sublayers`` (in execution order), ``self.mixers`` (one per layer), ``self.final_norm_w`` / ``self.lm_head`` and name
    their tensors in ``load_weights``."""

    supports_ragged = True
    dense = True                      # unquantised weights: no ``quantization`` block in config.json
    kernel_units = "sequence"         # key of _lib.UNIT_SETS: what a fresh checkout has to compile for this family

    def __init__(self, args):
        self.args = args
        self.model_type = args.model_type
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        self._arenas: Dict[tuple, dict] = {}
        self._lock = threading.RLock()
        self.tp_rank, self.tp_world = 0, 1
        self.embed: Optional[HashedBigramEmbedding] = None
        self.sublayers: List[Sublayer] = []
        self.mixers: list = []
        self.side_table: Optional[torch.Tensor] = None
        self.final_norm_w: Optional[torch.Tensor] = None
        self.lm_head: Optional[Linear] = None
        self.eps = 1e-6
        # debugging aid: callable(layer, kind, h [M, width]) run after every closed branch of an eager pass (never set it
        # while a decode step is being captured)
        self.residual_tap = None

    # -- surface shared with DecoderModel ---------------------------------------------------------------
    @property
    def layers(self):
        return self.mixers

    def eval(self):
        return self

    def graph_safe(self, B: int) -> bool:
        return True

    def greedy_tokens(self, logits, tok_out, probs_out=None):
        ops.argmax(logits, out=tok_out, probs_out=probs_out)

    def sample_tokens(self, logits, temp, top_p, seed, offset, tok_out, probs_out=None):
        ops.sample_top_p(logits, temp, top_p, seed, offset, out=tok_out, probs_out=probs_out)

    def set_tensor_parallel(self, rank, world, allreduce):
        if world > 1:
            raise NotImplementedError("tensor parallelism is not built for this model family")

    # -- state ----------------------------------------------------------------------------------------------
    def cache_key(self) -> tuple:
        return ("sequence", id(self))

    def new_cache(self, batch_size: int) -> List[RowState]:
        """One entry per layer (its mixer's state) and a last one for the previous token of every row."""
        return [m.new_state(batch_size) for m in self.mixers] + [TokenState(batch_size)]

    def make_cache(self, batch_size: int, step: Optional[int] = None, paged: bool = True) -> List[RowState]:
        from ._transformer import bind_cache_group
        caches = self.new_cache(batch_size)
        bind_cache_group(caches, self.device, step)
        return caches

    # -- scratch ----------------------------------------------------------------------------------------------
    def _arena(self, M: int, B: int, ragged: bool = False) -> dict:
        """Buffers for up to M packed tokens of B entries on the current stream.  The decode step's arena (M == B, not
        ``ragged``) has its plan inputs preset (one token per entry, rows 0..B-1 unless the caller rewrites ``rows``) so that
        a captured graph can replay over them; ragged passes rewrite theirs every time and use arenas of their own."""
        key = (M, B, ragged, torch.cuda.current_stream(self.device).cuda_stream)
        a = self._arenas.get(key)
        if a is None:
            dev, dt, W = self.device, self.dtype, self.args.width
            s = Scratch(dev, M)
            for m in self.mixers:
                m.reserve(s, dt)
            for sl in self.sublayers:
                if sl.kind != "mixer":
                    sl.module.reserve(s, dt)
            s.reserve("y", torch.float32, W)
            s.reserve("x", dt, W)
            s.reserve("xl", dt, W)
            s.allocate()
            i32 = dict(dtype=torch.int32, device=dev)
            a = dict(
                s=s, cap=M,
                h=torch.empty((M, W), dtype=torch.float32, device=dev),
                ids=torch.zeros((M,), **i32), t_row=torch.zeros((M,), **i32), t_pos=torch.zeros((M,), **i32),
                t_off=torch.zeros((M,), **i32),
                cu=torch.arange(B + 1, **i32) if not ragged else torch.zeros((B + 1,), **i32),
                rows=torch.arange(B, **i32),
            )
            if len(self._arenas) > 8:
                self._arenas.clear()
            self._arenas[key] = a
        return a

    # -- forward ----------------------------------------------------------------------------------------------
    def _layers_forward(self, ids_i32: torch.Tensor, B: int, L: int, cache: List[RowState], a: dict, M: Optional[int] = None,
                        max_n: int = 1):
        """Run the packed tokens ``ids_i32`` ([M]) of the B entries described by a["cu"] / a["rows"] through every layer;
        the residual stream is left in a["h"][:M].  (L is 1 for a decode step and unused otherwise: entries are ragged;
        ``max_n`` is the longest entry's token count, which picks prompt or decode kernels.)"""
        M = ids_i32.numel() if M is None else M
        s: Scratch = a["s"]
        dt, W = self.dtype, self.args.width
        lengths = cache[-1].lengths(self.device)
        plan = dict(cu=a["cu"], rows=a["rows"], nb=B, lengths=lengths, max_n=max_n, t_row=a["t_row"][:M], t_pos=a["t_pos"][:M], t_off=a["t_off"][:M])
        ops.ragged_plan(a["cu"], a["rows"], lengths, plan["t_row"], plan["t_pos"], plan["t_off"], B, M)
        e = self.embed
        h = a["h"][:M]
        ops.embed_hashed(ids_i32, plan["t_row"], plan["t_pos"], plan["t_off"], cache[-1].last_token, e.weight, e.bigram, h, e.scale,
                         e.buckets, e.mul_prev, e.mul_cur)
        x, y = s.get("x", dt, M, W), s.get("y", torch.float32, M, W)
        subs = self.sublayers

        def feed(nxt: Optional[Sublayer], y_in, post_w):
            """Close a branch (h += post_norm(y)) and prepare the input of the next one in the same pass over the row."""
            pre = nxt.pre_w if nxt is not None else None
            raw = nxt is not None and nxt.pre_w is None
            ops.norm_add_norm(h, self.eps, dt, y=y_in, w_post=post_w, w_next=pre, x_out=x if pre is not None else None,
                              raw_out=x if raw else None)

        feed(subs[0] if subs else None, None, None)
        for i, sl in enumerate(subs):
            if sl.kind == "mixer":
                sl.module(x, y, cache[sl.layer], plan, s, cache)
            elif sl.kind == "mlp":
                sl.module(x, y, s)
            else:
                sl.module(x, y, self.side_table, ids_i32, s)
            feed(subs[i + 1] if i + 1 < len(subs) else None, y, sl.post_w)
            if self.residual_tap is not None:
                self.residual_tap(sl.layer, sl.kind, h)

    def _advance_device(self, cache: List[RowState], a: dict, B: int, ids_i32: Optional[torch.Tensor] = None):
        """End of a step on the device: lengths += tokens brought, last token of every entry remembered."""
        ops.ragged_advance(cache[-1]._lengths, cache[-1].last_token, a["ids"] if ids_i32 is None else ids_i32, a["cu"], a["rows"], B)

    def _head(self, h_rows: torch.Tensor, a: dict, logits_out: Optional[torch.Tensor] = None, x_rows=None):
        """final norm + output projection of the given residual rows -> float32 logits."""
        n = h_rows.shape[0]
        xl = a["s"].get("xl", self.dtype, n, self.args.width)
        ops.norm_add_norm(h_rows, self.eps, self.dtype, w_next=self.final_norm_w, x_out=xl)
        return self.lm_head(xl, GEMM_STORE_F32, out=logits_out)

    def forward_ragged(self, seqs: Sequence[Sequence[int]], cache: List[RowState], rows: Optional[Sequence[int]] = None,
                       want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Feed entry i's tokens ``seqs[i]`` to cache row ``rows[i]`` (default i), continuing whatever the row holds.
        ``want[i]``: offsets into seqs[i] whose logits are returned (default: the last token of every non-empty entry), in
        entry order -> float32 [n_wanted, vocab]."""
        with self._lock:
            return self._forward_ragged_locked(seqs, cache, rows, want)

    def _forward_ragged_locked(self, seqs, cache, rows, want):
        from ._transformer import advance_rows, prepare_rows
        nb = len(seqs)
        rows = list(range(nb)) if rows is None else [int(r) for r in rows]
        if len(set(rows)) != nb or any(r < 0 or r >= cache[-1].batch_size for r in rows):
            raise ValueError("rows must be distinct rows of the cache")
        if want is None:
            want = [[len(q) - 1] if len(q) else [] for q in seqs]
        counts = [len(q) for q in seqs]
        dev = self.device
        outs = [[None] * len(w) for w in want]
        done = [0] * nb
        while True:
            # one pass: every entry brings its next tokens, the pass holds at most MAX_TOKENS_PER_FORWARD of them
            left = [counts[i] - done[i] for i in range(nb)]
            live = sum(1 for n in left if n > 0)
            if live == 0:
                break
            share = max(1, MAX_TOKENS_PER_FORWARD // live)
            take = [min(n, share) for n in left]
            M = sum(take)
            prepare_rows(cache, rows, take, self.dtype, dev)
            a = self._arena(_round_up_rows(M), nb, ragged=True)
            flat, cu = [], [0]
            for i in range(nb):
                flat.extend(seqs[i][done[i]:done[i] + take[i]])
                cu.append(cu[-1] + take[i])
            ids = a["ids"][:M]
            ids.copy_(torch.tensor(flat, dtype=torch.int32), non_blocking=False)
            a["cu"].copy_(torch.tensor(cu, dtype=torch.int32))
            a["rows"].copy_(torch.tensor(rows, dtype=torch.int32))
            self._layers_forward(ids, nb, 0, cache, a, M, max_n=max(take))
            self._advance_device(cache, a, nb, ids)
            advance_rows(cache, rows, take)
            pick, where = [], []
            for i in range(nb):
                for k, p in enumerate(want[i]):
                    if done[i] <= p < done[i] + take[i]:
                        pick.append(cu[i] + p - done[i])
                        where.append((i, k))
            if pick:
                hs = a["h"][:M].index_select(0, torch.tensor(pick, dtype=torch.int64, device=dev))
                lg = self._head(hs, a)
                for j, (i, k) in enumerate(where):
                    outs[i][k] = lg[j]
            for i in range(nb):
                done[i] += take[i]
        flat_out = [t for o in outs for t in o]
        if any(t is None for t in flat_out):
            raise ValueError("a wanted position lies outside its entry's tokens")
        V = self.lm_head.out_features
        return torch.stack(flat_out, 0) if flat_out else torch.empty((0, V), dtype=torch.float32, device=dev)

    def __call__(self, inputs, cache: Optional[List[RowState]] = None, last_only: bool = False, prompt_lengths=None):
        """inputs int [B, L] -> logits float32 [B, L, V] (or [B, 1, V] with last_only).  ``prompt_lengths[b]`` < L marks the
        first L - prompt_lengths[b] ids of row b as left padding: they are not fed to the model at all, and with
        last_only=False their logits are zero."""
        if not isinstance(inputs, torch.Tensor):
            inputs = torch.as_tensor(inputs)
        B, L = inputs.shape
        host = inputs.tolist()
        n = [L] * B if prompt_lengths is None else [int(v) for v in prompt_lengths]
        seqs = [host[b][L - n[b]:] for b in range(B)]
        if cache is None:
            cache = self.make_cache(B, step=max(L, 1))
        if last_only:
            return self.forward_ragged(seqs, cache).view(B, 1, -1)
        lg = self.forward_ragged(seqs, cache, want=[list(range(k)) for k in n])
        out = torch.zeros((B, L, lg.shape[-1]), dtype=torch.float32, device=lg.device)
        o = 0
        for b in range(B):
            out[b, L - n[b]:] = lg[o:o + n[b]]
            o += n[b]
        return out

    def release_rows(self, cache: List[RowState], rows: Sequence[int]):
        """Give rows back to the cache: the next sequence in them starts from nothing."""
        from ._transformer import release_rows
        with self._lock:
            release_rows(cache, [int(r) for r in rows])


def _round_up_rows(M: int) -> int:
    """Arena capacity for M packed tokens: powers of two from 64, so prompts of nearby sizes share scratch."""
    c = 64
    while c < M:
        c *= 2
    return c
