"""Slow float64 statement of the Pupopel design, one function per mechanism, whole sequences on the CPU.

Written from the design's equations; shares no code with mlx_parallm_b200 (it does not import it).  Notation: T tokens,
W width, x the residual stream [T, W], weights ``P[name]`` stored [out, in] and applied as a @ P.T.

The design: layers of one norm and two branches that both read it, x <- x + mixer(n(x)) + ff(n(x)); a span of layers that
runs several times on the same weights, each pass opened by a linear map of [x ; embedding]; two mixers (a delta rule whose
decay is per key channel, and an attention head group with a sink beside a constant-decay linear attention); feed-forwards
that are dense or a routed mixture with a shared expert.
"""
import math

import torch

F64 = torch.float64


# ---- elementwise --------------------------------------------------------------------------------------------------------
def rms_unit(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """rms norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv_silu(u, taps_w):
    """Per channel c: silu(sum_j taps_w[c, j] * u[t - (n - 1 - j), c]), zeros before the start; u [T, C], taps_w [C, n]."""
    T, C = u.shape
    n = taps_w.shape[1]
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(n):
            s = t - (n - 1 - j)
            if s >= 0:
                out[t] += taps_w[:, j] * u[s]
    return silu(out)


# ---- mixers -------------------------------------------------------------------------------------------------------------
def channel_delta(h, P, pre, m, eps):
    """Delta rule with one decay per head and key channel.  Per head, state S [dk, dv] from zero:
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ P[pre + "q"].T, P[pre + "q.conv"]).view(T, G, dk)
    k = short_conv_silu(h @ P[pre + "k"].T, P[pre + "k.conv"]).view(T, G, dk)
    v = short_conv_silu(h @ P[pre + "v"].T, P[pre + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P[pre + "b"].T)                                                       # [T, H]
    step = torch.nn.functional.softplus((h @ P[pre + "a1"].T) @ P[pre + "a2"].T + P[pre + "dt_bias"]).view(T, H, dk)
    g = torch.exp(-torch.exp(P[pre + "A_log"]).view(1, H, 1) * step)                                # [T, H, dk]
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        kv = head // (H // G)
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = g[t, head].unsqueeze(1) * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    gate = torch.sigmoid((h @ P[pre + "g1"].T) @ P[pre + "g2"].T).view(T, H, dv)
    out = rms_unit(out, eps) * P[pre + "norm"] * gate
    return out.reshape(T, H * dv) @ P[pre + "o"].T


def sink_attention(h, P, pre, m, eps):
    """Causal attention without rotation: per-head rms norm of q and k, a query temperature that grows with the logarithm
    of the position block, a bias linear in the distance, and one extra term exp(sink) in the softmax denominator."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit((h @ P[pre + "q"].T).view(T, H, dk), eps) * P[pre + "q.norm"]
    k = rms_unit((h @ P[pre + "k"].T).view(T, G, dk), eps) * P[pre + "k.norm"]
    v = (h @ P[pre + "v"].T).view(T, G, dv)
    qt = m.get("q_temp")
    if qt:
        pos = torch.arange(T, dtype=F64)
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((pos + 1) / qt["every"]) + 1.0)).view(T, 1, 1)
    out = torch.zeros(T, H, dv, dtype=F64)
    i = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    for head in range(H):
        kv = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        s = (q[:, head] @ k[:, kv].T) * m["scale"] - slope * (i - j).to(F64)
        s = s.masked_fill(j > i, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, P[pre + "sink"][head])
        e = torch.exp(s - top)
        out[:, head] = (e @ v[:, kv]) / (e.sum(-1, keepdim=True) + torch.exp(P[pre + "sink"][head] - top))
    return out.reshape(T, H * dv) @ P[pre + "o"].T


def decay_linear_attention(h, P, pre, m, eps):
    """Per head S_t = lambda S_{t-1} + k_t v_t^T, o_t = S_t^T q_t with q, k, v = silu of their projections; all heads
    rms-normed as one vector, gated by a sigmoid."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ P[pre + "q"].T).view(T, H, dk)
    k = silu(h @ P[pre + "k"].T).view(T, H, dk)
    v = silu(h @ P[pre + "v"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    o = rms_unit(out.reshape(T, H * dv), eps) * P[pre + "norm"] * torch.sigmoid(h @ P[pre + "g"].T)
    return o @ P[pre + "o"].T


def side_by_side(h, P, pre, m, eps):
    return (m["left_scale"] * sink_attention(h, P, pre + "left.", m["left"], eps)
            + m["right_scale"] * decay_linear_attention(h, P, pre + "right.", m["right"], eps))


# ---- feed-forwards ------------------------------------------------------------------------------------------------------
def glu(h, P, pre, act):
    return (act(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def routed_experts(h, P, pre, mlp, chosen=None):
    """Each token goes to the ``top`` experts of largest router logit, weighted by the softmax over those logits alone; a
    shared expert is added for every token.  ``chosen`` (optional list) receives the picked expert ids per token."""
    r = mlp["router"]
    z = h @ P[pre + "router"].T + P[pre + "router.b"]
    out = torch.zeros(h.shape[0], P[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        idx = torch.topk(z[t], r["top"]).indices
        wts = torch.softmax(z[t, idx], 0)
        if chosen is not None:
            chosen.append(sorted(idx.tolist()))
        for e, wt in zip(idx.tolist(), wts):
            out[t] += wt * glu(h[t:t + 1], P, f"{pre}e{e}.", silu)[0]
    if mlp.get("shared"):
        out = out + glu(h, P, pre + "shared.", silu)
    return out


def feed_forward(h, P, pre, mlp):
    if mlp is None:
        return torch.zeros_like(h)
    if mlp["kind"] == "dense":
        return glu(h, P, pre, gelu_tanh)
    return routed_experts(h, P, pre, mlp)


# ---- the model ----------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """Execution order: (layer index, opens a pass) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg, P, tokens, residuals=None):
    """Logits [T, vocab] of one whole sequence; ``residuals`` (optional list) receives x after every layer run."""
    P = {k: v.to(F64) for k, v in P.items()}
    eps = cfg["norm"]["eps"]
    x0 = P["embed"][torch.tensor(tokens)]
    x = x0
    for i, opens in layer_runs(cfg):
        L = cfg["layers"][i]
        if opens:
            x = torch.cat([x, x0], -1) @ P["loop.in"].T
        h = norm_one_plus(x, P[f"l{i}.norm1"], eps)
        mix = channel_delta if L["type"] == "channel_delta" else side_by_side
        x = x + (mix(h, P, f"l{i}.mix.", L["mixer"], eps) + feed_forward(h, P, f"l{i}.mlp.", L.get("mlp")))
        if residuals is not None:
            residuals.append(x)
    return norm_one_plus(x, P["final.norm"], eps) @ P["head"].T


# ---- configurations and random weights for the tests ----------------------------------------------------------------------
def delta_layer(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def pair_layer(heads, kv_heads, dim, vdim, scale, rheads, rdim, rvdim, decay, q_temp=None, left_scale=1.0, right_scale=1.0, mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp:
        left["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    right = {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": list(decay)}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}, "mlp": mlp}


def dense_mlp(ff):
    return {"kind": "dense", "ff": ff}


def moe_mlp(experts, top, ff, shared_ff=None):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def make_config(layers, vocab=97, width=48, eps=3e-6, loop=None):
    cfg = {"architecture": "Pupopel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def low_rank(width):
    """Inner size of the two-step decay and gate projections (the tensors' shapes carry it; this is the tests' choice)."""
    return max(4, width // 8)


def random_weights(cfg, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(n_out, n_in, gain=1.0):
        return (torch.randn(n_out, n_in, generator=g) * gain / math.sqrt(n_in)).to(dtype)

    def vec(n, scale=0.1, shift=0.0):
        return (torch.randn(n, generator=g) * scale + shift).to(dtype)

    def glu_w(pre, ff):
        P[pre + "gate"], P[pre + "up"], P[pre + "down"] = mat(ff, W), mat(ff, W), mat(W, ff)

    P = {"embed": mat(V, W, math.sqrt(W)), "head": mat(V, W), "final.norm": vec(W)}
    if cfg.get("loop"):
        P["loop.in"] = mat(W, 2 * W, 1.4)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        P[f"l{i}.norm1"] = vec(W)
        if L["type"] == "channel_delta":
            H, G, dk, dv, n, r = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], low_rank(W)
            P[p + "q"], P[p + "k"], P[p + "v"] = mat(G * dk, W, 2.0), mat(G * dk, W, 2.0), mat(H * dv, W, 2.0)
            for c, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                P[p + c + ".conv"] = (torch.randn(rows, n, generator=g) / math.sqrt(n)).to(dtype)
            P[p + "b"] = mat(H, W)
            P[p + "a1"], P[p + "a2"] = mat(r, W), mat(H * dk, r, 2.0)
            P[p + "A_log"], P[p + "dt_bias"] = vec(H, 0.5, -1.0), vec(H * dk, 0.5, -1.0)
            P[p + "g1"], P[p + "g2"] = mat(r, W), mat(H * dv, r, 2.0)
            P[p + "norm"] = vec(dv, 0.1, 1.0)
            P[p + "o"] = mat(W, H * dv)
        else:
            a, b = m["left"], m["right"]
            P[p + "left.q"], P[p + "left.k"] = mat(a["heads"] * a["dim"], W), mat(a["kv_heads"] * a["dim"], W)
            P[p + "left.v"] = mat(a["kv_heads"] * a["vdim"], W)
            P[p + "left.q.norm"], P[p + "left.k.norm"] = vec(a["dim"], 0.1, 1.0), vec(a["dim"], 0.1, 1.0)
            P[p + "left.sink"] = vec(a["heads"], 1.0)
            P[p + "left.o"] = mat(W, a["heads"] * a["vdim"])
            P[p + "right.q"], P[p + "right.k"] = mat(b["heads"] * b["dim"], W), mat(b["heads"] * b["dim"], W)
            P[p + "right.v"], P[p + "right.g"] = mat(b["heads"] * b["vdim"], W), mat(b["heads"] * b["vdim"], W)
            P[p + "right.norm"] = vec(b["heads"] * b["vdim"], 0.1, 1.0)
            P[p + "right.o"] = mat(W, b["heads"] * b["vdim"])
        mlp = L.get("mlp")
        if mlp is None:
            continue
        q = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            glu_w(q, mlp["ff"])
        else:
            for e in range(mlp["router"]["experts"]):
                glu_w(f"{q}e{e}.", mlp["expert"]["ff"])
            P[q + "router"], P[q + "router.b"] = mat(mlp["router"]["experts"], W, 3.0), vec(mlp["router"]["experts"], 0.3)
            if mlp.get("shared"):
                glu_w(q + "shared.", mlp["shared"]["ff"])
    return P


def logits_error(got, want):
    """Worst position: rms over the vocabulary of the centred difference, relative to the rms of the centred expected row."""
    got, want = got.to(F64).cpu(), want.to(F64).cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())
