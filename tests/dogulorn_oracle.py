"""Slow float64 statement of the Dogulorn design, one function per mechanism, whole sequences on the CPU.

Written from the design's equations; shares no code with mlx_parallm_b200 (it does not import it).  Notation: T tokens,
W width, x the residual stream [T, W], weights ``P[name]`` stored [out, in] and applied as x @ P.T.
"""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def silu(z):
    return z * torch.sigmoid(z)


def hashed_embedding(tokens, embed, bigram, scale, buckets, mul_prev, mul_cur):
    """token row * scale, plus (if there is a bigram table) the row picked by the token pair; the first token of the
    sequence takes the extra last row."""
    x = embed[torch.tensor(tokens)] * scale
    if bigram is not None:
        idx = [buckets] + [(tokens[t - 1] * mul_prev + tokens[t] * mul_cur) % buckets for t in range(1, len(tokens))]
        x = x + bigram[torch.tensor(idx)]
    return x


def short_conv_silu(u, taps_w):
    """Per channel c: silu(sum_j taps_w[c, j] * u[t - (n - 1 - j), c]) with zeros before the start; u [T, C], taps_w [C, n]."""
    T, C = u.shape
    n = taps_w.shape[1]
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(n):
            s = t - (n - 1 - j)
            if s >= 0:
                out[t] += taps_w[:, j] * u[s]
    return silu(out)


def gated_delta(h, P, pre, m, eps):
    """The delta-rule mixer on normed input h [T, W]; P[pre + name] its tensors; m its sizes."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = short_conv_silu(h @ P[pre + "q"].T, P[pre + "q.conv"]).view(T, G, dk)
    k = short_conv_silu(h @ P[pre + "k"].T, P[pre + "k.conv"]).view(T, G, dk)
    v = short_conv_silu(h @ P[pre + "v"].T, P[pre + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) / math.sqrt(dk)
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ P[pre + "b"].T)                                                    # [T, H]
    decay = torch.exp(-torch.exp(P[pre + "A_log"]) * torch.nn.functional.softplus(h @ P[pre + "a"].T + P[pre + "dt_bias"]))
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        g = head // (H // G)
        S = torch.zeros(dk, dv, dtype=F64)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, head] = S.T @ q[t, g]
    gate = silu(h @ P[pre + "g"].T).view(T, H, dv)
    out = rms_unit(out, eps) * P[pre + "norm"] * gate
    return out.reshape(T, H * dv) @ P[pre + "o"].T


def latent_attention(h, P, pre, m, eps, latents, index):
    """Latent attention on normed input h; ``latents`` collects each layer's key/value latent for layers that share it."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ P[pre + "dq"].T, P[pre + "dq.norm"], eps)
    q = (cq @ P[pre + "uq"].T).view(T, H, dk)
    if m.get("kv_from") is not None:
        c = latents[m["kv_from"]]
    else:
        c = rms_norm(h @ P[pre + "dkv"].T, P[pre + "dkv.norm"], eps)
        latents[index] = c
    k = (c @ P[pre + "uk"].T).view(T, H, dk)
    v = (c @ P[pre + "uv"].T).view(T, H, dv)
    scale = m.get("scale", dk ** -0.5)
    window = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        first = 0 if not window else max(0, i - window + 1)
        for head in range(H):
            s = (k[first:i + 1, head] @ q[i, head]) * scale
            p = torch.softmax(s, 0)
            out[i, head] = p @ v[first:i + 1, head]
    return out.reshape(T, H * dv) @ P[pre + "o"].T


def clamped_glu(h, P, pre, limit):
    g = torch.clamp(h @ P[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ P[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ P[pre + "down"].T


def token_side(x, tokens, P, layer, dim, eps):
    """The per-layer token input, already normed: what is added to x."""
    e = P["side.embed"][torch.tensor(tokens)][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ P[f"l{layer}.side.gate"].T) * e) @ P[f"l{layer}.side.proj"].T
    return rms_norm(y, P[f"l{layer}.side.norm"], eps)


def forward(cfg, weights, tokens, residuals=None):
    """logits [T, vocab] (float64) of one sequence from its first token."""
    P = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    emb = cfg.get("embedding") or {}
    big = emb.get("bigram")
    x = hashed_embedding(tokens, P["embed"], P["bigram"] if big else None, emb.get("scale", 1.0),
                         big["buckets"] if big else 0, big["mul_prev"] if big else 0, big["mul_cur"] if big else 0)
    latents = {}
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = rms_norm(x, P[pre + "norm1"], eps)
        if L["type"] == "delta":
            y = gated_delta(h, P, pre + "mix.", L["mixer"], eps)
        else:
            y = latent_attention(h, P, pre + "mix.", L["mixer"], eps, latents, i)
        x = x + rms_norm(y, P[pre + "norm1b"], eps)
        if L.get("mlp") is not None:
            y = clamped_glu(rms_norm(x, P[pre + "norm2"], eps), P, pre + "mlp.", L["mlp"]["limit"])
            x = x + rms_norm(y, P[pre + "norm2b"], eps)
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, P, i, cfg["token_side"]["dim"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return rms_norm(x, P["final.norm"], eps) @ P["head"].T


# ---- small random models ---------------------------------------------------------------------------------------------
def delta_layer(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def attn_layer(heads, dim, vdim, q_rank, kv_rank, window, scale=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank}
    if window:
        m["mask"] = {"size": window}
    if scale is not None:
        m["scale"] = scale
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def make_config(layers, vocab=97, width=48, eps=1e-5, emb_scale=0.7, bigram=(53, 5, 11), side_dim=8):
    cfg = {"architecture": "Dogulorn", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
           "embedding": {"scale": emb_scale}}
    if bigram:
        cfg["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if side_dim:
        cfg["token_side"] = {"dim": side_dim}
    return cfg


def random_weights(cfg, seed=0):
    """Weights of a config as bfloat16 tensors (vectors too, like a checkpoint on disk)."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    out = {}

    def lin(name, n_out, n_in, gain=1.0):
        out[name] = (torch.randn(n_out, n_in, generator=g) * gain / math.sqrt(n_in)).to(torch.bfloat16)

    def vec(name, n, mean=1.0, spread=0.2):
        out[name] = (mean + spread * torch.randn(n, generator=g)).to(torch.bfloat16)

    out["embed"] = torch.randn(V, W, generator=g).to(torch.bfloat16)
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        out["bigram"] = (0.5 * torch.randn(big["buckets"] + 1, W, generator=g)).to(torch.bfloat16)
    side = cfg.get("token_side")
    if side:
        out["side.embed"] = torch.randn(V, len(cfg["layers"]) * side["dim"], generator=g).to(torch.bfloat16)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", W)
        vec(p + "norm1b", W)
        if L["type"] == "delta":
            H, G, dk, dv, n = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m["conv"]
            for nm, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                lin(p + "mix." + nm, rows, W, 2.0)
                out[p + f"mix.{nm}.conv"] = (0.6 * torch.randn(rows, n, generator=g)).to(torch.bfloat16)
            lin(p + "mix.b", H, W, 2.0)
            lin(p + "mix.a", H, W, 2.0)
            lin(p + "mix.g", H * dv, W, 2.0)
            lin(p + "mix.o", W, H * dv)
            vec(p + "mix.A_log", H, -0.5, 0.8)
            vec(p + "mix.dt_bias", H, 0.0, 1.0)
            vec(p + "mix.norm", dv)
        else:
            H, dk, dv, rq, rk = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            lin(p + "mix.dq", rq, W)
            vec(p + "mix.dq.norm", rq)
            lin(p + "mix.uq", H * dk, rq, 2.0)
            if m.get("kv_from") is None:
                lin(p + "mix.dkv", rk, W)
                vec(p + "mix.dkv.norm", rk)
            lin(p + "mix.uk", H * dk, rk, 2.0)
            lin(p + "mix.uv", H * dv, rk)
            lin(p + "mix.o", W, H * dv)
        if L.get("mlp") is not None:
            ff = L["mlp"]["ff"]
            vec(p + "norm2", W)
            vec(p + "norm2b", W)
            lin(p + "mlp.gate", ff, W, 2.0)
            lin(p + "mlp.up", ff, W, 2.0)
            lin(p + "mlp.down", W, ff)
        if side:
            lin(p + "side.gate", side["dim"], W, 2.0)
            lin(p + "side.proj", W, side["dim"])
            vec(p + "side.norm", W)
    vec("final.norm", W)
    lin("head", V, W)
    return out


def logits_error(got, want):
    """Worst position: rms over the vocabulary of the centred difference, relative to the rms of the centred expected row."""
    got, want = got.to(F64).cpu(), want.to(F64).cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())
