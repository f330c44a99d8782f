"""Pupopel on the GPU against the slow float64 oracle (tests/pupopel_oracle.py): each mechanism alone, prompts against
token-by-token decoding, portions, ragged batches, rows given back and used again, far keys and chunk borders, the sink, the
query temperature's blocks, the looped span, other sizes, greedy generation through generate_step."""
import math

import numpy as np
import pytest
import torch

import pupopel_oracle as O

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4        # float32 model against the float64 oracle (centred rms over the vocabulary, relative)
BF16_TOL = 6e-2       # bfloat16 matrix products


def build(cfg, seed=0, dtype=torch.float32, weights=None):
    from mlx_parallm_b200.utils import _get_classes
    Model, Args = _get_classes(cfg)
    w = O.random_weights(cfg, seed) if weights is None else weights
    return Model(Args.from_dict(cfg)).load_weights(w, device="cuda", dtype=dtype), w


def toks(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


CONFIGS = {
    # every branch: both mixers, dense / routed / no feed-forward, experts with and without a shared one, a span of two layers
    # run three times from the first layer on
    "mixed": lambda: O.make_config([
        O.delta_layer(4, 2, 16, 8, conv=4, mlp=O.dense_mlp(40)),
        O.pair_layer(6, 2, 16, 24, 0.3, 2, 8, 16, [0.7, 0.97], q_temp=(0.4, 5), left_scale=1.3, right_scale=0.6,
                     mlp=O.moe_mlp(6, 2, 24, shared_ff=16)),
        O.delta_layer(3, 3, 8, 24, conv=2, mlp=O.moe_mlp(4, 3, 16)),
        O.pair_layer(2, 1, 8, 8, 0.5, 3, 16, 8, [0.5, 0.9, 0.999]),
    ], loop=(0, 2, 3)),
    # sizes off the fast paths (odd width, heads and ranks), one key head for three heads, a span that starts after the first
    # layer, all experts chosen, no query temperature
    "odd": lambda: O.make_config([
        O.delta_layer(3, 1, 5, 7, conv=3),
        O.pair_layer(6, 2, 10, 9, 0.25, 3, 6, 11, [0.8, 0.9, 0.95], mlp=O.moe_mlp(5, 5, 13, shared_ff=9)),
        O.delta_layer(1, 1, 12, 6, conv=5, mlp=O.dense_mlp(13)),
    ], vocab=31, width=27, eps=1e-3, loop=(1, 2, 2)),
    # wider heads: key size 40 pads to 64 state rows, value size 160 spans two thread blocks; as many key heads as heads, one
    # expert per token, no convolution, a span that runs once (its opening map still applies), temperature blocks of 3 tokens
    "wide": lambda: O.make_config([
        O.delta_layer(2, 1, 40, 160, conv=1, mlp=O.moe_mlp(3, 1, 24, shared_ff=8)),
        O.pair_layer(4, 4, 72, 40, 0.12, 1, 40, 96, [0.93], q_temp=(0.25, 3), mlp=O.dense_mlp(40)),
    ], vocab=130, width=64, loop=(0, 2, 1)),
    # no span at all
    "plain": lambda: O.make_config([
        O.pair_layer(4, 2, 8, 8, 0.35, 2, 8, 8, [0.6, 0.99], q_temp=(0.45, 16), mlp=O.dense_mlp(24)),
        O.delta_layer(2, 2, 8, 8, conv=4, mlp=O.dense_mlp(24)),
    ], vocab=50, width=32),
}


@pytest.fixture(scope="module")
def models():
    out = {}
    for name, mk in CONFIGS.items():
        cfg = mk()
        m, w = build(cfg, seed=len(name))
        out[name] = (cfg, m, w)
    return out


def run_order(cfg):
    return [i for i, _ in O.layer_runs(cfg)]


# ---- mechanisms alone ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("M", [2, 40, 300])
def test_gemm_gated_epilogues(dtype, act, M):
    from mlx_parallm_b200 import ops
    from mlx_parallm_b200.models._sequence import GatedFF
    g = torch.Generator().manual_seed(M)
    ff, K = 72, 64
    x = torch.randn(M, K, generator=g).to(dtype)
    gate, up = torch.randn(ff, K, generator=g).to(dtype), torch.randn(ff, K, generator=g).to(dtype)
    f = O.gelu_tanh if act == "gelu_tanh" else O.silu
    want = f(x.double() @ gate.double().T) * (x.double() @ up.double().T)
    got = ops.gemm(x.cuda(), GatedFF.interleave(gate, up).cuda(), GatedFF.EPILOGUES[act])
    assert got.shape == (M, ff) and got.dtype == dtype
    tol = 1e-4 if dtype == torch.float32 else 0.03
    assert ((got.double().cpu() - want).abs() / (1.0 + want.abs())).max() < tol * math.sqrt(K)


@pytest.mark.parametrize("E,top,M", [(5, 2, 7), (11, 4, 40), (70, 8, 33), (3, 3, 1), (4, 1, 300)])
def test_routing_and_grouped_products(E, top, M):
    """The chosen experts and their weights against topk + softmax; every (token, choice) has a slot inside its expert's
    segment; the grouped product of the sorted rows equals each expert's own product."""
    from mlx_parallm_b200 import _lib, ops
    g = torch.Generator().manual_seed(E * 100 + M)
    logits, bias = torch.randn(M, E, generator=g), torch.randn(E, generator=g) * 0.3
    i32 = dict(dtype=torch.int32, device="cuda")
    ids, slot_of, token_of = torch.zeros(M, top, **i32), torch.zeros(M, top, **i32), torch.zeros(M * top, **i32)
    wts, seg = torch.zeros(M, top, device="cuda"), torch.zeros(E + 1, **i32)
    ops.moe_route(logits.cuda(), bias.cuda(), ids, wts, seg, slot_of, token_of, top)
    z = (logits + bias).double()
    tv, ti = torch.topk(z, top, -1)
    assert torch.equal(ids.cpu().long(), ti)                       # largest first, like topk
    assert (wts.cpu().double() - torch.softmax(tv, -1)).abs().max() < 1e-6
    seg_h, slot_h, tok_h = seg.cpu().tolist(), slot_of.cpu().view(-1).tolist(), token_of.cpu().tolist()
    assert seg_h[0] == 0 and seg_h[-1] == M * top and sorted(slot_h) == list(range(M * top))
    for i, s in enumerate(slot_h):
        e = int(ids.view(-1)[i])
        assert seg_h[e] <= s < seg_h[e + 1] and tok_h[s] == i // top
    for dtype in (torch.float32, torch.bfloat16):
        K, N = 24, 40
        x = torch.randn(M, K, generator=g).to(dtype)
        w = torch.randn(E, N, K, generator=g).to(dtype)
        xs = torch.empty(M * top, K, dtype=dtype, device="cuda")
        ops.moe_gather(x.cuda(), token_of, xs)
        y = ops.gemm_grouped(xs, w.cuda(), seg, M, _lib.GEMM_STORE_F32)
        for s in range(M * top):
            e = next(k for k in range(E) if seg_h[k] <= s < seg_h[k + 1])
            want = x[tok_h[s]].double() @ w[e].double().T
            assert (y[s].double().cpu() - want).abs().max() < 1e-3
        ye = torch.randn(M * top, 16, generator=g).cuda()
        sh = torch.randn(M, 16, generator=g).cuda()
        out = torch.empty(M, 16, device="cuda")
        ops.moe_combine(ye, slot_of, wts, sh, out, top)
        want = sh.cpu().double() + (wts.cpu().double().unsqueeze(-1) * ye.cpu().double()[slot_of.cpu().long()]).sum(1)
        assert (out.cpu().double() - want).abs().max() < 1e-5


@pytest.mark.parametrize("sizes,N,K", [([130, 0, 77, 300, 1], 264, 128), ([64, 65, 128, 129], 512, 64), ([0, 0, 700], 72, 200), ([90] * 20, 256, 256)])
def test_grouped_products_of_many_rows(sizes, N, K):
    """Groups of more than 64 rows (prompts) in 16 bits: groups of 0, 1 and a multiple of the tile's rows, a group that ends
    where the tensor ends, plain and gated stores."""
    from mlx_parallm_b200 import _lib, ops
    from mlx_parallm_b200.models._sequence import GatedFF
    g = torch.Generator().manual_seed(N + K)
    E, total = len(sizes), sum(sizes)
    seg = torch.tensor([0] + list(np.cumsum(sizes)), dtype=torch.int32, device="cuda")
    x = torch.randn(total, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(E, N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    y = ops.gemm_grouped(x.cuda(), w.cuda(), seg, max(sizes), _lib.GEMM_STORE_F32).cpu().double()
    gate, up = w[:, :N // 2], w[:, N // 2:]
    wi = torch.stack([GatedFF.interleave(gate[e], up[e]) for e in range(E)]).contiguous()
    act = ops.gemm_grouped(x.cuda(), wi.cuda(), seg, max(sizes), _lib.GEMM_GLU_SILU).cpu().double()
    lo = 0
    for e, n in enumerate(sizes):
        xe = x[lo:lo + n].double()
        want = xe @ w[e].double().T
        assert (y[lo:lo + n] - want).abs().max() < 1e-3 if n else True
        wa = O.silu(xe @ gate[e].double().T) * (xe @ up[e].double().T)
        assert ((act[lo:lo + n] - wa).abs() / (1.0 + wa.abs())).max() < 2e-2 if n else True
        lo += n
    assert _lib.lib().b200p_gemm_tc_fault() == 0


def test_residual_add_norm_parts():
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(1)
    M, W = 9, 50
    h0, y1, y2, w = (torch.randn(M, W, generator=g) for _ in range(4))
    h = h0.clone().cuda()
    x = torch.empty(M, W, device="cuda")
    cat = torch.zeros(M, 2 * W, device="cuda")
    ops.residual_add_norm(h, 1e-3, torch.float32, y1=y1.cuda(), c1=1.0, y2=y2.cuda(), c2=-0.5, w_next=w[0].contiguous().cuda(), x_out=x,
                          raw_out=cat[:, W:])
    want = h0.double() + y1.double() - 0.5 * y2.double()
    assert (h.cpu().double() - want).abs().max() < 1e-5
    assert (cat[:, W:].cpu().double() - want).abs().max() < 1e-5 and float(cat[:, :W].abs().max()) == 0.0
    assert (x.cpu().double() - O.rms_unit(want, 1e-3) * w[0].double()).abs().max() < 1e-5
    h2 = h0.clone().cuda()
    ops.residual_add_norm(h2, 1e-3, torch.float32)                 # nothing to add, nothing to write: h unchanged
    assert torch.equal(h2.cpu(), h0)


def one_layer(layer, **kw):
    return O.make_config([layer], **kw)


def mixer_alone(cfg, w, T, seed, dtype=torch.float32):
    """Residual stream after the single layer of cfg for T random tokens: framework, oracle."""
    m, _ = build(cfg, dtype=dtype, weights=w)
    t = toks(cfg, T, seed)
    res, got = [], []
    O.forward(cfg, w, t, res)
    m.residual_tap = lambda layer, kind, h: got.append(h.clone())
    m.forward_ragged([t], m.make_cache(1))
    m.residual_tap = None
    return got[0].double().cpu(), res[0]


@pytest.mark.parametrize("H,G,dk,dv,conv", [(4, 4, 16, 16, 4), (3, 1, 5, 7, 3), (2, 1, 40, 160, 1), (2, 2, 130, 24, 2), (1, 1, 300, 70, 6)])
def test_channel_delta_alone(H, G, dk, dv, conv):
    cfg = one_layer(O.delta_layer(H, G, dk, dv, conv), vocab=40, width=24)
    w = O.random_weights(cfg, H * dk)
    got, want = mixer_alone(cfg, w, 37, 2)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_channel_decays_differ_per_channel():
    """One key channel forgets at once (decay near zero) while the others keep everything: a head-wide decay, or a decay
    applied along the value columns instead of the key rows, gives another answer."""
    cfg = one_layer(O.delta_layer(2, 2, 8, 8, 2), vocab=40, width=16)
    w = O.random_weights(cfg, 5)
    bias = torch.full((16,), -12.0)
    bias[3], bias[12] = 9.0, 9.0
    w["l0.mix.dt_bias"] = bias
    w["l0.mix.a2"] = w["l0.mix.a2"] * 0.01
    got, want = mixer_alone(cfg, w, 30, 3)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))
    w2 = dict(w)
    w2["l0.mix.dt_bias"] = torch.full((16,), -12.0)
    _, other = mixer_alone(cfg, w2, 30, 3)
    assert (other - want).abs().max() > 1e-2


@pytest.mark.parametrize("H,G,dk,dv,rh,rdk,rdv", [(8, 2, 16, 16, 4, 16, 16), (6, 2, 10, 9, 3, 6, 11), (4, 4, 72, 40, 1, 40, 96), (2, 1, 128, 64, 2, 64, 128)])
def test_side_by_side_alone(H, G, dk, dv, rh, rdk, rdv):
    decay = [0.5 + 0.49 * (i + 1) / rh for i in range(rh)]
    cfg = one_layer(O.pair_layer(H, G, dk, dv, dk ** -0.5, rh, rdk, rdv, decay, q_temp=(0.5, 4), left_scale=0.7, right_scale=1.4), vocab=40, width=32)
    w = O.random_weights(cfg, H + dk)
    got, want = mixer_alone(cfg, w, 41, 4)
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def attn_kernel_case(T, H, G, dk, dv, hot_query=None, hot_key=None, sink=None, slope_log2=-8.0, dtype=torch.float32, seed=0, boost=30.0):
    """sink_attn over T cached positions of one row; every token is a query at its own position.  A hot pair (query position,
    key position) gets a score far above the rest so that a key that is wrongly masked, skipped or misplaced shows."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(seed + T)
    q = torch.randn(T, H, dk, generator=g) * 0.3
    k = torch.randn(T, G, dk, generator=g) * 0.3
    v = torch.randn(T, G, dv, generator=g)
    if hot_query is not None:
        u = torch.randn(dk, generator=g)
        u = u / u.norm()
        q[hot_query] += boost * u
        k[hot_key] += u.view(1, dk)
    if dtype != torch.float32:
        q = q.to(dtype).float()            # the 16-bit kernels round the query to the cache's type: give both sides that query
    sk = torch.zeros(H) if sink is None else sink
    kc = torch.zeros(2, G, T + 3, dk)
    vc = torch.zeros(2, G, T + 3, dv)
    kc[1, :, :T] = k.transpose(0, 1)
    vc[1, :, :T] = v.transpose(0, 1)
    kc, vc = kc.to(dtype), vc.to(dtype)
    out = torch.zeros(T, H * dv + 8, dtype=dtype, device="cuda")
    i32 = dict(dtype=torch.int32, device="cuda")
    cu, rows = torch.tensor([0, T], **i32), torch.tensor([1], **i32)
    ops.sink_attn(q.reshape(T, -1).contiguous().cuda(), kc.cuda(), vc.cuda(), torch.ones(T, **i32), torch.arange(T, **i32), sk.cuda(),
                  slope_log2, out[:, :H * dv], H, G, dk, dv, out_scale=1.5, cu=cu, rows=rows, nb=1, max_n=T)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    kd, vd = kc[1, :, :T].double(), vc[1, :, :T].double()
    i, j = torch.arange(T).view(T, 1), torch.arange(T).view(1, T)
    for h in range(H):
        kv = h // (H // G)
        slope = 2.0 ** (slope_log2 * (h + 1) / H) if slope_log2 else 0.0
        s = q[:, h].double() @ kd[kv].T - slope * (i - j).double()
        s = s.masked_fill(j > i, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, sk[h].double())
        e = torch.exp(s - top)
        want[:, h] = 1.5 * (e @ vd[kv]) / (e.sum(-1, keepdim=True) + torch.exp(sk[h].double() - top))
    assert float(out[:, H * dv:].float().abs().max()) == 0.0          # columns beside the heads are not touched
    return out[:, :H * dv].double().cpu().view(T, H, dv), want


@pytest.mark.parametrize("T,hot_query,hot_key", [(600, 599, 3), (600, 580, 0), (70, 63, 31), (70, 64, 32), (70, 65, 33), (130, 128, 63),
                                                 (130, 129, 64), (97, 96, 96), (33, 32, 0), (1, None, None), (2, 1, 0)])
def test_sink_attention_far_keys_and_chunk_borders(T, hot_query, hot_key):
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        got, want = attn_kernel_case(T, 4, 2, 16, 24, hot_query, hot_key, dtype=dtype, slope_log2=-8.0 if T < 200 else -20.0)
        assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))
        if hot_query is not None:
            assert float(want[hot_query].abs().max()) > 0.05        # the hot key is what the query reads


def test_sink_attention_sink_and_bias():
    """A large sink takes the probability mass (outputs shrink towards zero), a very negative one changes nothing; without
    the bias the far keys count as much as the near ones."""
    T = 50
    big, want_big = attn_kernel_case(T, 4, 4, 8, 8, sink=torch.tensor([6.0, -30.0, 0.0, 2.0]))
    assert (big - want_big).abs().max() < 1e-4
    assert float(big[:, 0].abs().max()) < 0.2 * float(big[:, 1].abs().max())
    nob, want_nob = attn_kernel_case(T, 4, 4, 8, 8, slope_log2=0.0)
    assert (nob - want_nob).abs().max() < 1e-4
    withb, _ = attn_kernel_case(T, 4, 4, 8, 8)
    assert (nob - withb).abs().max() > 1e-2


@pytest.mark.parametrize("T,hot_query,hot_key", [(600, 599, 3), (70, 63, 31), (70, 64, 32), (130, 128, 63), (130, 129, 64), (129, 128, 128),
                                                 (65, 64, 0), (64, 63, 0), (5, 4, 1)])
def test_sink_attention_tile_kernel_far_keys_and_tile_borders(T, hot_query, hot_key):
    """Sizes the tensor-core kernel takes (16-bit, key / value sizes 64 and 128): hot pairs across its 64-key tiles and its
    64-query tiles."""
    for dk, dv in ((64, 64), (128, 64), (64, 128), (128, 128)):
        got, want = attn_kernel_case(T, 4, 2, dk, dv, hot_query, hot_key, dtype=torch.bfloat16, sink=torch.tensor([0.5, -1.0, 2.0, 0.0]),
                                     slope_log2=-8.0 if T < 200 else -20.0, seed=dk + dv)
        assert (got - want).abs().max() < 3e-2 * max(1.0, float(want.abs().max()))
        assert float(want[hot_query].abs().max()) > 0.05


def test_sink_attention_tiles_over_ragged_portions():
    """Three entries in one launch: a fresh prompt, a short and a long continuation of rows that already hold keys (their
    first positions are not multiples of the tile sizes), in rows out of order."""
    from mlx_parallm_b200 import ops
    H, G, dk, dv = 6, 3, 64, 128
    g = torch.Generator().manual_seed(5)
    entries = [(2, 0, 70), (0, 37, 5), (1, 100, 130)]                    # (cache row, first position, tokens)
    Tcap = 256
    kc = (torch.randn(3, G, Tcap, dk, generator=g) * 0.3).to(torch.bfloat16)
    vc = torch.randn(3, G, Tcap, dv, generator=g).to(torch.bfloat16)
    M = sum(n for _, _, n in entries)
    q = (torch.randn(M, H, dk, generator=g) * 0.3).to(torch.bfloat16).float()
    sink = torch.linspace(-1, 1, H)
    i32 = dict(dtype=torch.int32, device="cuda")
    cu, t_row, t_pos = [0], [], []
    for r, p0, n in entries:
        cu.append(cu[-1] + n)
        t_row += [r] * n
        t_pos += list(range(p0, p0 + n))
    out = torch.zeros(M, H * dv, dtype=torch.bfloat16, device="cuda")
    ops.sink_attn(q.reshape(M, -1).contiguous().cuda(), kc.cuda(), vc.cuda(), torch.tensor(t_row, **i32), torch.tensor(t_pos, **i32),
                  sink.cuda(), -8.0, out, H, G, dk, dv, cu=torch.tensor(cu, **i32), rows=torch.tensor([e[0] for e in entries], **i32),
                  nb=3, max_n=130)
    got = out.double().cpu().view(M, H, dv)
    for t in range(M):
        r, p = t_row[t], t_pos[t]
        for h in range(H):
            kv = h // (H // G)
            slope = 2.0 ** (-8.0 * (h + 1) / H)
            s = kc[r, kv, :p + 1].double() @ q[t, h].double() - slope * (p - torch.arange(p + 1)).double()
            top = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - top)
            want = (e @ vc[r, kv, :p + 1].double()) / (e.sum() + math.exp(float(sink[h]) - top))
            assert (got[t, h] - want).abs().max() < 3e-2 * max(1.0, float(want.abs().max())), (t, h)


@pytest.mark.parametrize("H,G,dk,dv,nb", [(8, 2, 64, 64, 5), (16, 1, 128, 128, 3), (4, 4, 64, 128, 40), (6, 3, 128, 64, 300), (32, 2, 64, 64, 2)])
def test_sink_attention_decode_steps_on_tiles(H, G, dk, dv, nb):
    """One token per entry at positions from 0 to several hundred (first token, tile borders, many tiles), rows out of order:
    the keys of an entry are split over several CTAs whose partial sums and the sink are merged afterwards."""
    from mlx_parallm_b200 import ops
    g = torch.Generator().manual_seed(H + nb)
    Tcap = 700
    special = [0, 1, 63, 64, 65, 127, 128, 129, 699, 640, 300]
    pos = [special[i] if i < len(special) else int(torch.randint(0, Tcap, (1,), generator=g)) for i in range(nb)]
    rows = torch.randperm(nb, generator=g).tolist()
    R = min(nb, 12)                                                        # check these entries against the slow sum
    kc = (torch.randn(nb, G, Tcap, dk, generator=g) * 0.3).to(torch.bfloat16)
    vc = torch.randn(nb, G, Tcap, dv, generator=g).to(torch.bfloat16)
    q = (torch.randn(nb, H, dk, generator=g) * 0.4).to(torch.bfloat16).float()
    sink = torch.linspace(-2, 2, H)
    i32 = dict(dtype=torch.int32, device="cuda")
    out = torch.zeros(nb, H * dv, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(ops.sink_attn_workspace_floats(min(nb, 64), H, dv), device="cuda")
    ops.sink_attn(q.reshape(nb, -1).contiguous().cuda(), kc.cuda(), vc.cuda(), torch.tensor(rows, **i32), torch.tensor(pos, **i32),
                  sink.cuda(), -8.0, out, H, G, dk, dv, out_scale=0.8, cu=torch.arange(nb + 1, **i32), rows=torch.tensor(rows, **i32),
                  nb=nb, max_n=1, workspace=ws)
    got = out.double().cpu().view(nb, H, dv)
    for e in range(R):
        r, p = rows[e], pos[e]
        for h in range(H):
            kv = h // (H // G)
            slope = 2.0 ** (-8.0 * (h + 1) / H)
            sc = kc[r, kv, :p + 1].double() @ q[e, h].double() - slope * (p - torch.arange(p + 1)).double()
            top = max(float(sc.max()), float(sink[h]))
            ex = torch.exp(sc - top)
            want = 0.8 * (ex @ vc[r, kv, :p + 1].double()) / (ex.sum() + math.exp(float(sink[h]) - top))
            assert (got[e, h] - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max())), (e, h, p)


@pytest.mark.parametrize("H,G,dk,dv", [(16, 2, 64, 64), (8, 8, 128, 128), (12, 4, 32, 48), (5, 5, 24, 200), (8, 1, 256, 64), (4, 2, 64, 128)])
def test_sink_attention_head_geometries(H, G, dk, dv):
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        got, want = attn_kernel_case(150, H, G, dk, dv, 149, 20, sink=torch.linspace(-1, 1, H), dtype=dtype, seed=H)
        assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max()))


# ---- whole models -------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prompt_logits_and_residuals_match_the_oracle(models, name):
    cfg, m, w = models[name]
    t = toks(cfg, 45, 1)
    res = []
    want = O.forward(cfg, w, t, res)
    got_res = []
    m.residual_tap = lambda layer, kind, h: got_res.append((layer, h.clone()))
    try:
        got = m.forward_ragged([t], m.make_cache(1), want=[list(range(len(t)))])
    finally:
        m.residual_tap = None
    assert [i for i, _ in got_res] == run_order(cfg)
    for k, r in enumerate(res):
        assert (got_res[k][1].double().cpu() - r).abs().max() < 2e-4 * max(1.0, float(r.abs().max())), f"residual after run {k}"
    assert O.logits_error(got, want) < F32_TOL


@pytest.mark.parametrize("name", list(CONFIGS))
def test_bfloat16_model(name):
    cfg = CONFIGS[name]()
    m, w = build(cfg, seed=3, dtype=torch.bfloat16)
    t = toks(cfg, 60, 2)
    got = m.forward_ragged([t], m.make_cache(1), want=[list(range(len(t)))])
    want = O.forward(cfg, w, t)
    per_pos = sorted(O.logits_error(got[i:i + 1], want[i:i + 1]) for i in range(len(t)))
    assert per_pos[len(t) // 2] < BF16_TOL and per_pos[-1] < 1.0, per_pos[-3:]


def test_bfloat16_model_on_the_tensor_core_paths():
    """Head sizes the tile attention kernels take (64 / 128), groups of experts large enough for the tcgen05 grouped product:
    a prompt, a ragged batch and decode steps through the captured step (whose attention splits the keys over CTAs) in
    bfloat16 against the oracle; positions compared by their typical error, as above."""
    from mlx_parallm_b200 import utils
    cfg = O.make_config([
        O.pair_layer(4, 2, 64, 128, 0.125, 2, 64, 64, [0.9, 0.99], q_temp=(0.2, 32), mlp=O.moe_mlp(4, 2, 64, shared_ff=64)),
        O.delta_layer(2, 2, 64, 64, conv=4, mlp=O.dense_mlp(128)),
        O.pair_layer(8, 8, 128, 64, 0.09, 1, 32, 32, [0.95]),
    ], vocab=200, width=128, loop=(0, 2, 2))
    m, w = build(cfg, seed=7, dtype=torch.bfloat16)
    t = toks(cfg, 330, 3)
    want = O.forward(cfg, w, t)
    got = m.forward_ragged([t[:300]], m.make_cache(1), want=[list(range(300))])
    per_pos = sorted(O.logits_error(got[i:i + 1], want[i:i + 1]) for i in range(300))
    assert per_pos[150] < BF16_TOL and per_pos[-1] < 1.0, per_pos[-3:]
    lens = [300, 70, 5]
    cache = utils._kv_pool.get_for(m, 3)
    first = m.forward_ragged([t[:n] for n in lens], cache, rows=[2, 0, 1])
    errs = [O.logits_error(first[i:i + 1], want[n - 1:n]) for i, n in enumerate(lens)]
    st = utils._decode_step_for(m, cache, 3, False)
    st.set_rows([2, 0, 1])
    for k in range(30):
        st.tok.copy_(torch.tensor([t[n + k] for n in lens], dtype=torch.int32))
        st.run()
        errs += [O.logits_error(st.logits[i:i + 1], want[n + k:n + k + 1]) for i, n in enumerate(lens)]
    errs.sort()
    assert errs[len(errs) // 2] < BF16_TOL and errs[-1] < 1.0, errs[-3:]


def test_experts_chosen_like_the_oracle(models):
    """The routed layer's choices, read back from the step's scratch, are the oracle's for every token."""
    cfg, m, w = models["mixed"]
    t = toks(cfg, 20, 9)
    res = []
    O.forward(cfg, w, t, res)
    m.forward_ragged([t], m.make_cache(1))
    # the last routed run is layer 2 (4 experts, 3 chosen): recompute its input from the oracle's residual before it
    x_in = res[-3]
    h = O.norm_one_plus(x_in, w["l2.norm1"].double(), cfg["norm"]["eps"])
    chosen = []
    O.routed_experts(h, {k: v.double() for k, v in w.items()}, "l2.mlp.", cfg["layers"][2]["mlp"], chosen)
    a = next(iter(m._arenas.values()))
    ids = a["s"].get("moe_ids", torch.int32, len(t), 3).cpu().tolist()
    assert [sorted(r) for r in ids] == chosen


@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_and_single_tokens_equal_one_pass(models, name):
    """A prompt cut into portions of 1, 2, 3, ... tokens, and fed token by token, gives the logits of one pass; the portions
    cross the convolution's reach, the attention's chunks and the temperature's blocks."""
    cfg, m, w = models[name]
    t = toks(cfg, 50, 4)
    want = O.forward(cfg, w, t)
    for cuts in ([50], [1, 2, 3, 5, 8, 13, 18], [2] * 25, [1] * 50, [47, 1, 2], [49, 1], [33, 17]):
        cache = m.make_cache(3)
        got, lo = [], 0
        for n in cuts:
            got.append(m.forward_ragged([t[lo:lo + n]], cache, rows=[2], want=[list(range(n))]))
            lo += n
        assert O.logits_error(torch.cat(got), want) < F32_TOL, cuts


@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_decode_step_graph_against_prompt(models, name):
    """Most of a prompt in one pass, the rest through the engine's captured decode step (the generation path)."""
    from mlx_parallm_b200 import utils
    cfg, m, w = models[name]
    t = toks(cfg, 100, 5)
    want = O.forward(cfg, w, t)
    cache = utils._kv_pool.get_for(m, 1)
    got = [m.forward_ragged([t[:30]], cache, want=[[29]])]
    st = utils._decode_step_for(m, cache, 1, False)
    for tok in t[30:]:
        st.tok.copy_(torch.tensor([tok], dtype=torch.int32))
        st.run()
        got.append(st.logits.clone())
    assert O.logits_error(torch.cat(got), want[29:]) < F32_TOL
    assert cache[-1].offsets == [100]
    # a second group of the same batch size, stepped in turns with the first one whose row list differs
    big = utils._kv_pool.get_for(m, 3)
    m.forward_ragged([t[:30]], big, rows=[2])
    st2 = utils._decode_step_for(m, big, 1, False)
    st2.set_rows([2])
    cache1 = m.make_cache(1)
    m.forward_ragged([t[:30]], cache1)
    st1 = utils._decode_step_for(m, cache1, 1, False)
    for k, tok in enumerate(t[30:36]):
        for s_ in (st2, st1):
            s_.tok.copy_(torch.tensor([tok], dtype=torch.int32))
            s_.run()
            assert torch.equal(s_.logits, got[1 + k]), (k, s_ is st1)


def test_ragged_batch_equals_each_alone_and_rows_end_early(models):
    """Four prompts of 1, 2, 17 and 40 tokens in one pass, then decoded together while the short ones end: equal to each
    request alone in a cache of its own, and right against the oracle."""
    from mlx_parallm_b200 import utils
    cfg, m, w = models["mixed"]
    lens, extra = [1, 2, 17, 40], [0, 3, 12, 12]
    seqs = [toks(cfg, n + e, 10 + n) for n, e in zip(lens, extra)]
    cache = utils._kv_pool.get_for(m, 4)
    rows = [2, 0, 3, 1]
    first = m.forward_ragged([s[:n] for s, n in zip(seqs, lens)], cache, rows=rows, want=[list(range(n)) for n in lens])
    together = {i: [] for i in range(4)}
    o = 0
    for i, n in enumerate(lens):
        together[i].append(first[o:o + n])
        o += n
    m.release_rows(cache, [rows[0]])
    for k in range(12):
        live = [i for i in range(1, 4) if k < extra[i]]
        st = utils._decode_step_for(m, cache, len(live), False)
        st.set_rows([rows[i] for i in live])
        st.tok.copy_(torch.tensor([seqs[i][lens[i] + k] for i in live], dtype=torch.int32))
        st.run()
        for j, i in enumerate(live):
            together[i].append(st.logits[j:j + 1].clone())
        if k + 1 == extra[1]:
            m.release_rows(cache, [rows[1]])
    for i in range(4):
        got = torch.cat(together[i])
        assert O.logits_error(got, O.forward(cfg, w, seqs[i])) < F32_TOL
        alone_cache = m.make_cache(1)
        alone = [m.forward_ragged([seqs[i][:lens[i]]], alone_cache, want=[list(range(lens[i]))])]
        for tok in seqs[i][lens[i]:]:
            alone.append(m.forward_ragged([[tok]], alone_cache))
        assert torch.equal(torch.cat(alone), got), f"request {i} depends on its batch"


def test_rows_given_back_start_from_nothing(models):
    """A row that held a long sequence is released and takes a new one, alone and beside a row that goes on: the new sequence
    sees no state and no keys of the old one, in any pass of the span."""
    cfg, m, w = models["mixed"]
    cache = m.make_cache(2)
    old, keep, new = toks(cfg, 60, 20), toks(cfg, 30, 21), toks(cfg, 25, 22)
    m.forward_ragged([old, keep[:20]], cache)
    m.release_rows(cache, [0])
    assert cache[0].offsets == [0, 20]
    got = m.forward_ragged([new[:3], keep[20:]], cache, want=[[0, 1, 2], list(range(10))])
    assert O.logits_error(got[:3], O.forward(cfg, w, new)[:3]) < F32_TOL
    assert O.logits_error(got[3:], O.forward(cfg, w, keep)[20:]) < F32_TOL
    rest = m.forward_ragged([new[3:]], cache, rows=[0], want=[list(range(22))])
    assert O.logits_error(rest, O.forward(cfg, w, new)[3:]) < F32_TOL


def test_first_tokens_and_short_sequences(models):
    for name in ("mixed", "odd"):
        cfg, m, w = models[name]
        seqs = [toks(cfg, n, 30 + n) for n in (1, 1, 2, 3, 4)]
        got = m.forward_ragged(seqs, m.make_cache(5), want=[list(range(len(s))) for s in seqs])
        want = torch.cat([O.forward(cfg, w, s) for s in seqs])
        assert O.logits_error(got, want) < F32_TOL


def test_each_pass_of_the_span_keeps_its_own_state():
    """A layer that runs twice holds two states: decoding after a prompt must continue each pass from its own.  With one
    shared state (or the second pass starting from the first one's) the continuation differs from the oracle."""
    cfg = O.make_config([O.delta_layer(2, 2, 8, 8, conv=3), O.pair_layer(2, 1, 8, 8, 0.4, 2, 8, 8, [0.9, 0.99])], vocab=40, width=16,
                        loop=(0, 2, 2))
    m, w = build(cfg, seed=11)
    t = toks(cfg, 40, 3)
    want = O.forward(cfg, w, t)
    cache = m.make_cache(1)
    assert len(cache) == 4 + 1
    got = [m.forward_ragged([t[:25]], cache, want=[[24]])]
    for tok in t[25:]:
        got.append(m.forward_ragged([[tok]], cache))
    assert O.logits_error(torch.cat(got), want[24:]) < F32_TOL


def test_far_memory_of_the_linear_state():
    """A decay close to one keeps a token readable 150 positions later, across a portion boundary; without the first
    portion's state the answer is clearly different."""
    cfg = O.make_config([O.pair_layer(1, 1, 8, 8, 0.3, 1, 32, 8, [0.9995], left_scale=0.05, right_scale=2.0)], vocab=40, width=16)
    m, w = build(cfg, seed=9)
    t = toks(cfg, 160, 6)
    t2 = list(t)
    t2[3] = (t[3] + 1) % 40
    a, b = O.forward(cfg, w, t)[-1], O.forward(cfg, w, t2)[-1]
    assert O.logits_error(a[None], b[None]) > 1e-3
    cache = m.make_cache(1)
    m.forward_ragged([t[:80]], cache)
    got = m.forward_ragged([t[80:]], cache)
    assert O.logits_error(got, a[None]) < F32_TOL
    lost = m.forward_ragged([t[80:]], m.make_cache(1))
    assert O.logits_error(lost, a[None]) > 1e-2


def test_long_decoding(models):
    from mlx_parallm_b200 import utils
    cfg, m, w = models["odd"]
    t = toks(cfg, 330, 8)
    want = O.forward(cfg, w, t)
    cache = utils._kv_pool.get_for(m, 1)
    m.forward_ragged([t[:5]], cache)
    st = utils._decode_step_for(m, cache, 1, False)
    got = []
    for tok in t[5:]:
        st.tok.copy_(torch.tensor([tok], dtype=torch.int32))
        st.run()
        got.append(st.logits.clone())
    assert O.logits_error(torch.cat(got), want[5:]) < F32_TOL


def test_greedy_generation_through_generate_step(models):
    """The engine's own entry point: left-padded prompts with their lengths, prefill, then the captured decode step feeding
    its own argmax back.  Compared with greedy decoding of the oracle, request by request."""
    from mlx_parallm_b200 import utils
    cfg, m, w = models["mixed"]
    prompts = [toks(cfg, n, 40 + n) for n in (3, 9, 6)]
    L = max(len(p) for p in prompts)
    padded = torch.tensor([[0] * (L - len(p)) + p for p in prompts])
    n_new = 8
    gen = utils.generate_step(padded, m, prompt_lengths=[len(p) for p in prompts])
    got = torch.cat([y for _, (y, _) in zip(range(n_new), gen)], 1).cpu().tolist()
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            lg = O.forward(cfg, w, seq)[-1]
            best = int(lg.argmax())
            assert tok == best or float(lg[best] - lg[tok]) < 1e-3 * float(lg.abs().max())
            seq.append(tok)


def test_batch_generate_front_end(models):
    from fake_tokenizer import FakeTokenizer
    from mlx_parallm_b200 import utils
    from mlx_parallm_b200.tokenizer_utils import TokenizerWrapper
    cfg, m, w = models["mixed"]
    tok = TokenizerWrapper(FakeTokenizer(vocab_size=cfg["vocab"]))
    out = utils.batch_generate(m, tok, ["w5 w6", "w5 w6 w7 w8 w9 w10 w11"], max_tokens=5, format_prompts=False)
    alone = utils.batch_generate(m, tok, ["w5 w6"], max_tokens=5, format_prompts=False)
    assert len(out) == 2 and out[0] == alone[0]


def test_checkpoint_on_disk_and_trace_runner(tmp_path, models):
    """config.json + model.safetensors through load_model (the registry picks the class by the architecture's name), then the
    command-line trace runner on the same folder: prompt, decode steps and a request that ends early, against the oracle."""
    import json
    import os
    import subprocess
    import sys
    from safetensors.torch import save_file
    cfg, _, w = models["odd"]
    d = tmp_path / "model"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
    wb = {k: v.to(torch.bfloat16) for k, v in w.items()}
    a, b = toks(cfg, 12, 1), toks(cfg, 5, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:9], "want": [0, 8]}, {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[9:10], "want": [0]}, {"id": "b", "tokens": b[4:5], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[10:11], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[11:12], "want": [0]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wbb = O.forward(cfg, wb, a), O.forward(cfg, wb, b)
    V = cfg["vocab"]
    s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, V))
    assert O.logits_error(s0, torch.stack([wa[0], wa[8], wbb[3]])) < F32_TOL
    s1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    assert O.logits_error(s1, wa[9:10]) < F32_TOL
    assert not (out / "2.f32").exists()
    s3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4").reshape(1, V))
    assert O.logits_error(s3, wa[11:12]) < F32_TOL
