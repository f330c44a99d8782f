"""Host-side parts of the Dogulorn integration (no GPU): registry, config validation, row bookkeeping, and known answers
of the oracle that the GPU tests lean on."""
import pytest
import torch

import dogulorn_oracle as O


def test_registry_resolves_the_architecture_key():
    from mlx_parallm_b200.utils import _get_classes
    cfg = O.make_config([O.delta_layer(2, 1, 4, 4, conv=2)])
    Model, Args = _get_classes(cfg)
    assert Model.__module__.endswith("models.dogulorn") and Model.dense and Model.supports_ragged
    a = Args.from_dict(dict(cfg, something_else=1))
    assert a.vocab_size == cfg["vocab"] and a.model_type == "dogulorn"
    with pytest.raises(ValueError):
        _get_classes({"vocab": 3})


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"].__setitem__(0, dict(c["layers"][0], type="conv")),
    lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1),
    lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 0),
    lambda c: c["layers"][2]["mixer"].__setitem__("kv_rank", 24),
    lambda c: c["layers"][2].__setitem__("mlp", {"kind": "experts", "ff": 8, "limit": 1.0}),
    lambda c: c["norm"].__setitem__("kind", "layer"),
])
def test_config_validation(bad):
    from mlx_parallm_b200.models.dogulorn import ModelArgs
    cfg = O.make_config([O.delta_layer(2, 1, 4, 4, conv=2), O.attn_layer(2, 4, 4, 8, 16, window=3),
                         O.attn_layer(2, 4, 4, 8, 16, window=3, kv_from=1)])
    ModelArgs.from_dict(cfg)
    bad(cfg)
    with pytest.raises((ValueError, NotImplementedError)):
        ModelArgs.from_dict(cfg)


def test_model_layout_follows_the_config():
    from mlx_parallm_b200.models.dogulorn import Model, ModelArgs
    cfg = O.make_config([O.attn_layer(3, 8, 16, 24, 32, window=7, scale=0.3, mlp={"kind": "dense", "ff": 40, "limit": 1.5}),
                         O.delta_layer(4, 2, 16, 8, conv=4), O.attn_layer(2, 16, 8, 16, 32, window=0, kv_from=0)])
    m = Model(ModelArgs.from_dict(cfg))
    assert [s.kind for s in m.sublayers] == ["mixer", "mlp", "side", "mixer", "side", "mixer", "side"]
    assert sorted(m.parameter_names()) == sorted(O.random_weights(cfg).keys())
    att, delta, shared = m.mixers
    assert (att.window, att.scale, att.own_kv, shared.own_kv, shared.kv_from, shared.window) == (7, 0.3, True, False, 0, 0)
    assert shared.scale == 16 ** -0.5 and delta.n_proj == 2 * 2 * 16 + 2 * 4 * 8 + 2 * 4 and delta.taps == 4
    states = m.new_cache(3)
    assert [type(s).__name__ for s in states] == ["LatentKVCache", "DeltaRuleState", "RowState", "TokenState"]
    with pytest.raises(KeyError):
        m.load_weights({}, device="cpu")


def test_row_bookkeeping():
    from mlx_parallm_b200.models.base import BatchedKVCache, LatentKVCache, RowState
    from mlx_parallm_b200.models._transformer import advance_rows, release_rows
    group = [LatentKVCache(8, 3), RowState(3), BatchedKVCache(4, 2, 3)]
    advance_rows(group, [2, 0], [5, 1])
    assert all(c.offsets == [1, 0, 5] and c.offset == 5 for c in group)
    release_rows(group, [2])
    assert all(c.offsets == [1, 0, 0] for c in group)
    lat = group[0]
    assert lat.ensure_capacity(300, torch.float32, "cpu") and lat.latent.shape == (3, 512, 8)
    lat.latent[0, 0, 0] = 7.0
    assert not lat.ensure_capacity(512, torch.float32, "cpu")
    assert lat.ensure_capacity(513, torch.float32, "cpu") and lat.capacity == 768 and float(lat.latent[0, 0, 0]) == 7.0
    lat.reset(2)
    assert lat.latent is None and lat.offsets == [0, 0]


def test_oracle_known_answers():
    # hashed pair index by hand: buckets 5, multipliers 3 and 2: tokens 4, 1, 3 -> rows 5 (first), (12 + 2) % 5 = 4, (3 + 6) % 5 = 4
    embed = torch.arange(10, dtype=torch.float64).view(5, 2)
    bigram = 100.0 * torch.arange(6, dtype=torch.float64)[:, None].expand(6, 2)
    x = O.hashed_embedding([4, 1, 3], embed, bigram, 0.5, 5, 3, 2)
    assert x.tolist() == [[504.0, 504.5], [401.0, 401.5], [403.0, 403.5]]
    # convolution: the last tap is the current token's, earlier inputs are zero before the start
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    z = O.short_conv_silu(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert torch.allclose(z, O.silu(torch.tensor([[1.0], [12.0], [124.0]], dtype=torch.float64)))
    # delta rule with unit decay, beta one and orthogonal unit keys is an exact key -> value store
    # (checked on the recurrence itself, written out here once more)
    k = torch.eye(3, dtype=torch.float64)
    v = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=torch.float64)
    S = torch.zeros(3, 2, dtype=torch.float64)
    for t in range(3):
        S = S + torch.outer(k[t], v[t] - S.T @ k[t])
    assert torch.equal(S.T @ k[1], v[1])
    # window of size w: position i sees exactly w positions (itself and w - 1 before it)
    cfg = O.make_config([O.attn_layer(1, 4, 4, 4, 4, window=3)], vocab=11, width=8, bigram=None, side_dim=0)
    w = O.random_weights(cfg, 1)
    t = [1, 2, 3, 4, 5, 6, 7]
    base = O.forward(cfg, w, t)[-1]
    far = O.forward(cfg, w, [9] + t[1:5] + t[5:])[-1]           # token 0 is 6 back: outside
    edge_out = O.forward(cfg, w, t[:3] + [9] + t[4:])[-1]       # position 3 is 3 back: outside
    edge_in = O.forward(cfg, w, t[:4] + [9] + t[5:])[-1]        # position 4 is 2 back: inside
    assert torch.equal(base, far) and torch.equal(base, edge_out) and not torch.equal(base, edge_in)
