"""Host-side logic of the Pupopel family that needs no GPU: the registry, the configuration's checks, the order of layer runs
of a looped span, the parameter list, and the oracle's own consistency."""
import pytest
import torch

import pupopel_oracle as O


def cfg_small(loop=None):
    return O.make_config([
        O.delta_layer(2, 1, 8, 8, conv=3, mlp=O.dense_mlp(16)),
        O.pair_layer(4, 2, 8, 8, 0.3, 2, 8, 8, [0.8, 0.9], mlp=O.moe_mlp(3, 2, 8, shared_ff=8)),
        O.delta_layer(2, 2, 8, 8, conv=2),
    ], vocab=20, width=16, loop=loop)


def test_registry_and_parameter_names():
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small(loop=(0, 2, 2))
    Model, Args = _get_classes(cfg)
    m = Model(Args.from_dict(cfg))
    assert m.model_type == "pupopel" and m.block_style == "parallel"
    assert sorted(m.parameter_names()) == sorted(O.random_weights(cfg).keys())
    no_loop = Model(Args.from_dict(cfg_small()))
    assert "loop.in" not in no_loop.parameter_names() and no_loop.loop_in is None


@pytest.mark.parametrize("loop,want", [
    (None, [(0, False), (1, False), (2, False)]),
    ((0, 2, 2), [(0, True), (1, False), (0, True), (1, False), (2, False)]),
    ((1, 3, 3), [(0, False)] + [(1, True), (2, False)] * 3),
    ((1, 2, 1), [(0, False), (1, True), (2, False)]),
    ((2, 2, 4), [(0, False), (1, False), (2, False)]),
])
def test_run_order_of_a_looped_span(loop, want):
    from mlx_parallm_b200.models._sequence import unroll_layers
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small(loop=loop)
    assert O.layer_runs(cfg) == want
    lp = cfg.get("loop") or {}
    assert unroll_layers(3, lp.get("start", 0), lp.get("stop", 0), lp.get("times", 1)) == want
    Model, Args = _get_classes(cfg)
    m = Model(Args.from_dict(cfg))
    assert [(r.layer, r.opens) for r in m.runs] == want
    assert [r.slot for r in m.runs] == list(range(len(want)))            # one state per run, also for a layer that runs again
    for r in m.runs:
        assert r.mixer is m.mixers[r.layer]                                # the same modules (weights) every pass


def test_config_checks():
    from mlx_parallm_b200.utils import _get_classes
    cfg = cfg_small()
    Model, Args = _get_classes(cfg)
    bad = dict(cfg, layers=[dict(cfg["layers"][0], type="delta")])
    with pytest.raises(NotImplementedError):
        Args.from_dict(bad)
    bad = dict(cfg, layers=[dict(cfg["layers"][0], mlp={"kind": "sparse"})])
    with pytest.raises(NotImplementedError):
        Args.from_dict(bad)
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, loop={"start": 2, "stop": 5, "times": 2}))
    with pytest.raises(ValueError):
        Args.from_dict(dict(cfg, layers=[O.delta_layer(3, 2, 8, 8, conv=2)]))


def test_oracle_prefix_property_and_sink():
    """The oracle is causal (a prefix gives the prefix's logits) and its sink only damps: these hold for any correct statement
    of the design and guard the oracle itself."""
    cfg = cfg_small(loop=(0, 2, 2))
    w = O.random_weights(cfg, 1)
    t = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5]
    full = O.forward(cfg, w, t)
    assert (O.forward(cfg, w, t[:6]) - full[:6]).abs().max() < 1e-9
    h = torch.randn(7, 16, dtype=O.F64)
    P = {k: v.double() for k, v in w.items()}
    m = cfg["layers"][1]["mixer"]["left"]
    a = O.sink_attention(h, P, "l1.mix.left.", m, 1e-5)
    P2 = dict(P)
    P2["l1.mix.left.sink"] = P["l1.mix.left.sink"] - 50.0                # no sink to speak of: plain softmax
    b = O.sink_attention(h, P2, "l1.mix.left.", m, 1e-5)
    assert (a - b).abs().max() > 1e-4
    # first token: one key and the sink share the softmax, so the output is the value row damped by a factor below one
    P3 = dict(P)
    P3["l1.mix.left.o"] = torch.eye(32, dtype=O.F64)[:16]                # reads heads 0 and 1 directly
    first = O.sink_attention(h[:1], P3, "l1.mix.left.", dict(m, q_temp=None), 1e-5)[0]
    v0 = (h[:1] @ P["l1.mix.left.v"].T).view(2, 8)[0]
    ratio = first[:8] / v0
    assert float(ratio.max() - ratio.min()) < 1e-9 and 0.0 < float(ratio[0]) < 1.0
