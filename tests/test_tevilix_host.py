"""Host-side parts of the Tevilix design that need no GPU: the configuration reader with its loop, the registry, the frequency
table, the pool's layout for a layer that keeps K/V rows beside a vector state, and the oracle's own consistency (causality;
the gated recurrence as a composition of affine maps, which is what the scan kernel relies on; the router's group rule)."""
import pytest
import torch

from tests import tevilix_oracle as O

F64 = torch.float64


def test_config_reader_loop_and_registry():
    from promptcache_b200.model import MODEL_REGISTRY, Tevilix  # noqa: F401
    from promptcache_b200.model.tevilix import TevilixConfig, layer_runs
    assert "Tevilix" in MODEL_REGISTRY
    layers = [O.parallel_layer(), O.mlstm_layer(mlp=None), O.mlstm_layer(mlp=O.moe()), O.parallel_layer(mlp=O.moe(groups=0))]
    cfg = TevilixConfig(O.make_config(layers, width=48, embed_scale=2.25, loop=(1, 3, 2)))
    assert (cfg.width, cfg.num_hidden_layers, cfg.embedding_scale, cfg.eps) == (48, 4, 2.25, 1e-5)
    assert cfg.runs == [0, 1, 2, 1, 2, 3] == O.layer_runs(O.make_config(layers, loop=(1, 3, 2)))
    assert cfg.layers[1]["mlp"] is None and cfg.layers[2]["mlp"]["kind"] == "moe" and cfg.layers[0]["type"] == "parallel"
    assert layer_runs(3, None) == [0, 1, 2] and layer_runs(3, {"start": 0, "stop": 3, "times": 2}) == [0, 1, 2, 0, 1, 2]
    assert layer_runs(3, {"start": 2, "stop": 2, "times": 5}) == [0, 1, 2]         # an empty span
    assert layer_runs(4, {"start": 3, "stop": 4, "times": 3}) == [0, 1, 2, 3, 3, 3]
    with pytest.raises(ValueError):
        layer_runs(3, {"start": 2, "stop": 5, "times": 2})
    bad = O.make_config([O.mlstm_layer()])
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError):
        TevilixConfig(bad)
    bad = O.make_config([O.mlstm_layer()])
    bad["layers"][0]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError):
        TevilixConfig(bad)


def test_divided_frequencies():
    from promptcache_b200.model.tevilix import divided_frequencies
    f = divided_frequencies(8, 1000.0, 4.0)
    assert f == pytest.approx([1000.0 ** (-2 * i / 8) / 4.0 for i in range(4)], rel=1e-15)
    assert f == pytest.approx(O.rotary_frequencies(8, 1000.0, 4.0), rel=1e-15)
    assert divided_frequencies(6, 50.0) == pytest.approx([50.0 ** (-i / 3) for i in range(3)]) and divided_frequencies(0, 10.0) == []


def test_pool_layout_per_layer_run():
    from promptcache_b200.model._state import KVSpec, MatrixMemorySpec, SeqState, SlotPool, VectorStateSpec
    specs = [(KVSpec(2, 6, 5), VectorStateSpec(9)), MatrixMemorySpec(2, 4, 3), MatrixMemorySpec(2, 4, 3)]   # the last two: one layer, two passes
    pool = SlotPool(specs, torch.bfloat16, "cpu", n_slots=1, cap=128)
    assert set(pool.layers[0]) == {"k", "v", "vec"} and set(pool.layers[1]) == {"s", "n", "m"}
    assert tuple(pool.layers[0]["vec"].shape) == (1, 9) and pool.layers[0]["vec"].dtype == torch.float32 and pool.layers[0]["k"].dtype == torch.bfloat16
    assert pool.layers[1]["s"].data_ptr() != pool.layers[2]["s"].data_ptr()                                  # every pass has a state of its own
    a = SeqState(pool)
    pool.layers[0]["vec"][a.slot] = 3.0
    pool.layers[0]["k"][a.slot, :, :4] = 2.0
    b = SeqState(pool)                       # the pool doubles; what live slots hold is carried over
    pool.reserve(b.slot, 300)                # more rows per slot: K/V rows move, the vector state is copied as it is
    assert pool.n_slots == 2 and pool.cap >= 300
    assert float(pool.layers[0]["vec"][a.slot].min()) == 3.0 and float(pool.layers[0]["k"][a.slot, :, :4].min()) == 2.0
    assert float(pool.layers[0]["k"][a.slot, :, 4:].abs().max()) == 0.0


def test_oracle_is_causal_and_its_window_forgets():
    cfg = O.make_config([O.parallel_layer(window=4), O.mlstm_layer(), O.parallel_layer(window=3, mlp=O.moe())], width=24, loop=(0, 2, 2))
    W = O.random_model(cfg, seed=1)
    toks = [3, 9, 27, 20, 1, 2, 3, 4, 5, 6, 7, 8]
    full = O.forward(cfg, W, toks)
    assert torch.allclose(O.forward(cfg, W, toks[:7]), full[:7], atol=1e-12)
    # attention alone with a window: a key outside it changes nothing, the one just inside does
    g = torch.Generator().manual_seed(0)
    q, k, v = torch.randn(1, 2, 4, generator=g, dtype=F64), torch.randn(6, 2, 4, generator=g, dtype=F64), torch.randn(6, 2, 3, generator=g, dtype=F64)
    pq, pk = torch.tensor([5]), torch.arange(6)
    talk = torch.tensor([[1.0, 0.5], [-0.25, 2.0]], dtype=F64)
    o = O.mixed_score_attention(q, k, v, pq, pk, 0.5, talk, 3)
    v2 = v.clone()
    v2[2] += 100.0                            # 5 - 2 = 3: outside a window of 3
    assert torch.equal(O.mixed_score_attention(q, k, v2, pq, pk, 0.5, talk, 3), o)
    v2 = v.clone()
    v2[3] += 100.0                            # 5 - 3 = 2: inside
    assert not torch.allclose(O.mixed_score_attention(q, k, v2, pq, pk, 0.5, talk, 3), o)
    # the mixing by hand for one pair of heads and one key
    s = torch.stack([(q[0, h] * k[5, h]).sum() * 0.5 for h in range(2)])
    one = O.mixed_score_attention(q, k[5:], v[5:], pq, pk[5:], 0.5, talk, 0)
    assert torch.allclose(one[0], v[5]) and torch.isfinite(talk @ s).all()


def test_gated_recurrence_is_a_composition_of_affine_maps():
    g = torch.Generator().manual_seed(2)
    z, u = torch.rand(11, 5, generator=g, dtype=F64), torch.randn(11, 5, generator=g, dtype=F64)
    c = O.gru_candidate(u)
    assert torch.equal(c[u >= 0], u[u >= 0] + 0.5) and torch.allclose(c[u < 0], torch.sigmoid(u[u < 0]))
    out, S = O.gru_recurrence(z, c)
    # cut in two: the second part continues from the first part's state
    o1, S1 = O.gru_recurrence(z[:4], c[:4])
    o2, S2 = O.gru_recurrence(z[4:], c[4:], S1)
    assert torch.allclose(torch.cat([o1, o2]), out, atol=1e-14) and torch.allclose(S2, S, atol=1e-14)
    # a stretch folded into (A, B): S_end = A S_start + B
    A, B = torch.ones(5, dtype=F64), torch.zeros(5, dtype=F64)
    for t in range(4, 11):
        A, B = A * (1 - z[t]), (1 - z[t]) * B + z[t] * c[t]
    assert torch.allclose(A * S1 + B, S, atol=1e-14)


def test_router_groups_and_weights():
    h = torch.eye(6, dtype=F64)[:1] * 0 + 1.0
    # six experts in three groups; logits chosen so that the group of experts 2 and 3 has the best PAIR although expert 4 is the best single
    z = torch.tensor([[-1.0, -2.0, 1.0, 0.9, 1.5, -3.0]], dtype=F64)
    w_router = z.T / 6.0 * torch.ones(1, 6, dtype=F64)
    idx, w = O.route(h, w_router, None, 2, 3, 1, 1.75)
    assert sorted(idx[0].tolist()) == [2, 3]
    s = torch.sigmoid(z[0])
    assert torch.allclose(w[0].sum(), torch.tensor(1.75, dtype=F64)) and torch.allclose(w[0, 0] / w[0, 1], s[2] / s[3])
    # a correction that decides the choice does not enter the weights
    corr = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 5.0], dtype=F64)
    idx, w = O.route(h, w_router, corr, 1, 1, 1, 1.0)
    assert idx[0].tolist() == [5] and torch.allclose(w[0, 0], torch.tensor(1.0, dtype=F64))
    # with two kept groups out of three the single best expert is reachable again
    idx, _ = O.route(h, w_router, None, 2, 3, 2, 1.0)
    assert 4 in idx[0].tolist()
