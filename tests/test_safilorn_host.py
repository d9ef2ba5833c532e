"""Host-side parts of the Safilorn design that need no GPU: the configuration reader, the registry, the frequency table, the
pool's layout for its two kinds of state, and the oracle's own consistency (a sequence recomputed from its first token must
not depend on what follows a position; the recurrence cut in two gives the same as in one piece)."""
import math

import pytest
import torch

from tests import safilorn_oracle as O


def test_config_reader_and_registry():
    from promptcache_b200.model import MODEL_REGISTRY, Safilorn  # noqa: F401
    from promptcache_b200.model.safilorn import SafilornConfig
    assert "Safilorn" in MODEL_REGISTRY
    cfg = SafilornConfig({k: v for k, v in O.make_config([O.latent_layer(), O.gla_layer(mlp=None)], width=48, embed_scale=2.5).items() if not k.startswith("_")})
    assert (cfg.width, cfg.num_hidden_layers, cfg.embedding_scale, cfg.eps) == (48, 2, 2.5, 1e-5)
    assert cfg.layers[0]["type"] == "latent_attention" and cfg.layers[1]["mlp"] is None and cfg.layers[0]["mlp"]["kind"] == "dense"
    bad = O.make_config([O.gla_layer()])
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError):
        SafilornConfig(bad)
    bad = O.make_config([O.gla_layer()])
    bad["layers"][0]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError):
        SafilornConfig(bad)


def test_frequency_ramp():
    from promptcache_b200.model.safilorn import ramp_scaled_frequencies
    f, m = ramp_scaled_frequencies(16, 10000.0, None)
    assert f == pytest.approx([10000.0 ** (-2 * i / 16) for i in range(8)]) and m == 1.0
    sc = {"factor": 8.0, "original": 64, "fast": 4.0, "slow": 0.5}
    g, m = ramp_scaled_frequencies(16, 10000.0, sc)
    go, mo = O.scaled_frequencies(16, 10000.0, sc)
    assert g == pytest.approx(go, rel=1e-14) and m == pytest.approx(mo) and m == pytest.approx(0.1 * math.log(8.0) + 1.0)
    lo = max(math.floor(16 * math.log(64 / (2 * math.pi * 4.0)) / (2 * math.log(10000.0))), 0)
    hi = min(math.ceil(16 * math.log(64 / (2 * math.pi * 0.5)) / (2 * math.log(10000.0))), 15)
    for i, (a, b) in enumerate(zip(f, g)):
        if i <= lo:
            assert b == a
        elif i >= hi:
            assert b == pytest.approx(a / 8)
        else:
            assert a / 8 < b < a
    assert ramp_scaled_frequencies(0, 10000.0, sc)[0] == []


def test_pool_layout_for_latent_rows_and_decaying_states():
    from promptcache_b200.model._state import DecayStateSpec, LatentKVSpec, SeqState, SlotPool
    pool = SlotPool([LatentKVSpec(10, 4), DecayStateSpec(2, 8, 12)], torch.float32, "cpu", n_slots=1, cap=128)
    assert set(pool.layers[0]) == {"ckv"} and set(pool.layers[1]) == {"s"}
    assert tuple(pool.layers[0]["ckv"].shape) == (1, 1, 128, 14) and tuple(pool.layers[1]["s"].shape) == (1, 2, 8, 12)
    a = SeqState(pool)
    pool.layers[0]["ckv"][a.slot, :, :3] = 2.0
    pool.layers[1]["s"][a.slot] = 5.0
    b = SeqState(pool)                       # the pool doubles; what live slots hold is carried over
    assert pool.n_slots == 2 and float(pool.layers[0]["ckv"][a.slot, :, :3].min()) == 2.0 and float(pool.layers[1]["s"][a.slot].min()) == 5.0
    pool.reserve(b.slot, 300)                # more rows per slot: the latent rows move, the states are copied as they are
    assert pool.cap >= 300 and float(pool.layers[0]["ckv"][a.slot, :, :3].min()) == 2.0 and float(pool.layers[1]["s"][a.slot].max()) == 5.0
    assert pool.layers[1]["s"].dtype == torch.float32
    half = SlotPool([LatentKVSpec(10, 4), DecayStateSpec(2, 8, 12)], torch.bfloat16, "cpu")
    assert half.layers[0]["ckv"].dtype == torch.bfloat16 and half.layers[1]["s"].dtype == torch.float32   # the state stays 32-bit


def test_oracle_is_causal_and_its_recurrence_can_be_cut():
    cfg = O.make_config([O.latent_layer(), O.gla_layer(), O.gla_layer(mlp="dense")], width=24)
    W = O.random_model(cfg, seed=1)
    toks = [3, 9, 27, 20, 1, 2, 3, 4, 5, 6, 7, 8]
    full = O.forward(cfg, W, toks)
    assert torch.allclose(O.forward(cfg, W, toks[:7]), full[:7], atol=1e-12)
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    alpha = torch.rand(9, 2, 4, generator=g, dtype=torch.float64)
    o = O.gla_recurrence(q, k, v, alpha)
    # closed form of the last step: o_T = sum_s (prod_{r > s} alpha_r * k_s . q_T) v_s
    want = torch.zeros(2, 4, dtype=torch.float64)
    for s in range(9):
        w = (torch.prod(alpha[s + 1:], 0) * k[s] * q[8]).sum(-1)
        want += w[:, None] * v[s]
    assert torch.allclose(o[8], want, atol=1e-12)
    # a sink that outweighs every key leaves nothing; one without weight leaves the plain softmax
    s = torch.tensor([0.3, -1.0, 2.0], dtype=torch.float64)
    assert float(O.softmax_with_sink(s, 60.0).sum()) < 1e-20
    assert torch.allclose(O.softmax_with_sink(s, -60.0), torch.softmax(s, 0), atol=1e-12)
