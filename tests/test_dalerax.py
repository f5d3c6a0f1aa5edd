"""Dalerax without a GPU: the configuration, the plan against the checkpoint layout, what the
layers ask of the cache, and the plain implementation's mechanisms against hand-worked numbers."""
import copy
import math

import numpy as np
import pytest

import plain_dalerax as plain
from tiny_configs import DALERAX_A, DALERAX_B, DALERAX_C


def test_configuration_reports_every_problem_at_once():
    from gemmars_b200.config.base import ConfigError
    from gemmars_b200.models.dalerax import DaleraxConfig
    cfg = DaleraxConfig.from_dict(DALERAX_A)
    assert cfg.vocab == 211 and cfg.logit_scale == 1.3 and cfg.embedding_scale == 3.0 and len(cfg.layers) == 5
    assert DaleraxConfig.from_dict(cfg.to_dict()) == cfg
    bad = copy.deepcopy(DALERAX_A)
    bad["layers"][1]["mixer"]["rot"]["dims"] = 34                   # more than dim
    bad["layers"][2]["mixer"]["heads"] = 5                          # not a multiple of kv_heads
    bad["layers"][0]["type"] = "conv"
    del bad["embedding"]
    bad["layers"][3]["mixer"]["kv_from"] = 2                        # other sizes than layer 2's
    bad["layers"][4]["mlp"]["router"]["top"] = 4                    # of 3 experts
    bad["layers"][1]["mlp"]["kind"] = "sparse"
    with pytest.raises(ConfigError) as e:
        DaleraxConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("rot.dims", "5 heads", "unknown mixer 'conv'", "embedding.scale", "kv_from: dim", "top: 4 of 3",
                  "unknown feed-forward 'sparse'"):
        assert piece in text, piece
    for j in (3, 4, 0):        # itself, a later layer, a recurrent layer
        bad = copy.deepcopy(DALERAX_A)
        bad["layers"][3]["mixer"]["kv_from"] = j
        with pytest.raises(ConfigError):
            DaleraxConfig.from_dict(bad)
    chain = copy.deepcopy(DALERAX_B)
    chain["layers"].append(copy.deepcopy(chain["layers"][2]))
    chain["layers"][4]["mixer"]["kv_from"] = 2                      # a layer that has no keys of its own
    with pytest.raises(ConfigError):
        DaleraxConfig.from_dict(chain)


@pytest.mark.parametrize("raw", [DALERAX_A, DALERAX_B, DALERAX_C], ids="ABC")
def test_plan_wants_exactly_the_checkpoint(raw):
    from gemmars_b200.config.registry import resolve_architecture
    from gemmars_b200.engine.model import DecoderModel
    arch = resolve_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    model = DecoderModel(arch.build_plan(cfg, None), "float32", "cpu")
    layout = {name: tuple(shape) for name, (shape, _) in arch.checkpoint_layout(cfg).items()}
    assert model.expected_tensors() == layout
    assert model.plan.max_positions == raw["max_positions"]
    borrowers = [i for i, layer in enumerate(raw["layers"]) if "kv_from" in layer["mixer"]]
    for i in borrowers:
        assert f"l{i}.mix.k" not in layout and f"l{i}.mix.v" not in layout and f"l{i}.mix.q" in layout


def test_the_decay_rank_comes_from_the_checkpoint():
    """config.json of a released model names no rank: the rows of w1 give it."""
    from gemmars_b200.engine.model import build_model
    from gemmars_b200.weights import random_weights
    tensors = random_weights(DALERAX_C, 1)
    raw = copy.deepcopy(DALERAX_C)
    del raw["layers"][1]["mixer"]["rank"]
    model = build_model(raw_config=raw, tensors=tensors, dtype="float32", device="cpu", compile_kernels=False)
    assert model.blocks[1].mixer.rank == 3
    assert model.expected_tensors()["l1.mix.w2"] == (24, 3)


def test_what_the_layers_keep_per_sequence():
    import torch
    from gemmars_b200.cache.pool import KVNeed, SequenceCache, StateNeed
    from gemmars_b200.engine.model import build_model
    from gemmars_b200.weights import random_weights
    model = build_model(raw_config=DALERAX_A, tensors=random_weights(DALERAX_A, 1), dtype="float32", device="cpu",
                        compile_kernels=False)
    needs = dict(model.cache_needs())
    # a recurrent layer: the input of the token before, and a matrix a head (dims padded to 32 a lane)
    assert needs[0] == [StateNeed((72,)), StateNeed((3, 32 * 24))]
    assert needs[4] == [StateNeed((72,)), StateNeed((1, 64 * 40))]
    # a cache that another layer reads through another mask keeps every page; so does one with kept
    # first tokens; a plain window of its own is a ring
    assert needs[1] == [KVNeed(2, 32, None, 16)]
    assert needs[2] == [KVNeed(4, 16, 7, 24)]
    assert 3 not in needs                                           # the reader owns nothing
    assert [e.cache_of for e in model.plan.schedule] == [None, None, None, 1, None]
    cache = SequenceCache(model.cache_needs(), 512, 4, 600, 64, torch.float32, "cpu")
    slot = cache.open()
    cache.extend(slot, 300)
    widths = sorted(g.table_width for g in cache.kv_groups)
    assert widths[0] < 5 <= widths[1]                               # a ring, and 300 tokens' worth of pages
    for g in cache.state_groups:
        g.data[:, slot] = 1.0
    cache.close(slot)
    assert cache.pages_held() == 0
    assert cache.open() == slot
    assert not any(g.data[:, slot].any() for g in cache.state_groups)      # a slot taken again starts from zero


def test_stretched_wavelengths_by_hand():
    # base 10, 8 dims: f = 1, 10^-0.25, 10^-0.5, 10^-0.75; wavelengths 6.28, 11.2, 19.9, 35.3
    s = {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 24.0}
    f = plain.rotary_frequencies(10.0, 8)
    g = plain.rotary_frequencies(10.0, 8, s)
    assert np.allclose(f, [1.0, 10 ** -0.25, 10 ** -0.5, 10 ** -0.75])
    assert g[0] == f[0] and g[1] == f[1]                            # shorter than 24 / 2
    assert np.isclose(g[3], f[3] / 4.0)                             # longer than 24 / 1
    t = (24.0 * f[2] / (2 * math.pi) - 1.0) / (2.0 - 1.0)           # in between
    assert 0.0 < t < 1.0 and np.isclose(g[2], (1 - t) * f[2] / 4.0 + t * f[2])
    # the package's table is the same numbers
    import torch
    from gemmars_b200.parts.rotary import Rotary
    got = Rotary.scaled(torch.tensor(f, dtype=torch.float64), s).numpy()
    assert np.allclose(got, g, rtol=1e-12)
    for raw in (DALERAX_A, DALERAX_B, DALERAX_C):                   # every band is met by some test model
        rot = raw["layers"][1 if raw is DALERAX_A else 0]["mixer"]["rot"]
        a, b = plain.rotary_frequencies(rot["base"], rot["dims"]), plain.rotary_frequencies(rot["base"], rot["dims"], rot["scaling"])
        ratio = b / a
        assert np.isclose(ratio.max(), 1.0) and np.isclose(ratio.min(), 1.0 / rot["scaling"]["factor"])
    rot = DALERAX_A["layers"][1]["mixer"]["rot"]
    ratio = plain.rotary_frequencies(rot["base"], rot["dims"], rot["scaling"]) / plain.rotary_frequencies(rot["base"], rot["dims"])
    assert ((ratio > 0.2500001) & (ratio < 0.9999999)).any()        # and the blend in between by A


def test_rotation_of_halves_by_hand():
    x = np.zeros((2, 1, 6))
    x[:, 0] = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    out = plain.rotate_half(x, np.array([0, 3]), np.array([1.0, 0.1]))
    assert np.allclose(out[0], x[0])                                # position 0 turns nothing
    a0, a1 = 3.0, 0.3
    assert np.allclose(out[1, 0, [0, 2]], [np.cos(a0) - 3 * np.sin(a0), 3 * np.cos(a0) + np.sin(a0)])
    assert np.allclose(out[1, 0, [1, 3]], [2 * np.cos(a1) - 4 * np.sin(a1), 4 * np.cos(a1) + 2 * np.sin(a1)])
    assert np.allclose(out[1, 0, 4:], [5.0, 6.0])                   # beyond the rotated dims


def test_window_kept_tokens_and_sink_by_hand():
    assert [j for j in range(10) if plain.visible(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    assert [j for j in range(10) if plain.visible(3, j, 3, 2)] == [0, 1, 2, 3]        # kept and window overlap: once each
    assert [j for j in range(10) if plain.visible(9, j, 3, 0)] == [7, 8, 9]
    k = np.zeros((6, 1, 2))
    k[:, 0, 0] = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    v = np.arange(6.0).reshape(6, 1, 1)
    q = np.ones((1, 1, 2))
    # the query at position 5, a window of 2 and one kept token: keys 0, 4, 5 and the sink
    out = plain.sink_attention(q, k, v, [5], np.arange(6), 0.5, 2, 1, np.array([1.5]))
    e = np.exp([0.5, 2.5, 3.0])
    assert np.allclose(out[0, 0, 0], (e @ [0.0, 4.0, 5.0]) / (e.sum() + np.exp(1.5)))
    # a sink far below the scores changes nothing; one far above takes all the weight
    low = plain.sink_attention(q, k, v, [5], np.arange(6), 0.5, 2, 1, np.array([-80.0]))
    assert np.allclose(low[0, 0, 0], (e @ [0.0, 4.0, 5.0]) / e.sum())
    high = plain.sink_attention(q, k, v, [5], np.arange(6), 0.5, 2, 1, np.array([80.0]))
    assert abs(high[0, 0, 0]) < 1e-30
    # the first token sees itself and the sink
    first = plain.sink_attention(q, k[:1], v[:1] + 7.0, [0], [0], 0.5, 2, 1, np.array([0.5]))
    assert np.allclose(first[0, 0, 0], 7.0 * np.exp(0.5) / (np.exp(0.5) + np.exp(0.5)))


def test_decayed_linear_attention_by_hand():
    # one head of two key channels and two value channels
    r = np.array([[[1.0, 0.0]], [[1.0, 1.0]], [[0.0, 1.0]]])
    k = np.array([[[2.0, 0.0]], [[0.0, 1.0]], [[1.0, 1.0]]])
    v = np.array([[[1.0, 10.0]], [[2.0, 20.0]], [[3.0, 30.0]]])
    w = np.array([[[0.5, 0.25]], [[0.5, 0.25]], [[1.0, 1.0]]])
    u = np.array([[3.0, 5.0]])
    y, S = plain.wkv_scan(r, k, v, w, u)
    # token 0: the state is empty, the bonus alone: r . (u * k) = 6
    assert np.allclose(y[0, 0], [6.0, 60.0])
    # S = [[2, 20], [0, 0]] after token 0 (its own decay has nothing to act on)
    # token 1: S^T r = [2, 20]; bonus r . (u * k) = 5 -> + 5 v
    assert np.allclose(y[1, 0], [2.0 + 10.0, 20.0 + 100.0])
    # S = diag(.5, .25) S + k v^T = [[1, 10], [2, 20]]
    # token 2: S^T r = [2, 20]; bonus = 5 -> + [15, 150]
    assert np.allclose(y[2, 0], [17.0, 170.0])
    assert np.allclose(S[0], [[1.0 + 3.0, 10.0 + 30.0], [2.0 + 3.0, 20.0 + 30.0]])
    # carried on from a state: the same as one walk
    y01, S01 = plain.wkv_scan(r[:2], k[:2], v[:2], w[:2], u)
    y2, S2 = plain.wkv_scan(r[2:], k[2:], v[2:], w[2:], u, S01)
    assert np.allclose(y2[0], y[2]) and np.allclose(S2, S)
    # the row before the first is zeros, or what is handed in
    h = np.array([[1.0, 2.0], [3.0, 4.0]])
    assert np.allclose(plain.shifted(h), [[0.0, 0.0], [1.0, 2.0]])
    assert np.allclose(plain.shifted(h, [9.0, 8.0]), [[9.0, 8.0], [1.0, 2.0]])


def test_routing_by_hand():
    chosen, weights = plain.route(np.array([0.1, 2.0, -1.0, 1.0]), 2)
    assert chosen == [1, 3]
    assert np.allclose(weights, np.exp([2.0, 1.0]) / np.exp([2.0, 1.0]).sum())
    chosen, weights = plain.route(np.array([0.1, 2.0, -1.0]), 3)    # every expert: a plain softmax
    assert sorted(chosen) == [0, 1, 2] and np.isclose(weights.sum(), 1.0)
    chosen, weights = plain.route(np.array([0.1, 2.0, -1.0]), 1)    # one expert has all the weight
    assert chosen == [1] and np.allclose(weights, [1.0])


def test_the_first_tokens_see_nothing_before_them():
    from gemmars_b200.weights import random_weights
    w = {k: v.double().numpy() for k, v in random_weights(DALERAX_C, 4).items()}
    toks = [3, 50, 7, 7, 90, 11]
    whole = plain.forward(DALERAX_C, w, toks)
    for n in (1, 2, 3):
        assert np.allclose(plain.forward(DALERAX_C, w, toks[:n]), whole[:n], atol=1e-12)     # causal throughout
    other = plain.forward(DALERAX_C, w, [4] + toks[1:])
    assert not np.allclose(other[-1], whole[-1])                    # the recurrent layer remembers the first token


def test_a_reader_of_another_layers_keys_differs_from_one_with_its_own():
    """The plain model's layer 3 of A reads layer 1's keys: changing layer 1's k matrix changes what
    layer 3 sees, and layer 3 has no k of its own to change."""
    from gemmars_b200.weights import random_weights
    w = {k: v.double().numpy() for k, v in random_weights(DALERAX_A, 2).items()}
    assert "l3.mix.k" not in w and "l3.mix.v" not in w
    toks = list(range(40, 70))
    _, layers = plain.forward(DALERAX_A, w, toks, return_layers=True)
    w2 = dict(w)
    w2["l1.mix.v"] = w["l1.mix.v"] * 1.5
    _, layers2 = plain.forward(DALERAX_A, w2, toks, return_layers=True)
    assert np.allclose(layers[0], layers2[0]) and not np.allclose(layers[1], layers2[1])
    # with layer 1's and layer 2's effect on the stream taken out, layer 3 still differs: it reads the values
    m = DALERAX_A["layers"][3]["mixer"]
    h = plain.offset_norm(layers[2], w["l3.norm1"], 1e-5)
    P = plain.sub(w, "l3.mix.")
    _, kv = plain.attention_mixer(plain.offset_norm(layers[0], w["l1.norm1"], 1e-5), plain.sub(w, "l1.mix."), DALERAX_A["layers"][1]["mixer"])
    a, _ = plain.attention_mixer(h, P, m, kv)
    b, _ = plain.attention_mixer(h, P, m, (kv[0], kv[1] * 1.5))
    assert not np.allclose(a, b)
