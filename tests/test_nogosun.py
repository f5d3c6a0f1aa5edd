"""Nogosun without a GPU: the configuration, the plan against the checkpoint layout, what the
layers ask of the cache, and the plain implementation's mechanisms against hand-worked numbers."""
import copy
import math

import numpy as np
import pytest

import plain_nogosun as plain
from tiny_configs import NOGOSUN_A, NOGOSUN_B, NOGOSUN_C


def test_configuration_reports_every_problem_at_once():
    from gemmars_b200.config.base import ConfigError
    from gemmars_b200.models.nogosun import NogosunConfig
    cfg = NogosunConfig.from_dict(NOGOSUN_A)
    assert cfg.vocab == 211 and cfg.embedding_scale == 3.0 and cfg.norm_eps == 1e-5 and len(cfg.layers) == 6
    assert NogosunConfig.from_dict(cfg.to_dict()) == cfg
    bad = copy.deepcopy(NOGOSUN_A)
    bad["layers"][1]["mixer"] = copy.deepcopy(bad["layers"][1]["mixer"])
    bad["layers"][1]["mixer"]["rot"]["dims"] = 34                   # more than dim
    bad["layers"][1]["mixer"]["vdim"] = 16                          # the values are the keys
    bad["layers"][2]["mixer"]["heads"] = 5                          # not a multiple of kv_heads
    bad["layers"][0]["type"] = "conv"
    del bad["embedding"]
    bad["layers"][3]["weights_of"] = 2                              # another kind of layer
    bad["layers"][4]["weights_of"] = 4                              # itself
    bad["layers"][5]["mlp"]["router"]["top"] = 4                    # of 3 experts
    bad["layers"][1]["mlp"]["kind"] = "dense"
    with pytest.raises(ConfigError) as e:
        NogosunConfig.from_dict(bad)
    text = str(e.value)
    for piece in ("rot.dims", "must equal dim", "5 heads", "unknown mixer 'conv'", "embedding.scale", "layers[3].weights_of",
                  "layers[4].weights_of", "top: 4 of 3", "unknown feed-forward 'dense'"):
        assert piece in text, piece
    bad = copy.deepcopy(NOGOSUN_B)
    bad["layers"][2]["mixer"] = copy.deepcopy(bad["layers"][2]["mixer"])
    bad["layers"][2]["mixer"]["right"]["tau"] = 0
    bad["layers"][2]["mixer"]["left"]["q_temp"]["every"] = 0
    del bad["layers"][2]["mixer"]["left_scale"]
    with pytest.raises(ConfigError) as e:
        NogosunConfig.from_dict(bad)
    for piece in ("right.tau", "q_temp.every", "left_scale"):
        assert piece in str(e.value), piece
    circle = copy.deepcopy(NOGOSUN_A)
    circle["layers"][1]["weights_of"] = 3                           # 1 -> 3 -> 1
    with pytest.raises(ConfigError) as e:
        NogosunConfig.from_dict(circle)
    assert "circle" in str(e.value)


def test_a_layer_may_run_the_tensors_of_a_later_layer():
    """The owner of shared tensors need not come first: here the first layer runs the last one's."""
    from gemmars_b200.config.registry import resolve_architecture
    from gemmars_b200.engine.model import DecoderModel
    from gemmars_b200.weights import random_weights
    raw = copy.deepcopy(NOGOSUN_C)
    raw["layers"].insert(0, dict(copy.deepcopy(raw["layers"][3]), weights_of=4))
    arch = resolve_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    model = DecoderModel(arch.build_plan(cfg, None), "float32", "cpu")
    assert [e.layer for e in model.plan.schedule] == [3, 0, 1, 2, 3] and len(model.blocks) == 4
    assert not any(name.startswith("l0.") for name in model.expected_tensors())
    w = {k: v.double().numpy() for k, v in random_weights(raw, 2).items()}
    toks = list(range(20))
    copies = dict(w)
    copies.update({"l0." + k[len("l4."):]: v for k, v in w.items() if k.startswith("l4.")})
    own = copy.deepcopy(raw)
    del own["layers"][0]["weights_of"]
    assert np.allclose(plain.forward(raw, w, toks), plain.forward(own, copies, toks), rtol=0, atol=1e-12)


@pytest.mark.parametrize("raw", [NOGOSUN_A, NOGOSUN_B, NOGOSUN_C], ids="ABC")
def test_plan_wants_exactly_the_checkpoint(raw):
    from gemmars_b200.config.registry import resolve_architecture
    from gemmars_b200.engine.model import DecoderModel
    arch = resolve_architecture(raw)
    cfg = arch.config_class.from_dict(raw)
    model = DecoderModel(arch.build_plan(cfg, None), "float32", "cpu")
    layout = {name: tuple(shape) for name, (shape, _) in arch.checkpoint_layout(cfg).items()}
    assert model.expected_tensors() == layout
    sharers = [i for i, layer in enumerate(raw["layers"]) if "weights_of" in layer]
    assert not any(name.startswith(f"l{i}.") for i in sharers for name in layout)
    # a layer that runs another layer's tensors is another entry of the schedule for the same block
    own = [i for i in range(len(raw["layers"])) if i not in sharers]
    assert len(model.blocks) == len(own) and len(model.plan.schedule) == len(raw["layers"])
    for i in sharers:
        assert model.plan.schedule[i].layer == own.index(raw["layers"][i]["weights_of"])
        assert model.plan.schedule[i].cache_of is None
    for i, layer in enumerate(raw["layers"]):
        if layer["mlp"] is None and i in own:
            assert f"l{i}.norm2" not in layout and f"l{i}.norm2" in model.plan.ignored_tensors


def test_the_inner_sizes_come_from_the_checkpoint():
    """config.json of a released model names no ranks: the rows of a1 and g1 give them."""
    from gemmars_b200.engine.model import build_model
    from gemmars_b200.weights import random_weights
    tensors = random_weights(NOGOSUN_C, 1)
    raw = copy.deepcopy(NOGOSUN_C)
    del raw["layers"][1]["mixer"]["decay_rank"], raw["layers"][1]["mixer"]["gate_rank"], raw["layers"][2]["mixer"]["right"]["rank"]
    model = build_model(raw_config=raw, tensors=tensors, dtype="float32", device="cpu", compile_kernels=False)
    delta, pair = model.blocks[1].mixer, model.blocks[2].mixer
    assert (delta.decay_rank, delta.gate_rank) == (2, 1) and pair.branches[1][1].rank == 3
    assert model.expected_tensors()["l1.mix.a2"] == (2 * 12, 2) and model.expected_tensors()["l2.mix.right.a2"] == (20, 3)


def test_what_the_layers_keep_per_sequence():
    from gemmars_b200 import kernels
    from gemmars_b200.cache.pool import KVNeed, StateNeed
    from gemmars_b200.engine.model import build_model
    from gemmars_b200.weights import random_weights
    model = build_model(raw_config=NOGOSUN_A, tensors=random_weights(NOGOSUN_A, 1), dtype="float32", device="cpu",
                        compile_kernels=False)
    needs = dict(model.cache_needs())
    assert sorted(needs) == [0, 1, 2, 3, 4, 5]               # every run of a layer keeps its own, shared tensors or not
    # the two-branch layer: keys of 16 with values of 24 for every position, and a matrix a head
    assert needs[0] == [KVNeed(2, 16, None, 24), StateNeed((3, kernels.recurrent_state_floats(8, 24)))] == needs[4]
    # kept first tokens: every page stays, the window is the kernels' mask; values as wide as keys
    assert needs[1] == [KVNeed(2, 32, None, 32)] == needs[3]
    # the delta rule: the filter's last three inputs of q | k | v, and a matrix a head
    assert needs[2] == [StateNeed((3, 2 * 2 * 24 + 4 * 16)), StateNeed((4, kernels.recurrent_state_floats(24, 16)))]
    model = build_model(raw_config=NOGOSUN_C, tensors=random_weights(NOGOSUN_C, 1), dtype="float32", device="cpu",
                        compile_kernels=False)
    needs = dict(model.cache_needs())
    assert needs[0] == [KVNeed(2, 20, None, 20)]             # no mask: every position
    assert needs[3] == [KVNeed(1, 12, 17, 12)]               # a window with nothing kept: a ring of pages
    assert needs[1][0] == StateNeed((0, 2 * 12 + 2 * 20))    # a filter of one tap remembers nothing


# ------------------------------------------------------------------ the mechanisms, by hand

def test_frequencies_blend_along_the_index():
    # dims 8, base 16: f = 16^(-i/4) = 1, 1/2, 1/4, 1/8.  d(t) = 8 ln(original / (2 pi t)) / (2 ln 16)
    scaling = {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 0.5}
    d_fast = 8 * math.log(64 / (2 * math.pi * 4.0)) / (2 * math.log(16))
    d_slow = 8 * math.log(64 / (2 * math.pi * 0.5)) / (2 * math.log(16))
    assert 1 < d_fast < 2 and 4 < d_slow < 5
    f, mag = plain.ramp_frequencies(16.0, 8, scaling)
    # lo = 1, hi = 5: ramp = (i - 1) / 4 = 0, 0, 1/4, 1/2
    assert np.allclose(f, [1.0, 0.5, 0.25 * (0.25 / 4 + 0.75), 0.125 * (0.5 / 4 + 0.5)])
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    plain_f, one = plain.ramp_frequencies(16.0, 8, None)
    assert np.allclose(plain_f, [1.0, 0.5, 0.25, 0.125]) and one == 1.0
    # hi is held below dims, lo above zero
    f, _ = plain.ramp_frequencies(16.0, 8, {"factor": 2.0, "original": 1e9, "fast": 1e12, "slow": 1e-12})
    assert np.allclose(f, plain_f * (1 - np.arange(4) / 7 / 2))
    from gemmars_b200.parts.base import build_part
    from gemmars_b200.parts.plan import PartSpec
    part = build_part("position", PartSpec("rotary", {"head_dim": 8, "rotary_dim": 8, "theta": 16.0, "scaling": scaling}), "float32")
    assert np.allclose(part._inv_freq_host.numpy(), plain.ramp_frequencies(16.0, 8, scaling)[0], rtol=1e-7)
    assert part.magnitude == pytest.approx(mag)


def test_rotation_turns_pairs_half_a_head_apart_and_stretches_them():
    x = np.zeros((2, 1, 6))
    x[:, 0] = [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    y = plain.rotate_half(x, [0, 1], np.array([math.pi / 2, math.pi]), magnitude=2.0)
    assert np.allclose(y[0, 0], [2.0, 4.0, 6.0, 8.0, 5.0, 6.0])                    # position 0: only the magnitude
    assert np.allclose(y[1, 0], [-6.0, -4.0, 2.0, -8.0, 5.0, 6.0])                 # (1, 3) by 90 degrees, (2, 4) by 180


def test_window_kept_tokens_and_the_one_in_the_denominator():
    assert [j for j in range(10) if plain.visible(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    assert [j for j in range(10) if plain.visible(3, j, 3, 2)] == [0, 1, 2, 3]
    assert [j for j in range(5) if plain.visible(4, j, None, 0)] == [0, 1, 2, 3, 4]
    q = np.zeros((3, 1, 2))
    k = np.zeros((3, 1, 2))
    v = np.array([[[1.0]], [[2.0]], [[4.0]]])
    # equal scores of zero: plain softmax averages the visible values; with one more in the
    # denominator each of n keys weighs 1 / (n + 1)
    assert np.allclose(plain.masked_attention(q, k, v, 1.0)[:, 0, 0], [1.0, 1.5, 7.0 / 3.0])
    assert np.allclose(plain.masked_attention(q, k, v, 1.0, plus_one=True)[:, 0, 0], [0.5, 1.0, 7.0 / 4.0])
    assert np.allclose(plain.masked_attention(q, k, v, 1.0, size=2)[:, 0, 0], [1.0, 1.5, 3.0])
    assert np.allclose(plain.masked_attention(q, k, v, 1.0, size=1, keep_first=1)[:, 0, 0], [1.0, 1.5, 2.5])
    # a cap holds a large score at the cap: exp(cap) against the one in the denominator
    q[:] = 100.0
    k[:] = 1.0
    out = plain.masked_attention(q[:1], k[:1], v[:1], 1.0, cap=2.0, plus_one=True)[0, 0, 0]
    assert out == pytest.approx(math.exp(2.0 * math.tanh(100.0)) / (1.0 + math.exp(2.0 * math.tanh(100.0))))


def test_query_temperature_steps_with_the_position():
    t = plain.query_temperature(9, 0.5, 4)
    assert np.allclose(t[:3], 1.0) and np.allclose(t[3:7], 1.0 + 0.5 * math.log(2.0)) and np.allclose(t[7:], 1.0 + 0.5 * math.log(3.0))


def test_delta_rule_two_tokens_by_hand():
    # one head, dim 2, vdim 1
    q = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    k = np.array([[[1.0, 0.0]], [[1.0, 1.0]]])
    v = np.array([[[2.0]], [[3.0]]])
    beta = np.array([[0.5], [1.0]])
    g = np.array([[[1.0, 1.0]], [[0.5, 0.25]]])
    o, S = plain.channel_delta_scan(q, k, v, beta, g)
    # token 0: S = 0; u = 0.5 * 2 = 1; S = [[1], [0]]; o = 1
    # token 1: S <- [[0.5], [0]]; u = 3 - 0.5 = 2.5; S = [[3.0], [2.5]]; o = S^T q = 2.5
    assert np.allclose(o[:, 0, 0], [1.0, 2.5]) and np.allclose(S[0, :, 0], [3.0, 2.5])
    # carried from the state it left
    o2, _ = plain.channel_delta_scan(q[1:], k[1:], v[1:], beta[1:], g[1:], state=plain.channel_delta_scan(q[:1], k[:1], v[:1], beta[:1], g[:1])[1])
    assert np.allclose(o2[0], o[1])


def test_gated_linear_attention_reads_after_it_writes():
    q = np.array([[[1.0, 1.0]], [[1.0, 0.0]]])
    k = np.array([[[1.0, 2.0]], [[0.0, 1.0]]])
    v = np.array([[[1.0, 10.0]], [[2.0, 20.0]]])
    alpha = np.array([[[0.5, 0.5]], [[0.5, 0.1]]])
    o, S = plain.decayed_outer_scan(q, k, v, alpha)
    # token 0: S = k0 v0^T = [[1, 10], [2, 20]]; o = S^T q = [3, 30]: the token's own write is read
    # token 1: S = diag(0.5, 0.1) S + k1 v1^T = [[0.5, 5], [0.2 + 2, 2 + 20]]; o = row 0
    assert np.allclose(o[0, 0], [3.0, 30.0]) and np.allclose(o[1, 0], [0.5, 5.0]) and np.allclose(S[0], [[0.5, 5.0], [2.2, 22.0]])


def test_short_filter_and_unit_vectors():
    x = np.array([[1.0], [2.0], [3.0]])
    assert np.allclose(plain.short_filter(x, np.array([[10.0, 1.0]]))[:, 0], [1.0, 12.0, 23.0])        # the last tap is the token's own
    assert np.allclose(plain.short_filter(x, np.array([[2.0]]))[:, 0], [2.0, 4.0, 6.0])
    assert np.allclose(plain.unit(np.array([3.0, 4.0]), 0.0), [0.6, 0.8])
    assert plain.unit(np.zeros(3), 1e-6).tolist() == [0.0, 0.0, 0.0]


def test_routing_keeps_the_shares_of_the_softmax_over_all():
    z = np.array([0.0, math.log(2.0), math.log(4.0), 0.0])          # softmax: 1/8, 2/8, 4/8, 1/8
    chosen, weights = plain.route_all(z, 2)
    assert chosen == [2, 1] and np.allclose(weights, [0.5, 0.25])
    chosen, _ = plain.route_all(z, 3)
    assert chosen == [2, 1, 0]                                       # the lower index wins a tie
    h = np.array([[1.0, 0.0]])
    P = {"router": np.array([[0.0, 0.0], [math.log(3.0), 0.0]]),
         "e0.up": np.array([[1.0, 0.0]]), "e0.down": np.array([[1.0], [0.0]]),
         "e1.up": np.array([[2.0, 0.0]]), "e1.down": np.array([[0.0], [1.0]])}
    out = plain.routed_ffn(h, P, {"router": {"experts": 2, "top": 1}})
    gelu2 = 0.5 * 2.0 * (1.0 + math.erf(2.0 / math.sqrt(2.0)))
    assert np.allclose(out, [[0.0, 0.75 * gelu2]])                  # expert 1 alone, at its share 3/4


def test_a_layer_that_runs_another_layers_tensors_has_a_state_of_its_own():
    """The same tensors twice in a row are not the same as once with the stream doubled: the second
    run sees another input and keeps another state.  Here: the model with the shared layers against
    the same model with copies of the tensors under the sharers' own names."""
    from gemmars_b200.weights import random_weights
    w = {k: v.double().numpy() for k, v in random_weights(NOGOSUN_A, 3).items()}
    toks = list(np.random.default_rng(1).integers(0, 211, 30))
    shared = plain.forward(NOGOSUN_A, w, toks)
    raw = copy.deepcopy(NOGOSUN_A)
    copies = dict(w)
    for i, layer in enumerate(raw["layers"]):
        if "weights_of" in layer:
            j = layer.pop("weights_of")
            copies.update({f"l{i}." + k[len(f"l{j}."):]: v for k, v in w.items() if k.startswith(f"l{j}.")})
    assert np.allclose(plain.forward(raw, copies, toks), shared, rtol=0, atol=1e-12)
