"""Nogosun on the GPU against the plain implementation: each mechanism's kernels alone, then whole
models through the trace runner, the step function and the generation entry point, with prompts
cut in every way, batches of unequal requests, reused slots and pages, keys that matter far back,
at page borders, on both sides of a window's edge and among the kept first tokens, long decoding
and the first tokens of a sequence."""
import json
import os

import numpy as np
import pytest
import torch

import plain_nogosun as plain
from replay_util import Trace, run_trace
from tiny_configs import NOGOSUN_A, NOGOSUN_B, NOGOSUN_C, _nogosun_attention, _nogosun_delta, _nogosun_moe, _nogosun_pair

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL_F32 = 3e-5
# bfloat16 engine against the float64 plain implementation, as a fraction of the largest logit
TOL_BF16 = 3e-2
PAGE = 64


def _dt(name):
    return torch.float32 if name == "float32" else torch.bfloat16


def _rand(rng, shape, dtype=torch.float32, scale=1.0, shift=0.0):
    """Random values that ``dtype`` holds exactly, as (device tensor, float64 numpy)."""
    t = torch.from_numpy(rng.standard_normal(shape) * scale + shift).to(dtype)
    return t.to(DEV), t.double().numpy()


def _i32(a):
    return torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)


def _packed(lens, slots, starts=None):
    """Index tensors of a packed step: (cu_seqlens, tok_seq, seq_slot, tok_pos)."""
    starts = starts or [0] * len(lens)
    cu = np.concatenate([[0], np.cumsum(lens)])
    seq = np.repeat(np.arange(len(lens)), lens)
    pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, lens)])
    return _i32(cu), _i32(seq), _i32(slots), _i32(pos)


def _cuts(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[min(i, len(sizes) - 1)], total - at)
        out.append((at, at + n))
        at, i = at + n, i + 1
    return out


def _steps(lens, sizes):
    """Walks sequences of ``lens`` tokens side by side in portions of ``sizes``: yields, step by
    step, [(sequence, lo, hi)] of the sequences that still have tokens."""
    cuts = [_cuts(n, sizes) for n in lens]
    for step in range(max(len(c) for c in cuts)):
        yield [(i, *cuts[i][step]) for i in range(len(lens)) if step < len(cuts[i])]


# ------------------------------------------------------------------ mechanisms alone

@pytest.mark.parametrize("mode", ["rate", "sigmoid_root", "plain"])
@pytest.mark.parametrize("w_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tokens,groups,group,rank", [(1, 3, 32, 16), (37, 4, 18, 8), (300, 1, 40, 5), (9, 25, 40, 1), (21, 2, 65, 300)])
def test_second_half_of_a_two_matrix_projection(mode, w_dtype, tokens, groups, group, rank):
    """z is a slice of columns of a wider tensor, as the parts hand it over."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(rank + tokens)
    channels = groups * group
    wide, widen = _rand(rng, (tokens, rank + 7), scale=1.5)
    z, zn = wide[:, 3:3 + rank], widen[:, 3:3 + rank]
    w2, w2n = _rand(rng, (channels, rank), _dt(w_dtype), scale=0.8 * min(1.0, 8.0 / rank ** 0.5))
    base, bn = _rand(rng, (channels,), scale=1.0)
    rate, rn = _rand(rng, (groups,), scale=0.5)
    a = zn @ w2n.T + bn
    if mode == "rate":
        got = kernels.lowrank_map(z, w2, base, "rate", rate=rate, rate_group=group)
        want = np.exp(-np.repeat(np.exp(rn), group)[None, :] * plain.softplus(a))
    elif mode == "sigmoid_root":
        got = kernels.lowrank_map(z, w2, base, "sigmoid_root", tau=7.0)
        want = plain.sigmoid(a) ** (1.0 / 7.0)
    else:
        got = kernels.lowrank_map(z, w2, None, "plain")
        want = a - bn
    got = got.double().cpu().numpy()
    assert got.shape == want.shape and np.abs(got - want).max() < 3e-6 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,n", [(1, 72), (9, 52), (8, 4096), (600, 320), (513, 1024), (700, 5120), (520, 6000), (3, 6001)])
def test_two_norms_of_the_same_rows_in_one_pass(dtype, rows, n):
    """Every form of the norm kernel (few rows, many rows held in registers, rows too wide for that,
    widths that are no multiple of four): the pair gives the bits of two norms run one after the other."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(rows + n)
    x, xn = _rand(rng, (rows, n), scale=3.0)
    w1, w1n = _rand(rng, (n,), shift=1.0, scale=0.2)
    w2, w2n = _rand(rng, (n,), shift=-0.5, scale=0.7)
    outs = [torch.empty((rows, n), dtype=_dt(dtype), device=DEV) for _ in range(4)]
    kernels.rmsnorm(x, w1, outs[0], 1e-5)
    kernels.rmsnorm(x, w2, outs[1], 1e-5)
    kernels.rmsnorm(x, w1, outs[2], 1e-5, second=(w2, outs[3]))
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])
    want = plain.rms_norm(xn, w2n, 1e-5)
    assert np.abs(outs[3].double().cpu().numpy() - want).max() < (1e-5 if dtype == "float32" else 1e-2) * np.abs(want).max()


def _scan_case(rng, lens, heads, groups, dim, vdim, planted):
    """Random q | k | v rows (one tensor), beta logits and decays per sequence.  With ``planted``, in
    the longest sequence one early key is made loud on channels whose decay is held at one, with a
    distinctive v, every later key is kept off those channels, and a query hundreds of tokens later
    points at it."""
    out = []
    qk = groups * dim
    for n in lens:
        xn = rng.standard_normal((n, 2 * qk + heads * vdim + 3)) * 0.5
        bn = rng.standard_normal((n, heads + 2))
        gn = np.exp(-np.exp(rng.standard_normal((n, heads * dim + 1)) * 1.5 - 1.5))
        if planted and n > 200:
            gn[:, :4] = 1.0
            xn[5, qk:qk + 4] = 4.0
            xn[6:, qk:qk + 4] = 0.0
            xn[250, :4] = 3.0
            xn[250, 4:dim] *= 0.01
            xn[5, 2 * qk:2 * qk + vdim] = np.arange(vdim) - 3.0
            bn[5, 0] = 6.0
        out.append((torch.from_numpy(xn).float().to(DEV), torch.from_numpy(bn).float().to(DEV),
                    torch.from_numpy(gn).float().to(DEV)))
    return out


@pytest.mark.parametrize("heads,groups,dim,vdim", [(3, 3, 24, 16), (4, 2, 40, 8), (2, 1, 64, 70), (2, 2, 128, 32), (4, 1, 16, 33),
                                                   (1, 1, 200, 24), (2, 2, 33, 40)])
def test_delta_rule_with_a_decay_per_channel_alone(heads, groups, dim, vdim):
    """Whole sequences against portions of 1, 2, 5 and 33 tokens and token by token, in slots out of
    order, twice over in slots that were cleared: the state carries from step to step, and the loud
    key of token 5 is found by the query at token 250 however the walk was cut."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(heads * 1000 + dim)
    lens, slots = [260, 2, 40], [1, 3, 0]
    qk, hv = groups * dim, heads * vdim
    data = _scan_case(rng, lens, heads, groups, dim, vdim, planted=True)
    want = []
    for (x, b, g), n in zip(data, lens):
        xn, bn, gn = x.double().cpu().numpy(), b.double().cpu().numpy(), g.double().cpu().numpy()
        rep = heads // groups
        q = np.repeat(plain.unit(xn[:, :qk].reshape(n, groups, dim), 1e-6) * dim ** -0.5, rep, axis=1)
        k = np.repeat(plain.unit(xn[:, qk:2 * qk].reshape(n, groups, dim), 1e-6), rep, axis=1)
        o, _ = plain.channel_delta_scan(q, k, xn[:, 2 * qk:2 * qk + hv].reshape(n, heads, vdim), plain.sigmoid(bn[:, :heads]),
                                        gn[:, :heads * dim].reshape(n, heads, dim))
        want.append(o.reshape(n, hv))
    # the planted write is what the late query reads: without it the read-out there is far smaller
    assert np.abs(want[0][250, :vdim]).max() > 4 * np.abs(want[0][249, :vdim]).max()
    state = torch.zeros((5, heads, kernels.recurrent_state_floats(dim, vdim)), dtype=torch.float32, device=DEV)
    for sizes in ([1000], [1, 2, 5, 33], [1]):
        for s in slots:
            state[s] = 0.0
        got = [np.zeros((n, hv)) for n in lens]
        for live in _steps(lens, sizes):
            x = torch.cat([data[i][0][lo:hi] for i, lo, hi in live])
            b = torch.cat([data[i][1][lo:hi] for i, lo, hi in live])
            g = torch.cat([data[i][2][lo:hi] for i, lo, hi in live])
            cu, _, slot, _ = _packed([hi - lo for _, lo, hi in live], [slots[i] for i, _, _ in live])
            y = torch.empty((x.shape[0], hv), dtype=torch.float32, device=DEV)
            kernels.channel_delta_rule(x[:, :qk], x[:, qk:2 * qk], x[:, 2 * qk:2 * qk + hv], b[:, :heads], g[:, :heads * dim], state,
                                       cu, slot, y, heads, groups, dim, vdim, float(dim) ** -0.5)
            y = y.double().cpu().numpy()
            at = 0
            for i, lo, hi in live:
                got[i][lo:hi] = y[at:at + hi - lo]
                at += hi - lo
        for i in range(3):
            assert np.abs(got[i] - want[i]).max() < 2e-5 * max(1.0, np.abs(want[i]).max()), (sizes, i)
        assert not state[2].any() and not state[4].any()


@pytest.mark.parametrize("heads,dim,vdim", [(3, 24, 16), (1, 40, 64), (2, 64, 64), (2, 128, 48), (4, 16, 33), (1, 200, 8), (2, 33, 20)])
def test_gated_linear_attention_alone(heads, dim, vdim):
    """The read-out follows the write: y_t sees k_t v_t^T.  Whole, in portions and token by token."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(heads * 100 + dim)
    lens, slots = [260, 1, 40], [2, 0, 3]
    hd, hv = heads * dim, heads * vdim
    data, want = [], []
    for n in lens:
        xn = rng.standard_normal((n, 2 * hd + hv + 5)) * 0.5
        an = np.exp(-np.exp(rng.standard_normal((n, hd)) * 1.5 - 1.5))
        if n > 200:
            an[:, :4] = 1.0                                        # the first channels of head 0 forget nothing
            xn[5, hd:hd + 4] = 30.0                                # a loud key at token 5 ...
            xn[6:, hd:hd + 4] *= 0.01
            xn[250, :4] = 2.0                                      # ... that the query at 250 asks for
            xn[250, 4:dim] *= 0.01
            xn[5, 2 * hd:2 * hd + vdim] = np.arange(vdim) - 3.0
        x, a = torch.from_numpy(xn).float().to(DEV), torch.from_numpy(an).float().to(DEV)
        xn, an = x.double().cpu().numpy(), a.double().cpu().numpy()
        o, _ = plain.decayed_outer_scan(xn[:, :hd].reshape(n, heads, dim) * dim ** -0.5, xn[:, hd:2 * hd].reshape(n, heads, dim),
                                        xn[:, 2 * hd:2 * hd + hv].reshape(n, heads, vdim), an.reshape(n, heads, dim))
        data.append((x, a))
        want.append(o.reshape(n, hv))
    assert np.abs(want[0][250, :vdim]).max() > 4 * np.abs(want[0][249, :vdim]).max()
    state = torch.zeros((5, heads, kernels.recurrent_state_floats(dim, vdim)), dtype=torch.float32, device=DEV)
    for sizes in ([1000], [1, 2, 5, 33], [1]):
        for s in slots:
            state[s] = 0.0
        got = [np.zeros((n, hv)) for n in lens]
        for live in _steps(lens, sizes):
            x = torch.cat([data[i][0][lo:hi] for i, lo, hi in live])
            a = torch.cat([data[i][1][lo:hi] for i, lo, hi in live])
            cu, _, slot, _ = _packed([hi - lo for _, lo, hi in live], [slots[i] for i, _, _ in live])
            y = torch.empty((x.shape[0], hv), dtype=torch.float32, device=DEV)
            kernels.wkv_scan(x[:, :hd], x[:, hd:2 * hd], a, x[:, 2 * hd:2 * hd + hv], None, state, cu, slot, y, heads, dim, vdim,
                             out_scale=float(dim) ** -0.5)
            y = y.double().cpu().numpy()
            at = 0
            for i, lo, hi in live:
                got[i][lo:hi] = y[at:at + hi - lo]
                at += hi - lo
        for i in range(3):
            assert np.abs(got[i] - want[i]).max() < 2e-5 * max(1.0, np.abs(want[i]).max()), (sizes, i)
        assert not state[1].any() and not state[4].any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,groups,dim,rot,normed,temper,own_values", [
    (4, 2, 32, 8, False, None, False), (3, 1, 20, 0, True, (0.7, 3), True), (2, 2, 96, 96, True, (0.5, 1), True),
    (1, 1, 12, 4, False, (2.0, 5), False), (8, 4, 64, 16, True, None, True)])
def test_rows_into_queries_and_pages(dtype, heads, groups, dim, rot, normed, temper, own_values):
    """The kernel between the projection and the attention: norm of q and k heads, rotation with a
    magnitude, the query's factor by position, and values that are the keys as projected (or columns
    of their own), for sequences that start at positions 0, 61 (a page border inside the step) and 200."""
    from gemmars_b200 import kernels
    rng = np.random.default_rng(heads * 10 + dim)
    vdim = dim + 8 if own_values else dim
    lens, starts, slots = [7, 9, 1], [0, 61, 200], [1, 0, 2]
    cu, seq, slot, pos = _packed(lens, slots, starts)
    t = sum(lens)
    cols = (heads + groups) * dim + (groups * vdim if own_values else 0)
    u, un = _rand(rng, (t, cols + 4), _dt(dtype))
    qw, qwn = _rand(rng, (dim,), shift=1.0, scale=0.2)
    kw, kwn = _rand(rng, (dim,), shift=1.0, scale=0.2)
    freq, mag = plain.ramp_frequencies(300.0, rot, {"factor": 4.0, "original": 16, "fast": 2.0, "slow": 0.5}) if rot else (np.zeros(0), 1.0)
    inv = torch.tensor(freq, dtype=torch.float32, device=DEV) if rot else None
    table = torch.arange(3 * 4, dtype=torch.int32, device=DEV).reshape(3, 4)
    kc = torch.zeros((12, groups, PAGE, dim), dtype=_dt(dtype), device=DEV)
    vc = torch.zeros((12, groups, vdim, PAGE), dtype=_dt(dtype), device=DEV)
    q = torch.empty((t, heads * dim), dtype=_dt(dtype), device=DEV)
    kernels.filter_rope_cache(u[:, 2:2 + cols], None, None, inv, rot, pos, seq, slot, cu, table, PAGE, q, kc, vc, heads, groups, dim,
                              vdim, q_norm=qw if normed else None, k_norm=kw if normed else None, norm_eps=1e-5,
                              rot_magnitude=mag, q_temper=temper, values_are_keys=not own_values)
    positions = pos.cpu().numpy()
    qn = un[:, 2:2 + heads * dim].reshape(t, heads, dim)
    kn = un[:, 2 + heads * dim:2 + (heads + groups) * dim].reshape(t, groups, dim)
    vn = un[:, 2 + (heads + groups) * dim:2 + cols].reshape(t, groups, vdim) if own_values else kn.copy()
    if normed:
        qn, kn = plain.rms_norm(qn, qwn, 1e-5), plain.rms_norm(kn, kwn, 1e-5)
    freq32 = np.asarray(freq, dtype=np.float32).astype(np.float64)
    qn, kn = plain.rotate_half(qn, positions, freq32, mag), plain.rotate_half(kn, positions, freq32, mag)
    if temper:
        qn = qn * np.array([1.0 + temper[0] * np.log((p + 1) // temper[1] + 1) for p in positions])[:, None, None]
    tol = 4e-5 if dtype == "float32" else 1.5e-2
    assert np.abs(q.double().cpu().numpy().reshape(t, heads, dim) - qn).max() < tol * np.abs(qn).max()
    for i in range(t):
        b = int(seq[i])
        page = int(table[slots[b], positions[i] // PAGE])
        off = positions[i] % PAGE
        assert np.abs(kc[page, :, off].double().cpu().numpy() - kn[i]).max() < tol * np.abs(kn).max()
        assert np.abs(vc[page, :, :, off].double().cpu().numpy() - vn[i]).max() < tol * np.abs(vn).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("t,width,experts,top,ff", [(1, 64, 4, 2, 32), (9, 52, 3, 3, 20), (15, 72, 6, 1, 40), (40, 64, 5, 2, 48),
                                                    (255, 128, 16, 4, 64), (300, 128, 9, 3, 64), (700, 64, 4, 4, 32)])
def test_experts_without_gates(dtype, t, width, experts, top, ff):
    """Token-major (fewer than 16 tokens, and float32), grouped (16 to 255) and on the tcgen05 product
    (256 and more): the exact GELU, the weights from the softmax over all experts."""
    from gemmars_b200.parts.base import build_part
    from gemmars_b200.parts.plan import PartSpec
    rng = np.random.default_rng(t + experts)
    dt = _dt(dtype)
    names, w, wn = {}, {}, {}

    def add(name, shape, scale):
        names[name] = name
        w[name], wn[name] = _rand(rng, shape, torch.bfloat16, scale=scale)

    add("router", (experts, width), 0.4)
    for e in range(experts):
        add(f"e{e}.up", (ff, width), 0.25)
        add(f"e{e}.down", (width, ff), 0.25)
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    part = build_part("ffn", PartSpec("moe", {"hidden_size": width, "experts": experts, "top": top, "ff": ff, "limit": None,
                                              "router_bias": False, "gated": False, "routing": "softmax_all", "shared": None},
                                      names), dtype)
    part.load({k: v.to(dt) for k, v in w.items()})
    h, hn = _rand(rng, (t, width), dt)
    res, resn = _rand(rng, (t, width), torch.float32)
    part.forward(type("Ctx", (), dict(host=None))(), h, res)
    want = resn + plain.routed_ffn(hn, wn, mlp)
    assert np.abs(want - resn).max() > 0.05          # the weights are not renormalized: the sum is far from nothing
    # a token whose last chosen and first unchosen logits are closer than rounding may go either way
    z = np.sort(hn @ wn["router"].T, axis=1)[:, ::-1]
    sure = np.ones(t, bool) if top == experts else (z[:, top - 1] - z[:, top]) > (1e-4 if dtype == "float32" else 0.05)
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    assert sure.mean() > 0.7
    assert np.abs(res.double().cpu().numpy() - want)[sure].max() <= tol * np.abs(want).max()


# ------------------------------------------------------------------ whole models

def _sharp_folder(tmp_path_factory, raw, seed, factor):
    """Random weights whose attention query and key matrices are scaled by ``factor`` (and the q/k
    norms' weights of the tempered attention): scores grow with its square, the softmax picks single
    keys (or the one added to its denominator) instead of averaging, and a wrong key, a window that
    is off by one, a missing sink, a wrong page or slot shows in the logits.  The recurrent mixers'
    keys are scaled too, so that single writes stand out in their states."""
    from gemmars_b200.weights import random_weights, write_safetensors
    tensors = random_weights(raw, seed=seed)
    for name in tensors:
        attention = name.endswith((".mix.q", ".mix.k")) and name[:-1] + "q.b" in tensors
        if attention or name.endswith((".left.q.norm", ".left.k.norm")):
            tensors[name] = (tensors[name].float() * factor).bfloat16()
        elif name.endswith((".right.k", ".right.q")):
            tensors[name] = (tensors[name].float() * 3.0).bfloat16()
    d = str(tmp_path_factory.mktemp("nogosun"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(raw, f)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


def _within(errors, tol, dtype, what, share=0.04):
    """float32: every position within ``tol``.  bfloat16: rounding the router's input moves a token
    whose candidate experts have nearly equal logits to another expert now and then, which changes
    that position's logits (and through the recurrent state, a few after it) by more than rounding;
    up to ``share`` of the positions (at least one) may be over, and the rest must be within ``tol``."""
    errors = np.asarray(errors)
    over = int((errors > tol).sum())
    allowed = 0 if dtype == "float32" else max(1, int(share * errors.size))
    assert over <= allowed, f"{what}: {over} of {errors.size} positions are over {tol:.2e} (worst {errors.max():.2e})"


# A: a window of 20 beside 3 kept tokens, a temperature step every 7; B: a window of 130 beside 70 kept, and 64
REQUESTS = {"A": (NOGOSUN_A, [15, 21, 9, 70, 44, 131]), "B": (NOGOSUN_B, [17, 33, 3, 80, 150, 300])}
GROUPS = [[0, 1, 2], [3, 4, 5]]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (raw, lengths) in REQUESTS.items():
        folder = _sharp_folder(tmp_path_factory, raw, seed=31 + len(name), factor=9.0 if name == "A" else 6.0)
        cfg, w = plain.load_folder(folder)
        rng = np.random.default_rng(lengths[0])
        reqs = [rng.integers(0, raw["vocab"], n).tolist() for n in lengths]
        out[name] = (folder, cfg, w, reqs, [plain.forward(cfg, w, r) for r in reqs])
    return out


def test_the_test_models_show_a_fault(models):
    """The scaled queries and keys do what they are for: in the plain model, a window one token
    narrower, one kept token fewer, the softmax without the one in its denominator or the queries
    without their temperature move the logits by far more than any tolerance."""
    folder, cfg, w, reqs, ref = models["A"]
    toks = reqs[5]
    scale = np.abs(ref[5]).max()

    def changed(edit):
        other = json.loads(json.dumps(cfg))
        edit(other["layers"])
        return plain.forward(other, w, toks)

    def narrower(layers):
        for i in (1, 3):
            layers[i]["mixer"]["mask"]["size"] -= 1

    def fewer_kept(layers):
        for i in (1, 3):
            layers[i]["mixer"]["mask"]["keep_first"] -= 1

    def no_temperature(layers):
        for i in (0, 4):
            layers[i]["mixer"]["left"]["q_temp"] = None

    runs = [changed(narrower), changed(fewer_kept), changed(no_temperature)]
    saved = plain.masked_attention
    try:
        plain.masked_attention = lambda *a, **k: saved(*a, **{**k, "plus_one": False})
        runs.append(plain.forward(cfg, w, toks))
    finally:
        plain.masked_attention = saved
    for other in runs:
        moved = np.abs(other - ref[5]).max(axis=1)
        assert moved.max() > 3 * TOL_BF16 * scale and (moved[40:] > 100 * TOL_F32 * scale).mean() > 0.3


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_the_plain_implementation(name, dtype, models, tmp_path):
    """Through bin/trace_run: each request whole, with its last 40 tokens one by one (the window of A
    passes over decoded tokens), and in two batches of unequal requests that follow one another in a
    cache sized to the peak, so that the second batch lives in the slots and pages the first gave back."""
    folder, cfg, w, reqs, ref = models[name]
    tr = Trace()
    tr.whole("w", reqs)
    tr.tail("t", reqs, n_tail=40)
    prompt_lens = [max(1, len(r) - 8 - 3 * i) for i, r in enumerate(reqs)]
    prompt_lens[2] = len(reqs[2])
    prompt_lens[1] = 1
    tr.batches("b", reqs, GROUPS, prompt_lens)
    got = run_trace(tr, folder, dtype, str(tmp_path / "out"))
    scale = max(float(np.abs(r).max()) for r in ref)
    tol = (TOL_F32 if dtype == "float32" else TOL_BF16) * scale
    for tag in "wtb":
        _within([np.abs(got[(f"{tag}{i}", p)] - r[p]).max() for i, r in enumerate(ref) for p in range(len(r))], tol, dtype,
                f"cutting {tag!r}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_residual_after_every_layer(dtype, models):
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, cfg, w, reqs, _ = models["A"]
    toks = reqs[3]
    _, want = plain.forward(cfg, w, toks, return_layers=True)
    model = build_model(folder, dtype=dtype)
    assert len(model.blocks) == 4 and len(model.plan.schedule) == 6          # two layers run another layer's tensors
    seen = []
    for block in model.blocks:
        def run(ctx, x, caches, writes_cache=True, _inner=block.forward):
            _inner(ctx, x, caches, writes_cache=writes_cache)
            assert x.dtype == torch.float32                      # the residual stream is 32-bit in both modes
            seen.append(x.double().cpu().numpy())
        block.forward = run
    runner = Runner(model, max_tokens=256, max_batch=1, use_graphs=False)
    runner.step([StepItem(runner.open(), toks, [])])
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        tol = (1e-5 if dtype == "float32" else 2e-2) * np.abs(b).max()
        # the stream itself, not logits: a token that went to another expert early stays off through every layer
        _within(np.abs(a - b).max(axis=1), tol, dtype, f"layer {i}", share=0.08)


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_long_decoding_and_reused_slots(name, dtype, models):
    """One runner, a cache of eight pages.  A prompt in portions of 2, 3, 64, 1, 65 and the rest;
    another from its first token one by one for 300 steps, across four page borders and past every
    window and the kept tokens, beside a neighbour that comes and goes; then the same again in the
    slots and pages given back: in float32 to the last bit."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder, cfg, w, reqs, ref = models[name]
    model = build_model(folder, dtype=dtype)
    runner = Runner(model, max_tokens=8 * PAGE, max_batch=3)
    rng = np.random.default_rng(8)
    long_toks = rng.integers(0, cfg["vocab"], 300).tolist()
    long_ref = plain.forward(cfg, w, long_toks)
    scale = float(np.abs(long_ref).max())
    tol = (TOL_F32 if dtype == "float32" else TOL_BF16) * scale
    first_round = None
    for round_ in range(2):
        got = {}
        a = runner.open()
        at = 0
        for n in (2, 3, 64, 1, 65, 15):
            part = reqs[4][at:at + n]
            if not part:
                break
            got.update({("a", at + i): r for i, r in enumerate(runner.step([StepItem(a, part, range(len(part)))]).cpu().numpy())})
            at += len(part)
        assert at == len(reqs[4])
        runner.close(a)
        b = runner.open()
        c = None
        for p, tok in enumerate(long_toks):
            items = [StepItem(b, [tok], [0])]
            if p == 20:
                c = runner.open()
                items.append(StepItem(c, reqs[0], range(len(reqs[0]))))     # a prompt beside a decoded token
            elif c is not None and p < 20 + 30:
                items.append(StepItem(c, [reqs[1][(p - 21) % len(reqs[1])]], [0]))
            out = runner.step(items).cpu().numpy()
            got[("b", p)] = out[0]
            if p == 20:
                got.update({("c", i): r for i, r in enumerate(out[1:])})
            if p == 49:
                runner.close(c)
                c = None
        runner.close(b)
        assert runner.cache.pages_held() == 0
        _within([np.abs(got[("a", p)] - ref[4][p]).max() for p in range(len(reqs[4]))], tol, dtype, "portions")
        _within([np.abs(got[("b", p)] - long_ref[p]).max() for p in range(len(long_toks))], tol, dtype, "decoded")
        _within([np.abs(got[("c", p)] - ref[0][p]).max() for p in range(len(reqs[0]))], tol, dtype, "neighbour")
        if first_round is None:
            first_round = got
        elif dtype == "float32":
            assert all(np.array_equal(got[k], first_round[k]) for k in got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_the_tensor_cores_do_not_take(dtype, tmp_path_factory):
    """A width of 52 and heads of 20 and 12: every product and the attention run on the plain
    kernels; a window on a ring of pages; a filter of one tap.  Prompts in portions of two tokens,
    then token by token, against the whole."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    folder = _sharp_folder(tmp_path_factory, NOGOSUN_C, seed=5, factor=12.0)
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(13)
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (61, 2, 30)]
    ref = [plain.forward(cfg, w, r) for r in reqs]
    scale = max(float(np.abs(r).max()) for r in ref)
    runner = Runner(build_model(folder, dtype=dtype), max_tokens=4 * PAGE, max_batch=3)
    slots = [runner.open() for _ in reqs]
    errs = []
    for live in _steps([len(r) for r in reqs], [2, 2, 2, 2, 1]):
        out = runner.step([StepItem(slots[i], reqs[i][lo:hi], range(hi - lo)) for i, lo, hi in live]).cpu().numpy()
        at = 0
        for i, lo, hi in live:
            errs += list(np.abs(out[at:at + hi - lo] - ref[i][lo:hi]).max(axis=1))
            at += hi - lo
    assert len(errs) == sum(len(r) for r in reqs)
    _within(errs, (TOL_F32 if dtype == "float32" else TOL_BF16) * scale, dtype, "portions of two")
    for s in slots:
        runner.close(s)
    assert runner.cache.pages_held() == 0


def test_routed_layers_of_unequal_shapes_in_long_prompts(tmp_path_factory):
    """Prompts of more than 256 tokens on the tensor cores, the routed layers with other expert counts
    and other numbers chosen from layer to layer; several prompts one after the other, the status of
    every bounded wait checked, the logits against the plain implementation."""
    from gemmars_b200 import kernels
    from gemmars_b200.engine import Runner, StepItem, build_model
    raw = {"architecture": "Nogosun", "vocab": 150, "width": 192, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
           "layers": [{"type": "channel_delta", "mixer": _nogosun_delta(4, 4, 16, 16, 3, 8, 8), "mlp": _nogosun_moe(14, 1, 48)},
                      {"type": "attention", "mixer": _nogosun_attention(6, 2, 48, 0.125, 129, 9, 1e6, 48), "mlp": _nogosun_moe(7, 4, 48)},
                      {"type": "parallel", "mixer": _nogosun_pair((2, 1, 32, 16, 0.2, 20.0, (0.3, 100)), (1, 16, 32, 8.0, 8), 1.0, 0.7),
                       "mlp": _nogosun_moe(2, 2, 48)}]}
    folder = _sharp_folder(tmp_path_factory, raw, seed=7, factor=3.0)
    cfg, w = plain.load_folder(folder)
    rng = np.random.default_rng(7)
    runner = Runner(build_model(folder, dtype="bfloat16"), max_tokens=16 * PAGE, max_batch=2)
    for n in (301, 261, 496, 260):
        toks = rng.integers(0, raw["vocab"], n).tolist()
        slot = runner.open()
        got = runner.step([StepItem(slot, toks, [n - 2, n - 1])]).cpu().numpy()
        kernels.check_status()
        runner.close(slot)
        want = plain.forward(cfg, w, toks)[-2:]
        assert np.abs(got - want).max() <= 2 * TOL_BF16 * np.abs(want).max(), f"a prompt of {n} tokens"


def _random_configuration(rng):
    """Layers of the three kinds in any order with sizes drawn at random, some of them running the
    tensors of another layer, named before or after them."""
    def moe():
        if rng.random() < 0.15:
            return None
        experts = int(rng.integers(1, 13))
        return _nogosun_moe(experts, int(rng.integers(1, min(experts, 5) + 1)), int(rng.choice([24, 32, 40, 64])))

    def attention():
        g = int(rng.choice([1, 2, 4]))
        d = int(rng.choice([16, 24, 32, 40, 64, 80]))
        size = int(rng.integers(3, 150)) if rng.random() < 0.85 else None
        keep = int(rng.choice([0, 1, 5, 66])) if size is not None and rng.random() < 0.8 else None
        dims = int(rng.choice([0, d, d // 2 - (d // 2) % 2, 4]))
        scaling = None if rng.random() < 0.4 else (float(rng.choice([2.0, 6.0, 20.0])), int(rng.choice([32, 300, 2000])),
                                                   float(rng.choice([16.0, 4.0])), float(rng.choice([2.0, 0.5])))
        return _nogosun_attention(g * int(rng.choice([1, 2, 3])), g, d, float(d ** -0.5 * rng.uniform(0.7, 1.5)), size, keep,
                                  float(rng.choice([1e4, 3e5, 400.0])), dims if dims else None, scaling if dims else None)

    def delta():
        g = int(rng.choice([1, 2, 3]))
        d = int(rng.choice([16, 24, 32, 48, 64, 72]))
        return _nogosun_delta(g * int(rng.choice([1, 2])), g, d, int(rng.choice([16, 24, 40, 64, d])), int(rng.integers(1, 6)),
                              int(rng.choice([3, 8, 20])), int(rng.choice([2, 8, 12])))

    def pair():
        g = int(rng.choice([1, 2]))
        d = int(rng.choice([16, 24, 32, 64]))
        left = (g * int(rng.choice([1, 2, 4])), g, d, int(rng.choice([16, 40, 64, d])), float(d ** -0.5),
                float(rng.choice([4.0, 20.0])) if rng.random() < 0.8 else None,
                (float(rng.uniform(0.1, 1.0)), int(rng.choice([1, 9, 64]))) if rng.random() < 0.8 else None)
        right = (int(rng.integers(1, 6)), int(rng.choice([16, 24, 48, 64])), int(rng.choice([16, 40, 64])),
                 float(rng.choice([1.0, 3.0, 12.0])), int(rng.choice([3, 8, 10])))
        return _nogosun_pair(left, right, float(rng.uniform(0.3, 1.2)), float(rng.uniform(0.3, 1.2)))

    layers = []
    for i in range(int(rng.integers(3, 8))):
        owners = [j for j, layer in enumerate(layers) if "weights_of" not in layer]
        if owners and rng.random() < 0.3:
            j = int(rng.choice(owners))
            layers.append(dict(json.loads(json.dumps(layers[j])), weights_of=j))
            continue
        kind = str(rng.choice(["attention", "channel_delta", "parallel"]))
        layers.append({"type": kind, "mixer": {"attention": attention, "channel_delta": delta, "parallel": pair}[kind](),
                       "mlp": moe()})
    sharers = [i for i, layer in enumerate(layers) if "weights_of" in layer]
    if sharers and rng.random() < 0.5:            # the later layer owns the tensors, the earlier one names it
        i = sharers[0]
        j = layers[i].pop("weights_of")
        if not any(layer.get("weights_of") == j for layer in layers):
            layers[j]["weights_of"] = i
        else:
            layers[i]["weights_of"] = j
    return {"architecture": "Nogosun", "vocab": int(rng.choice([97, 300, 1000])), "width": int(rng.choice([52, 64, 96, 136, 200])),
            "embedding": {"scale": float(rng.uniform(1.0, 20.0))}, "norm": {"eps": float(rng.choice([1e-5, 1e-6]))},
            "layers": layers}


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_random_configurations(seed, tmp_path_factory):
    """A configuration drawn at random, in float32: three unequal prompts in one batch, then token by
    token together until the shortest ends and on, against the plain implementation's whole prompts."""
    from gemmars_b200.engine import Runner, StepItem, build_model
    rng = np.random.default_rng(1000 + seed)
    raw = _random_configuration(rng)
    folder = _sharp_folder(tmp_path_factory, raw, seed=seed, factor=2.0)
    cfg, w = plain.load_folder(folder)
    lens = [int(n) for n in rng.choice([2, 17, 70, 131, 200], 3)]
    reqs = [rng.integers(0, raw["vocab"], n).tolist() for n in lens]
    ref = [plain.forward(cfg, w, r) for r in reqs]
    scale = max(float(np.abs(r).max()) for r in ref)
    runner = Runner(build_model(folder, dtype="float32"), max_tokens=12 * PAGE, max_batch=3)
    slots = [runner.open() for _ in reqs]
    heads = [max(1, n - 9) for n in lens]
    errs = []
    out = runner.step([StepItem(s, r[:h], range(h)) for s, r, h in zip(slots, reqs, heads)]).cpu().numpy()
    at = 0
    for r, h in zip(ref, heads):
        errs += list(np.abs(out[at:at + h] - r[:h]).max(axis=1))
        at += h
    for k in range(9):
        live = [i for i in range(3) if heads[i] + k < lens[i]]
        out = runner.step([StepItem(slots[i], [reqs[i][heads[i] + k]], [0]) for i in live]).cpu().numpy()
        errs += [np.abs(out[n] - ref[i][heads[i] + k]).max() for n, i in enumerate(live)]
    assert len(errs) == sum(lens)
    assert max(errs) <= TOL_F32 * scale, f"{max(errs) / scale:.2e} of the largest logit, configuration {json.dumps(raw)}"
    for s in slots:
        runner.close(s)
    assert runner.cache.pages_held() == 0


def test_greedy_generation_through_the_engine(models):
    from gemmars_b200 import Engine
    folder, cfg, w, reqs, _ = models["A"]
    eng = Engine.load(folder, "dtype=float32;max_batch=3;max_tokens=2048")
    prompts = [reqs[0], reqs[2], [5], reqs[4][:33], reqs[3]]
    free_run, _ = plain.generate(cfg, w, prompts[0], 10)
    stop = [free_run[4]]
    res = eng.generate(prompts, max_tokens=10, stop_ids=stop)
    for p, r in zip(prompts, res):
        want, reason = plain.generate(cfg, w, p, 10, stop=stop)
        assert r.tokens == want and r.reason == reason
    assert eng.runner.cache.pages_held() == 0
    again = eng.generate(list(reversed(prompts)), max_tokens=10, stop_ids=stop)
    assert [r.tokens for r in reversed(again)] == [r.tokens for r in res]
    # bfloat16 decodes through captured steps: the tokens it picks are the plain model's best or within
    # rounding of it (but for the few that follow a token routed to another expert, see _within)
    eng16 = Engine.load(folder, "dtype=bfloat16;max_batch=4;max_tokens=2048")
    near, total = 0, 0
    for p, r in zip(prompts, eng16.generate(prompts, max_tokens=8, stop_ids=[])):
        assert len(r.tokens) == 8
        for i, tok in enumerate(r.tokens):
            row = plain.forward(cfg, w, list(p) + r.tokens[:i])[-1]
            near += bool(row[tok] >= row.max() - TOL_BF16 * np.abs(row).max())
            total += 1
    assert near >= 0.9 * total
    assert eng16.runner.cache.pages_held() == 0
