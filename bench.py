#!/usr/bin/env python3
"""Decode and prefill throughput of Qwen3-shaped models with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference] [--config 8b|4b|32b]
    python bench.py --compare toretar|kuporax|dalerax|nogosun [--sizes small,lite,mid] [--batch 8] [--context 4096]

``--config 8b`` (the default) is the headline benchmark.  A step is one decode step of a batch
of 8 sequences at a context of 8,192 tokens.  One JSON line is printed: ``value`` = decoded
tokens a second measured on the device over exactly K steps; ``e2e`` = the same through
``Engine.generate`` (host token ids in, host token ids out, every step's host-to-device and
device-to-host copies included) over 256 generated tokens a sequence; ``prefill`` = one prompt
of 2,048 tokens; ``roofline`` = bytes a decode step has to read (every weight once, the cache of
the live requests) over its time, against the measured copy bandwidth; ``points`` = decode at
batch 1 and 64, with the time, bytes, fraction and clocks of each under ``points_detail``.

``--config 4b``: 16 prompts of 128 to 4,096 tokens (uniform, seeded), 256 tokens each at
temperature 0.7 with a fixed seed, through ``Engine.generate``.  ``--config 32b``: a prompt of
2,048 tokens, then greedy decoding at batch 1 and 32 up to a context of 4,096.  Each prints one
line of the same form.

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else 6.65 TB/s and
1.59 PFLOP/s (an earlier measurement on the same pool).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


from gemmars_b200.tuning import SHAPES as CONFIGS, random_engine, synthetic_fill   # noqa: E402  (the layer sizes measured at)

CONTEXT = 8192
PREFILL_TOKENS = 2048
E2E_TOKENS = 256


def peaks():
    """(copy GB/s, bf16 TFLOP/s as a burst, bf16 TFLOP/s sustained under the power cap, where from)."""
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    hbm, tf, tf_sustained, src = 6650.0, 1590.0, 1400.0, "fallback"
    try:
        with open(path) as f:
            p = json.load(f)
        hbm = float(p.get("hbm_gbs", hbm))
        tf = float(p.get("bf16_tflops", tf))
        tf_sustained = float(p.get("bf16_tflops_sustained", min(tf, tf_sustained)))
        src = "measured"
    except (OSError, ValueError):
        pass
    return hbm, tf, tf_sustained, src


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(int(r[0]))
                mx.append(int(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def kv_bytes_per_token(runner):
    """Bytes of keys and values one cached position takes over all layers (groups that keep all keys)."""
    return sum(g.n_layers * g.need.num_kv_heads * (g.need.head_dim + _value_dim(g)) * g.k.element_size()
               for g in runner.cache.kv_groups)


def _value_dim(group):
    return group.need.head_dim if group.need.value_dim is None else group.need.value_dim


def decode_bytes(model, runner, lengths, cache_bytes=None):
    """Bytes one decode step has to read: every weight once and the cached keys and values of
    the live sequences (``cache_bytes``: that share, where masks and not rings bound what is read)."""
    kv = 0
    for g in (runner.cache.kv_groups if cache_bytes is None else ()):
        per_token = g.n_layers * g.need.num_kv_heads * (g.need.head_dim + _value_dim(g)) * g.k.element_size()
        for n in lengths:
            kv += per_token * (min(n, g.need.window) if g.need.window else n)
    # a part whose reads grow with the batch (routed experts: every expert some token chose) says so itself
    extra = 0
    for block in model.blocks:
        for part in block.parts().values():
            if hasattr(part, "decode_bytes"):
                extra += part.decode_bytes(len(lengths)) - part.weight_bytes()
    # a fixed-size state per sequence (a recurrent mixer's) is read and written once a step
    state = 0
    for g in runner.cache.state_groups:
        per_seq = g.data.element_size() * g.data.shape[0]
        for n in g.need.shape:
            per_seq *= n
        state += 2 * per_seq * len(lengths)
    return model.weight_bytes() + extra + kv + state + (cache_bytes or 0)


def prefill_flops(cfg, t):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_token = 2 * (h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * i)
    attn = 4 * nh * hd * (t * (t + 1) // 2)           # QK^T and PV over the causal half
    return cfg["num_hidden_layers"] * (per_token * t + attn) + 2 * h * v  # logits of the last row only


def toretar_prefill_flops(cfg, t):
    """Floating-point operations of a prompt of ``t`` tokens from position 0, counted as useful
    arithmetic of the way the engine takes: over expanded heads where it expands keys and values
    (scores over dim + rot_dim, values of vdim, and the two expansions of the latents), else over
    the latent rows (scores over kv_rank + rot_dim, values of kv_rank, and the two per-head products
    on the query side)."""
    import torch
    from gemmars_b200 import kernels
    w, total = cfg["width"], 0
    pairs = t * (t + 1) // 2
    for layer in cfg["layers"]:
        m, mlp = layer["mixer"], layer["mlp"]
        nh, dim, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        per_token = 2 * (w * (nh * (dim + rd) + r + rd + nh) + nh * vd * w)
        if t >= kernels.LATENT_EXPAND_MIN_TOKENS and kernels.latent_expand_usable(torch.bfloat16, r, dim, rd, vd):
            per_token += 2 * nh * (dim + vd) * r
            attention = 2 * nh * (dim + rd + vd) * pairs
        else:
            per_token += 2 * (nh * dim * r + nh * r * vd)
            attention = 2 * nh * (2 * r + rd) * pairs
        if mlp is not None:
            per_token += 2 * w * mlp["router"]["experts"] + 6 * w * mlp["router"]["top"] * mlp["expert"]["ff"]
            if mlp.get("shared"):
                per_token += 6 * w * mlp["shared"]["ff"]
        total += per_token * t + attention
    return total + 2 * w * cfg["vocab"]


def kuporax_prefill_flops(cfg, t):
    """Floating-point operations of a prompt of ``t`` tokens from position 0: every product, the
    attention's scores and weighted values over the keys a window lets a token see, and the
    recurrences as they are written (delta rule: two reads of the state and one update a token,
    6 dim vdim a head; state space: one update and one read, 4 state vdim a head)."""
    w, total = cfg["width"], 0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        if layer["type"] == "delta":
            qk, hv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            per_token = 2 * w * (2 * qk + 2 * hv + 2 * m["heads"]) + 2 * hv * w + 6 * m["heads"] * m["dim"] * m["vdim"]
            pairs = 0
        else:
            a, r = m["left"], m["right"]
            size = a["mask"]["size"]
            seen = sum(min(p + 1, size) for p in range(t))
            pairs = 2 * a["heads"] * (a["dim"] + a["vdim"]) * seen
            inner = r["heads"] * r["vdim"]
            per_token = (2 * w * ((a["heads"] + a["kv_heads"]) * a["dim"] + a["kv_heads"] * a["vdim"] + a["heads"] * a["vdim"])
                         + 2 * a["heads"] * a["vdim"] * w
                         + 2 * w * (2 * inner + 2 * r["groups"] * r["state"] + r["heads"]) + 2 * inner * w
                         + 4 * r["heads"] * r["state"] * r["vdim"])
        if layer.get("mlp") is not None:
            per_token += 6 * w * layer["mlp"]["ff"]
        total += per_token * t + pairs
    return total + 2 * w * cfg["vocab"]


def _dalerax_seen(mask, p):
    """Keys position ``p`` sees: itself and the window before it, and the kept first ones the window has left."""
    size, keep = mask["size"], mask.get("keep_first", 0)
    return min(p + 1, size) + max(0, min(keep, p + 1 - size))


def dalerax_prefill_flops(cfg, t):
    """Floating-point operations of a prompt of ``t`` tokens from position 0: every product, the
    scores and weighted values over the keys each token's mask lets it see, the decay's two small
    products, the recurrence as it is written (one update and one read of the state a token,
    4 dim dim a head), and for a routed feed-forward the router and the chosen experts."""
    w, total = cfg["width"], 0
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        if layer["type"] == "attention":
            own = 0 if "kv_from" in m else m["kv_heads"] * (m["dim"] + m["vdim"])
            per_token = 2 * w * (m["heads"] * m["dim"] + own) + 2 * m["heads"] * m["vdim"] * w
            pairs = 2 * m["heads"] * (m["dim"] + m["vdim"]) * sum(_dalerax_seen(m["mask"], p) for p in range(t))
        else:
            n, rank = m["heads"] * m["dim"], m.get("rank", 32)
            per_token = 2 * w * (4 * n + rank) + 2 * rank * n + 2 * n * w + 4 * m["heads"] * m["dim"] * m["dim"]
            pairs = 0
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "dense":
            per_token += 6 * w * mlp["ff"]
        elif mlp is not None:
            per_token += 2 * w * mlp["router"]["experts"] + 6 * w * mlp["router"]["top"] * mlp["expert"]["ff"]
            if mlp.get("shared"):
                per_token += 6 * w * mlp["shared"]["ff"]
        total += per_token * t + pairs
    return total + 2 * w * cfg["vocab"]


def dalerax_cache_bytes(cfg, lengths, element_size=2):
    """Bytes of cached keys and values one decode step reads: every attention layer, also one that
    reads another layer's cache, reads what its own mask sees."""
    total = 0
    for layer in cfg["layers"]:
        if layer["type"] != "attention":
            continue
        m = layer["mixer"]
        per_key = m["kv_heads"] * (m["dim"] + m["vdim"]) * element_size
        total += sum(per_key * _dalerax_seen(m["mask"], n - 1) for n in lengths)
    return total


def nogosun_prefill_flops(cfg, t):
    """Floating-point operations of a prompt of ``t`` tokens from position 0: every product (a layer
    that runs another layer's tensors counts like one of its own), the scores and weighted values over
    the keys each token's mask lets it see, the two-matrix projections, the recurrences as they are
    written (delta rule: 6 dim vdim a head and token; gated linear attention: 4 dim vdim), the router
    and the chosen experts (two matrices each)."""
    w, total = cfg["width"], 0
    for layer in cfg["layers"]:
        m, pairs = layer["mixer"], 0
        if layer["type"] == "attention":
            per_token = 2 * w * (m["heads"] + m["kv_heads"]) * m["dim"] + 2 * m["heads"] * m["vdim"] * w
            mask = m.get("mask")
            seen = sum(_dalerax_seen(mask, p) for p in range(t)) if mask else t * (t + 1) // 2
            pairs = 2 * m["heads"] * (m["dim"] + m["vdim"]) * seen
        elif layer["type"] == "channel_delta":
            qk, hv, hd = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"] * m["dim"]
            ra, rg = m.get("decay_rank", 16), m.get("gate_rank", 16)
            per_token = (2 * w * (2 * qk + hv + m["heads"] + ra + rg) + 2 * (ra * hd + rg * hv) + 2 * hv * w
                         + 6 * m["heads"] * m["dim"] * m["vdim"])
        else:
            a, r = m["left"], m["right"]
            per_token = (2 * w * ((a["heads"] + a["kv_heads"]) * a["dim"] + (a["kv_heads"] + a["heads"]) * a["vdim"])
                         + 2 * a["heads"] * a["vdim"] * w)
            pairs = 2 * a["heads"] * (a["dim"] + a["vdim"]) * (t * (t + 1) // 2)
            hd, hv, rank = r["heads"] * r["dim"], r["heads"] * r["vdim"], r.get("rank", 16)
            per_token += 2 * w * (2 * hd + 2 * hv + rank) + 2 * rank * hd + 2 * hv * w + 4 * r["heads"] * r["dim"] * r["vdim"]
        mlp = layer.get("mlp")
        if mlp is not None:
            per_token += 2 * w * mlp["router"]["experts"] + 4 * w * mlp["router"]["top"] * mlp["expert"]["ff"]
        total += per_token * t + pairs
    return total + 2 * w * cfg["vocab"]


def nogosun_cache_bytes(cfg, lengths, element_size=2):
    """Bytes of cached keys and values one decode step reads: what each attention's mask sees (every
    key for the two-branch layer's attention); values that are the keys are cached, and read, as values too."""
    total = 0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        if layer["type"] == "parallel":
            m = m["left"]
        elif layer["type"] != "attention":
            continue
        per_key = m["kv_heads"] * (m["dim"] + m["vdim"]) * element_size
        mask = m.get("mask")
        total += sum(per_key * (_dalerax_seen(mask, n - 1) if mask else n) for n in lengths)
    return total


def fill_cache(runner, slots, length, real, vocab, gen):
    """Brings every slot to ``length`` cached tokens: by running prompts (real) or by
    reserving the pages and writing random keys and values (synthetic)."""
    import torch
    from gemmars_b200.engine.step import StepItem
    if real:
        for s in slots:
            toks = torch.randint(0, vocab, (length,), generator=gen).tolist()
            runner.step([StepItem(s, toks, [])])
        return
    synthetic_fill(runner, slots, length)


def time_decode(eng, batch, ctx_end, steps, warmup, real_fill, hbm_gbs, cfg=None):
    """Device time of exactly ``steps`` decode steps of ``batch`` sequences ending at ``ctx_end``,
    with the clocks sampled meanwhile: {"tokens_per_s", "ms_per_step", "steps", "bytes_per_step",
    "achieved_gbs", "frac", "clocks", "launches"}."""
    import torch
    from gemmars_b200 import kernels
    from gemmars_b200.engine.step import StepItem
    from gemmars_b200.sampling.sampler import BatchSampler, SamplingParams
    runner, vocab = eng.runner, eng.model.plan.vocab_size
    gen = torch.Generator().manual_seed(1)
    slots = [runner.open() for _ in range(batch)]
    start_len = ctx_end - steps - warmup
    fill_cache(runner, slots, start_len, real_fill, vocab, gen)
    sampler = BatchSampler([SamplingParams()] * batch, runner.device)
    toks = torch.randint(0, vocab, (batch,), generator=gen).tolist()

    rows = list(range(batch))
    ahead = eng.options.decode_ahead and runner.use_graphs

    def one(logits):
        """A step as the generation loop runs it: draw from the logits, launch the next step from
        the drawn tokens where they lie, then read them on the host (what generation needs them
        for: stop tokens, limits, the caller)."""
        drawn = sampler.draw(logits, rows)
        nxt = runner.decode_from_device(slots, drawn) if ahead else None
        toks = sampler.read(drawn)
        if nxt is None:
            nxt = runner.step([StepItem(s, [t], [0]) for s, t in zip(slots, toks)])
        return nxt

    logits = runner.step([StepItem(s, [t], [0]) for s, t in zip(slots, toks)])
    for _ in range(warmup - 1):
        logits = one(logits)
    torch.cuda.synchronize()
    clocks = ClockSampler().start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = kernels.launch_count()
    e0.record()
    for _ in range(steps):
        logits = one(logits)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    clock_rec = clocks.stop()
    lengths = [runner.length(s) for s in slots]
    masked = {"Dalerax": dalerax_cache_bytes, "Nogosun": nogosun_cache_bytes}.get(cfg.get("architecture")) if cfg else None
    nbytes = decode_bytes(eng.model, runner, lengths, masked(cfg, lengths) if masked else None)
    for s in slots:
        runner.close(s)
    kernels.check_status()
    achieved = nbytes / (ms / 1e3) / 1e9
    return {"tokens_per_s": round(batch / (ms / 1e3), 1), "ms_per_step": round(ms, 4), "steps": steps,
            "bytes_per_step": nbytes, "achieved_gbs": round(achieved, 1), "frac": round(achieved / hbm_gbs, 4),
            "clocks": clock_rec, "launches": kernels.launch_count() - launches0}


def time_prefill(eng, cfg, tokens, tflops, tflops_sustained):
    """The median of seven prompts of ``tokens`` tokens after three warm-up prompts."""
    import torch
    from gemmars_b200.engine.step import StepItem
    runner = eng.runner
    vocab = cfg["vocab_size"] if "vocab_size" in cfg else cfg["vocab"]
    toks = torch.randint(0, vocab, (tokens,), generator=torch.Generator().manual_seed(3)).tolist()
    pre_ms = []
    for it in range(10):
        s = runner.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepItem(s, toks, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        if it >= 3:
            pre_ms.append(e0.elapsed_time(e1))
        runner.close(s)
    pre = statistics.median(pre_ms)
    if cfg.get("architecture") == "Kuporax":
        flops = kuporax_prefill_flops(cfg, tokens)
    elif cfg.get("architecture") == "Dalerax":
        flops = dalerax_prefill_flops(cfg, tokens)
    elif cfg.get("architecture") == "Nogosun":
        flops = nogosun_prefill_flops(cfg, tokens)
    elif cfg.get("sliding_window") and cfg.get("use_sliding_window"):
        size = cfg["sliding_window"]      # a window on every layer: the keys a token sees, not the causal half
        seen = sum(min(p + 1, size) for p in range(tokens))
        flops = (prefill_flops(cfg, tokens) + cfg["num_hidden_layers"] * 4 * cfg["num_attention_heads"] * cfg["head_dim"]
                 * (seen - tokens * (tokens + 1) // 2))
    else:
        flops = toretar_prefill_flops(cfg, tokens) if "layers" in cfg else prefill_flops(cfg, tokens)
    frac = flops / (pre / 1e3) / (tflops * 1e12)
    return {"value": round(tokens / (pre / 1e3), 1), "tokens": tokens, "ms": round(pre, 3), "frac": round(frac, 4),
            # a prompt is tens of milliseconds of products under the power cap: also against the sustained rate
            "frac_sustained": round(frac * tflops / tflops_sustained, 4)}


def make_engine(cfg, max_batch, cache_tokens, options=""):
    return random_engine(cfg, max_batch, cache_tokens, options)


def config_record(name, cfg, layers_full, batch, context, fill, peak_line):
    return {"model": name, "layers": cfg["num_hidden_layers"], "layers_full": layers_full,
            "hidden_size": cfg["hidden_size"], "intermediate_size": cfg["intermediate_size"],
            "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "vocab_size": cfg["vocab_size"],
            "tie_word_embeddings": cfg["tie_word_embeddings"], "global_batch": batch, "seq_len": context,
            "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU", "cache_fill": fill,
            "points_cache_fill": "synthetic", "l2": "weights and cache read per step exceed L2 (no flush needed)",
            "peaks": peak_line}


def run_8b(args, name, cfg, layers_full):
    import torch
    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    warmup = max(3, args.warmup)
    points = not args.no_points
    max_batch = 64 if points else args.batch
    eng = make_engine(cfg, max_batch, max_batch * (args.context + 64), args.options)
    vocab = cfg["vocab_size"]
    # a prompt first: it is a burst of work on a GPU that was waiting
    prefill = time_prefill(eng, cfg, PREFILL_TOKENS, tflops, tflops_sustained)
    main = time_decode(eng, args.batch, args.context, args.steps, warmup, args.fill == "real", hbm_gbs)

    # end to end through the entry point: host ids in, host ids out, 256 tokens a sequence
    gen = torch.Generator().manual_seed(2)
    e2e_new = max(2, args.e2e_tokens)
    prompts = [torch.randint(0, vocab, (args.context - e2e_new,), generator=gen).tolist() for _ in range(args.batch)]
    clocks = ClockSampler().start()
    res = eng.generate(prompts, max_tokens=e2e_new, stop_ids=[])
    e2e_clocks = clocks.stop()
    st = eng.stats
    assert all(len(r.tokens) == e2e_new for r in res)

    pts, detail = {}, {}
    if points:
        for b in (1, 64):
            d = time_decode(eng, b, args.context, min(args.steps, 16), 3, False, hbm_gbs)
            pts[f"decode_b{b}"] = d["tokens_per_s"]
            detail[f"decode_b{b}"] = {k: d[k] for k in ("ms_per_step", "steps", "bytes_per_step", "achieved_gbs", "frac", "clocks")}
    return {
        "metric": f"decode tok/s at batch {args.batch}, context {args.context} ({name}, bf16, random weights)",
        "value": main["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids",
        "config": config_record(name, cfg, layers_full, args.batch, args.context, args.fill,
                                f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})"),
        "clocks": main["clocks"],
        "e2e": {"value": round(st.generated_tokens / max(st.decode_secs, 1e-9), 1), "unit": "tokens/s",
                "h2d_bytes_per_step": (8 * args.batch + 1) * 4, "d2h_bytes_per_step": args.batch * 4,
                "generated": st.generated_tokens, "decode_steps": st.decode_steps,
                "prefill_secs": round(st.prefill_secs, 3), "sm_mhz": e2e_clocks["sm_mhz"]},
        "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main["achieved_gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": main["frac"], "bytes_per_step": main["bytes_per_step"]},
        "points": pts,
        "points_detail": detail,
    }


def run_4b(args, name, cfg, layers_full):
    """16 prompts of 128 to 4,096 tokens, 256 tokens each at temperature 0.7, seed fixed, through
    ``Engine.generate``."""
    import numpy as np
    import torch
    from gemmars_b200.sampling.sampler import SamplingParams
    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    batch, new = 16, 256
    rng = np.random.default_rng(4)
    lengths = [int(x) for x in rng.integers(128, 4097, batch)]
    eng = make_engine(cfg, batch, batch * (4096 + new + 64), args.options)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]
    sampling = SamplingParams(temperature=0.7, top_k=64, top_p=0.95, seed=42)
    prefill = time_prefill(eng, cfg, PREFILL_TOKENS, tflops, tflops_sustained)
    eng.generate([p[:64] for p in prompts], max_tokens=8, sampling=sampling, stop_ids=[])      # warm-up: builds, graphs
    clocks = ClockSampler().start()
    res = eng.generate(prompts, max_tokens=new, sampling=sampling, stop_ids=[])
    clock_rec = clocks.stop()
    st = eng.stats
    assert all(len(r.tokens) == new for r in res)
    # bytes the decode steps had to read: the weights every step, and each sequence's cache as it grows
    per_tok = kv_bytes_per_token(eng.runner)
    steps = st.decode_steps
    kv = sum(per_tok * (n + k) for n in lengths for k in range(1, steps + 1))
    nbytes = steps * eng.model.weight_bytes() + kv
    achieved = nbytes / max(st.decode_secs, 1e-9) / 1e9
    ms = st.decode_secs * 1e3 / max(steps, 1)
    value = st.generated_tokens / max(st.decode_secs, 1e-9)
    return {
        "metric": f"decode tok/s, 16 prompts of 128-4096 tokens, 256 tokens each at temperature 0.7 ({name}, bf16, random weights)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 8,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids",
        "config": dict({k: v for k, v in config_record(name, cfg, layers_full, batch, max(lengths) + new, "real",
                                                       f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})").items()
                        if k not in ("cache_fill", "points_cache_fill")},
                       prompt_tokens=sum(lengths), mean_prompt=round(sum(lengths) / batch, 1),
                       sampling="temperature 0.7, top_k 64, top_p 0.95, seed 42", timing="wall clock through Engine.generate"),
        "clocks": clock_rec,
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "h2d_bytes_per_step": (8 * batch + 1) * 4 + 16 * batch,
                "d2h_bytes_per_step": batch * 4, "generated": st.generated_tokens, "decode_steps": steps,
                "prefill_secs": round(st.prefill_secs, 3),
                "prefill_tokens_per_s": round(sum(lengths) / max(st.prefill_secs, 1e-9), 1)},
        "gpu_launches": None,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s",
                     "frac": round(achieved / hbm_gbs, 4), "bytes_per_step": nbytes // max(steps, 1)},
        "points": {},
    }


def run_32b(args, name, cfg, layers_full):
    """A prompt of 2,048 tokens, then greedy decoding at batch 1 and 32 up to a context of 4,096."""
    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    context, steps, warmup = 4096, args.steps, max(3, args.warmup)
    eng = make_engine(cfg, 32, 32 * (context + 64), args.options)
    prefill = time_prefill(eng, cfg, PREFILL_TOKENS, tflops, tflops_sustained)
    main = time_decode(eng, 32, context, steps, warmup, args.fill == "real", hbm_gbs)
    one = time_decode(eng, 1, context, steps, warmup, args.fill == "real", hbm_gbs)
    keep = ("ms_per_step", "steps", "bytes_per_step", "achieved_gbs", "frac", "clocks")
    return {
        "metric": f"decode tok/s at batch 32, context {context} ({name}, bf16, random weights)",
        "value": main["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, random token ids",
        "config": config_record(name, cfg, layers_full, 32, context, args.fill,
                                f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})"),
        "clocks": main["clocks"], "gpu_launches": main["launches"], "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main["achieved_gbs"], "peak": hbm_gbs, "unit": "GB/s",
                     "frac": main["frac"], "bytes_per_step": main["bytes_per_step"]},
        "points": {"decode_b1": one["tokens_per_s"], "decode_b32": main["tokens_per_s"]},
        "points_detail": {"decode_b1": {k: one[k] for k in keep}, "decode_b32": {k: main[k] for k in keep}},
    }


def kernel_table(eng, tokens, batch, context):
    """Per kernel, without captured steps: calls, microseconds a call and the bytes the launch said
    it moves, for one prompt of ``tokens`` tokens and for one decode step of ``batch`` sequences at
    ``context`` cached tokens."""
    import torch
    from gemmars_b200 import kernels
    from gemmars_b200.engine.step import StepItem
    runner = eng.runner
    was, runner.use_graphs = runner.use_graphs, False
    out = {}
    try:
        toks = torch.randint(0, eng.model.plan.vocab_size, (tokens,), generator=torch.Generator().manual_seed(5)).tolist()
        for phase in ("prompt", "decode"):
            if phase == "prompt":
                warm = runner.open()              # a warm-up prompt in a slot of its own
                runner.step([StepItem(warm, toks, [tokens - 1])])
                runner.close(warm)
                slots = [runner.open()]
                items = [StepItem(slots[0], toks, [tokens - 1])]
            else:
                slots = [runner.open() for _ in range(batch)]
                synthetic_fill(runner, slots, context - 2)
                items = [StepItem(s, [1], [0]) for s in slots]
                runner.step(items)
            torch.cuda.synchronize()
            kernels.profile_start()
            runner.step(items)
            totals = kernels.profile_totals()
            out[phase] = {name: {"calls": c, "us_per_call": round(ms * 1e3 / c, 2), "mb_per_call": round(nb / c / 1e6, 3)}
                          for name, (c, ms, nb) in sorted(totals["kernels"].items(), key=lambda kv: -kv[1][1])}
            for s in slots:
                runner.close(s)
    finally:
        runner.use_graphs = was
    return out


def run_compare(args):
    """Prompt and decode throughput of models of one architecture beside models of another with the
    same width, depth and per-token feed-forward size (Toretar and Kuporax beside Qwen3, Dalerax
    beside Kuporax, Nogosun beside Dalerax), with a table of each one's kernels."""
    from gemmars_b200.tuning import DALERAX_PAIRS, KUPORAX_PAIRS, NOGOSUN_PAIRS, PAIRS
    pairs = {"kuporax": KUPORAX_PAIRS, "dalerax": DALERAX_PAIRS, "nogosun": NOGOSUN_PAIRS}.get(args.compare, PAIRS)
    beside = {"dalerax": "kuporax", "nogosun": "dalerax"}.get(args.compare, "qwen3")
    hbm_gbs, tflops, tflops_sustained, peak_src = peaks()
    sizes = [s for s in args.sizes.split(",") if s]
    out = {}
    for size in sizes:
        out[size] = {}
        for arch, cfg in zip((args.compare, beside), pairs[size]):
            eng = make_engine(cfg, args.batch, args.batch * (args.context + 64) + PREFILL_TOKENS + 64, args.options)
            rec = {"prefill": time_prefill(eng, cfg, PREFILL_TOKENS, tflops, tflops_sustained),
                   "decode": time_decode(eng, args.batch, args.context, args.steps, max(3, args.warmup), False, hbm_gbs, cfg)}
            if not args.no_points:
                rec["kernels"] = kernel_table(eng, PREFILL_TOKENS, args.batch, args.context)
            out[size][arch] = rec
            del eng
            import gc
            import torch
            gc.collect()
            torch.cuda.empty_cache()
    return {"compare": f"{args.compare} beside {beside}", "sizes": out, "batch": args.batch, "context": args.context,
            "prefill_tokens": PREFILL_TOKENS, "peaks": f"{hbm_gbs:.0f} GB/s, {tflops:.0f} TFLOP/s ({peak_src})",
            "dtype": "bf16", "data": "synthetic: random weights, random token ids, cache filled with random rows"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", choices=sorted(CONFIGS), default="8b", help="which model shape and workload")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in config)")
    ap.add_argument("--fill", choices=["real", "synthetic"], default="real",
                    help="how the cache is brought to the context length before decoding is timed")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--e2e-tokens", type=int, default=E2E_TOKENS,
                    help="tokens a sequence generates in the end-to-end run (fewer for runs under a profiler)")
    ap.add_argument("--options", default="", help='further engine options, "key=value;key=value"')
    ap.add_argument("--compare", choices=["toretar", "kuporax", "dalerax", "nogosun"], default=None,
                    help="instead of the headline: models of that architecture beside ones of equal size (Qwen3-shaped; "
                         "Kuporax-shaped for dalerax; Dalerax-shaped for nogosun)")
    ap.add_argument("--sizes", default="small,lite,mid", help="with --compare: which pairs of tuning.PAIRS")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate (oxinfer); no cargo/rustc offline, so pip cannot build it; "
                          "it publishes no NVIDIA path that runs decode on the GPU"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported", flush=True)
        return 2
    if args.compare:
        print(json.dumps(run_compare(args)), flush=True)
        return 0
    name, cfg = CONFIGS[args.config]
    layers_full = cfg["num_hidden_layers"]
    cfg = dict(cfg, num_hidden_layers=args.layers or layers_full)
    # three shapes have workloads of their own; any other runs the 8B workload at its own sizes
    line = {"4b": run_4b, "32b": run_32b}.get(args.config, run_8b)(args, name, cfg, layers_full)
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
