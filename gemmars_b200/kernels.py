"""Python faces of the CUDA units: argument checks, then one call into the compiled library.

Every function here works on CUDA tensors only and launches on PyTorch's current stream.  There
is no CPU or library fallback: a tensor that is not on a CUDA device, or a unit that cannot be
built, raises.

Two kernels keep scratch memory per device between their launches (the decode attention's parts,
the words that order the parts of a split prompt tile): work for one device is therefore launched
on one stream at a time, as the engine does; two engines on one device take turns.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
OUT_STORE, OUT_ACCUMULATE = 0, 1
FLAG_NORM, FLAG_ROPE, FLAG_CACHE, FLAG_INPLACE, FLAG_SINGLE = 1, 2, 4, 8, 32
MAX_TOP_K = 1024

_ERRORS = {-2: "unsupported element type", -3: "unsupported size", -4: "missing argument"}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dt} is not supported by the CUDA kernels (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    # the raw handle of the current stream of the current device (what
    # torch.cuda.current_stream().cuda_stream gives, without building a Stream object per launch)
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


_launches = [0]


def launch_count() -> int:
    """Kernels of this package launched so far (launches replayed from CUDA graphs included)."""
    return _launches[0]


def count_launches(n: int) -> None:
    _launches[0] += n


# Timing for --profile: an event after every launch; the time between two events is put down to
# the later kernel (kernels of one stream run one after the other).  Every face also says which
# category its kernel belongs to and how many bytes the launch has to move (weights, inputs,
# results, cached keys and values where the host knows the lengths), so that the report can give
# time, calls, bytes and bandwidth per category as the reference's does (src/prof.rs:8-83).
CATEGORIES = ("matmul", "attention", "norm", "elementwise", "embed", "lm_head", "sampling")
_profile = {"on": False, "events": [], "category": None}


def profile_start() -> None:
    """Starts collecting one CUDA event per launch (use without CUDA graphs)."""
    _profile["on"], _profile["events"] = True, []
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    _profile["events"].append(("start", None, 0, ev))


class profile_category:
    """Within the block, launches are put down to ``name`` whatever their own category (the
    output head's product is a matmul that the report lists on its own)."""

    def __init__(self, name: str):
        self.name, self.before = name, None

    def __enter__(self):
        self.before, _profile["category"] = _profile["category"], self.name

    def __exit__(self, *exc):
        _profile["category"] = self.before


def profile_totals() -> dict:
    """{"kernels": {name: [calls, ms, bytes]}, "categories": {name: [calls, ms, bytes]}} since
    profile_start; stops collecting.  Synchronizes."""
    _profile["on"] = False
    torch.cuda.synchronize()
    ev = _profile["events"]
    per_kernel, per_cat = {}, {}
    for (_, _, _, a), (name, cat, nbytes, b) in zip(ev, ev[1:]):
        ms = a.elapsed_time(b)
        t = per_kernel.setdefault(name, [0, 0.0, 0])
        t[0] += 1
        t[1] += ms
        t[2] += nbytes
        c = per_cat.setdefault(cat, [0, 0.0, 0])
        c[0] += 1
        c[1] += ms
        c[2] += nbytes
    _profile["events"] = []
    return {"kernels": per_kernel, "categories": per_cat}


def profile_report(tokens: int = 1, totals: Optional[dict] = None) -> str:
    """The time since profile_start per category and per kernel, in the manner of the
    reference's --profile (src/prof.rs:51-83): ms a token, calls a token, us a call, and for the
    categories the bytes a token and the bandwidth they come to.  ``tokens``: the forward tokens
    that ran meanwhile."""
    totals = totals or profile_totals()
    tokens = max(1, tokens)
    whole = sum(t[1] for t in totals["kernels"].values()) or 1.0
    lines = [f"[profile over {tokens} forward tokens, {whole / tokens:.3f} ms/token on the device]",
             f"{'category':14s} {'ms/tok':>9s} {'calls/tok':>10s} {'us/call':>9s} {'MB/tok':>10s} {'GB/s':>8s} {'share':>7s}"]
    for cat in CATEGORIES + tuple(c for c in totals["categories"] if c not in CATEGORIES):
        if cat not in totals["categories"]:
            continue
        calls, ms, nbytes = totals["categories"][cat]
        lines.append(f"{str(cat):14s} {ms / tokens:9.4f} {calls / tokens:10.2f} {ms * 1e3 / calls:9.1f} "
                     f"{nbytes / tokens / 1e6:10.4f} {nbytes / max(ms, 1e-9) / 1e6:8.1f} {100 * ms / whole:6.1f}%")
    lines.append(f"{'kernel':28s} {'ms/tok':>9s} {'calls/tok':>10s} {'us/call':>9s} {'share':>7s}")
    for name, (calls, ms, _) in sorted(totals["kernels"].items(), key=lambda kv: -kv[1][1]):
        lines.append(f"{name:28s} {ms / tokens:9.4f} {calls / tokens:10.2f} {ms * 1e3 / calls:9.1f} {100 * ms / whole:6.1f}%")
    lines.append(f"{'total':28s} {whole / tokens:9.4f}")
    return "\n".join(lines)


def _check(code: int, what: str, category: str = "elementwise", nbytes: int = 0):
    if code == 0:
        _launches[0] += 1
        if _profile["on"]:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _profile["events"].append((what, _profile["category"] or category, nbytes, ev))
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, 'refused')} (code {code})")
    raise KernelError(f"{what}: CUDA launch failed with error {code}")


def _nbytes(*tensors) -> int:
    """Bytes of the given tensors (None counts nothing): what a launch reads and writes."""
    return sum(t.numel() * t.element_size() for t in tensors if t is not None) if _profile["on"] else 0


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels of gemmars_b200 run on CUDA tensors only (got a CPU tensor); "
                              "there is no CPU path")


_sigs = {}


def _fn(unit: str, name: str, argtypes, defines=()):
    if build.pdl():
        defines = tuple(defines) + (build.PDL_DEFINE,)
    key = (unit, name, tuple(defines))
    f = _sigs.get(key)
    if f is None:
        lib = build.load(unit, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        _sigs[key] = f
    return f


# --------------------------------------------------------------------------- elementwise

def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0):
    """out[t] = table[tokens[t]] * scale; out is the float32 residual stream [T, H]."""
    _cuda(table, tokens, out)
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    f = _fn("elementwise", "gb_embed_gather",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), out.data_ptr(), tokens.numel(),
             table.shape[1], table.shape[0], scale, _stream()), "embed_gather", "embed",
           _nbytes(out) + tokens.numel() * table.shape[1] * table.element_size())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows_index: Optional[torch.Tensor] = None, second=None):
    """out[r] = rmsnorm(x[rows_index[r] or r]) * weight.  x float32 [*, n]; weight float32 [n].
    ``second`` (weight2, out2): another norm of the same rows with the same eps, whose statistics are
    the same; out2[r] = rmsnorm(x[...]) * weight2 is written in the same pass."""
    _cuda(x, weight, out, rows_index)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n = x.shape[-1]
    rows = out.numel() // n
    assert weight.numel() == n and out.shape[-1] == n
    if rows_index is not None:
        assert rows_index.dtype == torch.int32 and rows_index.numel() == rows
    w2, out2 = second if second is not None else (None, None)
    if second is not None:
        _cuda(w2, out2)
        assert w2.dtype == torch.float32 and w2.numel() == n and out2.shape == out.shape and out2.dtype == out.dtype
        assert out2.is_contiguous()
    f = _fn("elementwise", "gb_rmsnorm_pair",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p])
    _check(f(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype), _ptr(rows_index), rows, n,
             eps, _ptr(w2), _ptr(out2), _stream()), "rmsnorm", "norm", _nbytes(out, weight, out2, w2) + rows * n * 4)


def head_norm_rope_cache(qkv, nh, nkv, hd, rot, q_weight, k_weight, eps, inv_freq, q_scale, tok_pos, tok_seq,
                         seq_slot, page_table, page_size, kcache, vcache, flags):
    """Per-head RMSNorm, rotation and scale of q and k in place in ``qkv`` [T, (nh+2nkv)*hd], and
    the write of k and v into the paged cache; ``flags`` selects the steps."""
    _cuda(qkv, q_weight, k_weight, inv_freq, tok_pos, tok_seq, seq_slot, page_table, kcache, vcache)
    assert qkv.is_contiguous() and qkv.shape[-1] == (nh + 2 * nkv) * hd
    if flags & FLAG_CACHE:
        assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous()
        assert kcache.shape[1:] == (nkv, page_size, hd)
    f = _fn("elementwise", "gb_head_norm_rope_cache",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_float,
             c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.shape[0], nh, nkv, hd, rot, _ptr(q_weight), _ptr(k_weight),
             eps, _ptr(inv_freq), q_scale, tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(),
             _ptr(page_table), page_table.shape[1] if page_table is not None else 1, page_size, _ptr(kcache),
             _ptr(vcache), flags, _stream()), "head_norm_rope_cache", "elementwise",
           _nbytes(qkv) * (2 if flags & FLAG_INPLACE else 1)
           + (qkv.shape[0] * 2 * nkv * hd * qkv.element_size() if flags & FLAG_CACHE else 0))
    if (flags & FLAG_CACHE) and not (flags & FLAG_SINGLE) and nkv > 0 and qkv.shape[0] >= 64:
        count_launches(1)   # prompts: the values go through a second, transposing kernel


def silu_mul(gu: torch.Tensor, out: torch.Tensor):
    """out[t, i] = silu(gu[t, i]) * gu[t, I + i]."""
    _cuda(gu, out)
    inter = out.shape[-1]
    assert gu.shape[-1] == 2 * inter and gu.dtype == out.dtype and gu.is_contiguous() and out.is_contiguous()
    f = _fn("elementwise", "gb_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(gu.data_ptr(), out.data_ptr(), dtype_code(out.dtype), out.numel() // inter, inter, _stream()), "silu_mul",
           "elementwise", _nbytes(gu, out))


# --------------------------------------------------------------------------- matrix products

def gemm_ref(x, w, out, bias=None, accumulate=False):
    """out = x @ w.T (+ bias), or out += ... (float32 out) with ``accumulate``; CUDA cores, float32
    accumulation in ascending order of the inner index."""
    _cuda(x, w, out, bias)
    assert x.dtype == w.dtype and x.stride(-1) == 1 and out.stride(-1) == 1 and w.is_contiguous()
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    f = _fn("gemm_ref", "gb_gemm_ref",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong,
             c_longlong, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), dtype_code(x.dtype), _ptr(bias), out.data_ptr(), dtype_code(out.dtype),
             OUT_ACCUMULATE if accumulate else OUT_STORE, m, n, k, x.stride(0), out.stride(0), _stream()), "gemm_ref",
           "matmul", _nbytes(x, w, bias, out) * 1 + (_nbytes(out) if accumulate else 0))


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current CUDA device when None), read once per
    device: tile splits, persistent grids and the decode attention's share of the cache are sized
    by it, so a part with fewer SMs (or a slice of one) is neither oversubscribed nor left idle."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


_TC_MODES = {(torch.bfloat16, False): 0, (torch.float32, False): 1, (torch.float32, True): 2}


def gemm_tc_usable(x, w) -> bool:
    """Whether the tensor-core kernel takes these operands (TMA wants 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_tiling(m: int, n: int, k: int, gated: bool = False, sms: Optional[int] = None):
    """(tokens per tile, K splits) for an [m, k] x [n, k]^T product (``gated``: n features from
    2n rows, two accumulators per tile) on a device of ``sms`` multiprocessors (None: the current
    device's)."""
    sms = sms or sm_count()
    tiles_n = -(-n // 128)
    if m <= 64:
        bn = 16 if m <= 16 else (32 if m <= 32 else 64)
        tiles, kb = tiles_n, -(-k // 64)
        splits = 1
        # too few tiles to keep every SM streaming: split the inner dimension over a cluster, whose
        # ranks each add a share of the tile's tokens.  The CTAs wanted in all: two per SM for tiles of
        # 16 tokens, one per SM for wider tiles (every split sends all the tile's tokens' partial sums
        # once more through the cluster, which costs more the more tokens there are), about one per
        # SM for the gated product with 16 tokens and no split above that.  Measured with cold
        # weights at the layer sizes of 4B / 8B / 32B models (us, 1/2/4/8 splits):
        #  8 tokens: 6144x4096 22.6/15.4/13.6/12.8, 4096x12288 59/33/23/21, 10240x5120 28/23/21/24,
        #            gated 12288x4096 40/36/40/40, gated 25600x5120 82/86/86/95;
        # 32 tokens: 6144x2560 16/14/12/16, 6144x4096 23/17/16/18, 10240x5120 29/25/30/32,
        #            5120x8192 42/30/21/25, 5120x25600 121/72/51/58, 2560x4096 23/18/12/11;
        # 64 tokens: 6144x4096 23/20/18/23, 4096x4096 23/23/16/15, 10240x5120 30/29/34/39,
        #            5120x25600 122/83/58/63, gated 12288x4096 42/60/61/88.
        if gated:
            enough = sms + 2 if bn == 16 else 0
        else:
            enough = 2 * sms if bn == 16 else sms
        while splits < 8 and tiles * splits < enough and kb // (splits * 2) >= 4:
            splits *= 2
        return bn, splits
    best, best_score = 128, -1.0
    # a tile of 256 tokens runs the tensor pipe best; measured at 2,048 x 12,288 x 4,096 gated:
    # 384 us with 256-token tiles, 450 us with 128-token tiles
    for bn, tile_eff in ((256, 1.0), (128, 0.85 if gated else 0.92)):
        tiles = tiles_n * -(-m // bn)
        waves = -(-tiles // sms)
        fill = m / (-(-m // bn) * bn)
        score = tile_eff * fill * tiles / (waves * sms)
        if score > best_score:
            best, best_score = bn, score
    return best, 1


class UnscaledRows:
    """The input of an RMSNorm that is taken into the products around it (decode steps): ``rows``
    [tokens, width] = bfloat16(residual * the norm's weight), and ``partial`` [tiles, 64], the
    sums of squares of the residual's rows in tiles of 128 features, both left by the product
    that added into the residual.  The norm's output is rows * rstd, rstd[t] = (sum of
    partial[:, t] / width + eps) ** -0.5; the product that takes these rows applies rstd to its
    results instead (float32), so the norm needs no kernel of its own."""

    def __init__(self, rows, partial, eps: float, width: int):
        self.rows, self.partial, self.eps, self.width = rows, partial, float(eps), int(width)

    @property
    def shape(self):
        return self.rows.shape

    def materialize(self) -> torch.Tensor:
        """The norm's output as a plain tensor, for a consumer that cannot take unscaled rows."""
        m = self.rows.shape[0]
        rstd = (self.partial[:, :m].sum(0) / self.width + self.eps).rsqrt()
        return (self.rows.float() * rstd[:, None]).to(self.rows.dtype)


LINK_MAX_TOKENS = 64


def norm_link_usable(x, w, m: int, accumulate_splits: Optional[int] = None) -> bool:
    """Whether gemm_tc can take an RMSNorm into itself for these operands: at most 64 tokens on
    the tensor-core path; the product that leaves the rows must have its inner dimension split."""
    ok = m <= LINK_MAX_TOKENS and gemm_tc_usable(x, w)
    return ok and (accumulate_splits is None or accumulate_splits >= 2)


#: the builds of the product unit whose gated epilogue applies another activation than SiLU
GATED_ACT_DEFINES = {"silu": (), "gelu_tanh": (("GB_GATED_ACT", 1),)}


def gemm_tc(x, w, out, bias=None, accumulate=False, bn=None, splits=None, stages=4, swiglu=False, link_in=None,
            link_out=None, act="silu"):
    """out = x @ w.T (+ bias) (bfloat16 or float32 out) or out += ... (float32 out), bfloat16
    operands, on the tcgen05 tensor cores.  With ``swiglu``, w stacks a gate matrix over an up
    matrix ([2N, K]) and out[M, N] = silu(x @ gate.T) * (x @ up.T) in bfloat16.
    ``link_in``: an UnscaledRows whose ``rows`` are x: every token's results are scaled by its
    rstd.  ``link_out`` = (norm weight float32 [N], eps): with ``accumulate``, also leaves
    bfloat16(out * weight) and the sums of squares of out's rows, returned as UnscaledRows."""
    if link_in is not None:
        assert x is link_in.rows
    _cuda(x, w, out, bias)
    m, k = x.shape
    n = w.shape[0] // 2 if swiglu else w.shape[0]
    assert w.shape[1] == k and w.is_contiguous() and out.shape == (m, n) and out.stride(1) == 1
    if not gemm_tc_usable(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows (K and the row stride "
                          "multiples of 8)")
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate or bias is not None or w.shape[0] % 2:
            raise KernelError("gemm_tc: the gated product writes bfloat16, without bias, from an even number of rows")
        mode = 3
    else:
        mode = _TC_MODES.get((out.dtype, bool(accumulate)))
    if mode is None:
        raise KernelError(f"gemm_tc: cannot {'add into' if accumulate else 'store'} {out.dtype}")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    auto_bn, auto_splits = gemm_tc_tiling(m, n, k, gated=swiglu)
    if link_in is None and link_out is None:
        f = _fn("gemm_tc", "gb_gemm_tc",
                [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
                 c_int, c_int, c_void_p], GATED_ACT_DEFINES[act] if swiglu else ())
        _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, m, n, k, x.stride(0), out.stride(0),
                 bn or auto_bn, splits or auto_splits, stages, _stream()), "gemm_tc", "matmul",
               _nbytes(x, w, bias, out) + (_nbytes(out) if accumulate else 0))
        return None
    if m > LINK_MAX_TOKENS:
        raise KernelError(f"gemm_tc: a norm can be taken into the product for at most {LINK_MAX_TOKENS} tokens")
    left = None
    if link_out is not None:
        weight, eps = link_out
        if not accumulate or (splits or auto_splits) < 2:
            raise KernelError("gemm_tc: rows for a norm are left by a product that adds into the residual with its "
                              "inner dimension split")
        assert weight.dtype == torch.float32 and weight.numel() == n
        left = UnscaledRows(torch.empty((m, n), dtype=torch.bfloat16, device=x.device),
                            torch.empty((-(-n // 128), 64), dtype=torch.float32, device=x.device), eps, n)
    f = _fn("gemm_tc", "gb_gemm_tc_linked",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
             c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, m, n, k, x.stride(0), out.stride(0),
             bn or auto_bn, splits or auto_splits, stages,
             link_in.partial.data_ptr() if link_in is not None else None,
             link_in.partial.shape[0] if link_in is not None else 0, link_in.eps if link_in is not None else 0.0,
             link_in.width if link_in is not None else 0,
             link_out[0].data_ptr() if left is not None else None, left.rows.data_ptr() if left is not None else None,
             left.rows.stride(0) if left is not None else 0, left.partial.data_ptr() if left is not None else None,
             _stream()), "gemm_tc", "matmul",
           _nbytes(x, w, bias, out) + (_nbytes(out) if accumulate else 0) + (_nbytes(left.rows) if left is not None else 0))
    return left


_part_flags = {}
PERSISTENT_SPLIT_LAST_ROUND = True


def gemm_tc_persistent(x, w, out, bias=None, accumulate=False, swiglu=False, bn=None, ctas=None, split_last=None,
                       act="silu"):
    """The tensor-core product for prompts (more than 64 rows of x): one CTA per SM walks the output
    tiles, and the epilogue of a tile runs while the next tile's MMAs fill the other accumulator
    buffer.  Operands and modes as gemm_tc.  Where the last round of tiles would leave SMs idle, a
    product that adds into ``out`` cuts that round's tiles into parts along the inner dimension,
    which are added in a fixed order (``split_last=False``: never)."""
    if split_last is None:
        split_last = PERSISTENT_SPLIT_LAST_ROUND
    _cuda(x, w, out, bias)
    m, k = x.shape
    n = w.shape[0] // 2 if swiglu else w.shape[0]
    assert w.shape[1] == k and w.is_contiguous() and out.shape == (m, n) and out.stride(1) == 1
    if not gemm_tc_usable(x, w):
        raise KernelError("gemm_tc_persistent: operands must be bfloat16 with 16-byte aligned rows")
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate or bias is not None or w.shape[0] % 2:
            raise KernelError("gemm_tc_persistent: the gated product writes bfloat16, without bias")
        mode = 3
    else:
        mode = _TC_MODES.get((out.dtype, bool(accumulate)))
    if mode is None:
        raise KernelError(f"gemm_tc_persistent: cannot {'add into' if accumulate else 'store'} {out.dtype}")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    if bn is None:
        # 256 tokens a tile.  Narrower tiles that fill the last round of tiles better were measured and
        # are slower: 240 tokens for 2,048 x 4,096 (1.5 % faster alone, 4 % slower inside a prompt step),
        # and 128 tokens where 256 leave the last round nearly empty (2,048 x 2,560 is 160 tiles on 148
        # SMs; a 2,048-token prompt of a 4B-shaped model took 20.5 ms against 18.4, of a 32B-shaped one
        # 35.3 ms against 30.9 over 16 layers)
        bn = 128 if m <= 128 else 256
    ctas = ctas or sm_count(x.device)
    flags = None
    if accumulate and split_last:
        # a word per tile of the last round and epilogue warp; zero between launches
        flags = _part_flags.get(x.device.index)
        if flags is None or flags.numel() < 4 * ctas:
            if flags is not None:
                _outgrown.append(flags)       # a captured step may still point at it: never freed
            flags = _part_flags[x.device.index] = torch.zeros(max(4 * ctas, 1024), dtype=torch.int32, device=x.device)
    f = _fn("gemm_tc", "gb_gemm_tc_persistent",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
             c_int, c_void_p, c_void_p], GATED_ACT_DEFINES[act] if swiglu else ())
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, m, n, k, x.stride(0), out.stride(0), bn,
             ctas, _ptr(flags), _stream()), "gemm_tc_persistent", "matmul",
           _nbytes(x, w, bias, out) + (_nbytes(out) if accumulate else 0))


# measured inside replayed steps: +1.5 % tokens/s at batch 1 and 8 (8B layer sizes), even at batch 16
# (4B), -1.5 % at batch 24 (8B), -2.5 % at batch 32 (32B), -1 % at batch 64 (8B): a rank finishes
# its share of the tokens one after the other, three barriers each
QKV_FUSED_MAX_TOKENS = 16


QKV_KERNEL_MAX_TOKENS = 64     # what the kernel takes; the dispatch stops earlier, where it stops paying


def gemm_qkv_usable(x, w, nh: int, nkv: int, hd: int, rot: int, limit: Optional[int] = None) -> bool:
    """Whether the q/k/v product of a step can do the per-head work in its epilogue: a decode step
    in bfloat16 of at most ``limit`` tokens (None: as many as it pays for) with heads of 128 (a
    head is a tile of the product), rotated over all dims or not at all."""
    limit = QKV_FUSED_MAX_TOKENS if limit is None else limit
    return (x.dtype == torch.bfloat16 and x.shape[0] <= limit and hd == 128 and rot in (0, hd)
            and w.shape[0] == (nh + 2 * nkv) * hd and gemm_tc_usable(x, w))


def gemm_qkv(x, w, bias, qkv, nh, nkv, hd, q_weight, k_weight, eps, inv_freq, q_scale, tok_pos, tok_seq, seq_slot,
             page_table, page_size, kcache, vcache, bn=None, splits=None, link_in=None):
    """qkv[:, :nh*hd] = the step's queries, normed per head, rotated and scaled; the keys (normed,
    rotated) and the values go into the paged cache (``page_table`` None: into qkv as well): the
    q/k/v product and head_norm_rope_cache in one kernel.  See gemm_qkv_usable."""
    _cuda(x, w, bias, qkv, q_weight, k_weight, inv_freq, tok_pos, tok_seq, seq_slot, page_table, kcache, vcache)
    m, k = x.shape
    n = w.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.shape == (m, n) and qkv.stride(1) == 1 and w.is_contiguous()
    if not gemm_qkv_usable(x, w, nh, nkv, hd, hd if inv_freq is not None else 0, limit=QKV_KERNEL_MAX_TOKENS):
        raise KernelError(f"gemm_qkv: needs bfloat16, at most {QKV_KERNEL_MAX_TOKENS} tokens and heads of 128")
    if page_table is not None:
        assert kcache.dtype == torch.bfloat16 and kcache.is_contiguous() and kcache.shape[1:] == (nkv, page_size, hd)
        assert vcache.is_contiguous() and vcache.shape[1:] == (nkv, hd, page_size)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    auto_bn, auto_splits = gemm_tc_tiling(m, n, k)
    f = _fn("gemm_tc", "gb_gemm_tc_qkv",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p])
    if link_in is not None:
        assert x is link_in.rows
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), qkv.data_ptr(), m, n, k, x.stride(0), qkv.stride(0),
             bn or auto_bn, splits or auto_splits, _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), eps, q_scale, nh, nkv,
             tok_pos.data_ptr(), _ptr(tok_seq), _ptr(seq_slot), _ptr(page_table),
             page_table.shape[1] if page_table is not None else 1, page_size, _ptr(kcache), _ptr(vcache),
             link_in.partial.data_ptr() if link_in is not None else None,
             link_in.partial.shape[0] if link_in is not None else 0, link_in.eps if link_in is not None else 0.0,
             link_in.width if link_in is not None else 0, _stream()),
           "gemm_qkv", "matmul", _nbytes(x, w, bias, qkv))


def rope_table(tok_pos, inv_freq):
    """[tokens, half] pairs (cos, sin) of float32(position) * inv_freq, float32 [tokens, half, 2]:
    the angles of a step's packed tokens, computed once for all layers."""
    _cuda(tok_pos, inv_freq)
    assert tok_pos.dtype == torch.int32 and inv_freq.dtype == torch.float32
    ntok, half = tok_pos.numel(), inv_freq.numel()
    table = torch.empty((ntok, half, 2), dtype=torch.float32, device=tok_pos.device)
    f = _fn("gemm_tc", "gb_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(tok_pos.data_ptr(), inv_freq.data_ptr(), table.data_ptr(), ntok, half, _stream()), "rope_table",
           "elementwise", _nbytes(table))
    return table


def token_place(tok_pos, tok_seq, seq_slot, page_table, page_size):
    """int32 [tokens, 2]: (page, position in the page) of every packed token of a step in the cache
    that ``page_table`` describes; made once a step for all the layers that share the table."""
    _cuda(tok_pos, tok_seq, seq_slot, page_table)
    ntok = tok_pos.numel()
    place = torch.empty((ntok, 2), dtype=torch.int32, device=tok_pos.device)
    f = _fn("gemm_tc", "gb_token_place", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(f(tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), page_table.data_ptr(), page_table.shape[1],
             page_size, place.data_ptr(), ntok, _stream()), "token_place", "elementwise", _nbytes(place))
    return place


def gemm_qkv_prompt_usable(x, w, nh: int, nkv: int, hd: int, rot: int, page_size: int) -> bool:
    """Whether the q/k/v product of a prompt step can do the per-head work in its epilogue:
    bfloat16, more than 64 tokens, heads of 128 rotated over all dims or not at all."""
    return (x.dtype == torch.bfloat16 and x.shape[0] > 64 and hd == 128 and rot in (0, hd) and page_size % 8 == 0
            and w.shape[0] == (nh + 2 * nkv) * hd and gemm_tc_usable(x, w))


def gemm_qkv_prompt(x, w, bias, q_out, nh, nkv, hd, q_weight, k_weight, eps, table, q_scale, place, page_size, kcache,
                    vcache, ctas=None):
    """q_out[:, :nh*hd] = a prompt step's queries, normed per head, rotated and scaled; the keys
    (normed, rotated) and the values go into the paged cache: the q/k/v product of more than 64
    tokens and head_norm_rope_cache in one kernel.  ``table``: rope_table of the step's tokens
    (None: no rotation); ``place``: token_place of the step's tokens in this cache (None with no
    kv heads).  See gemm_qkv_prompt_usable."""
    _cuda(x, w, bias, q_out, q_weight, k_weight, table, place, kcache, vcache)
    m, k = x.shape
    n = w.shape[0]
    assert q_out.dtype == torch.bfloat16 and q_out.shape == (m, nh * hd) and q_out.stride(1) == 1 and w.is_contiguous()
    if not gemm_qkv_prompt_usable(x, w, nh, nkv, hd, hd if table is not None else 0, page_size):
        raise KernelError("gemm_qkv_prompt: needs bfloat16, more than 64 tokens and heads of 128")
    if nkv:
        assert kcache.dtype == torch.bfloat16 and kcache.is_contiguous() and kcache.shape[1:] == (nkv, page_size, hd)
        assert vcache.is_contiguous() and vcache.shape[1:] == (nkv, hd, page_size)
        assert place.dtype == torch.int32 and place.shape == (m, 2) and place.is_contiguous()
    if table is not None:
        assert table.dtype == torch.float32 and table.shape == (m, hd // 2, 2) and table.is_contiguous()
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    f = _fn("gemm_tc", "gb_gemm_tc_qkv_prompt",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p, c_void_p,
             c_void_p, c_float, c_float, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), q_out.data_ptr(), m, n, k, x.stride(0), q_out.stride(0),
             ctas or sm_count(x.device), _ptr(q_weight), _ptr(k_weight), _ptr(table), eps, q_scale, nh, nkv,
             _ptr(place) if nkv else None, page_size, _ptr(kcache), _ptr(vcache), _stream()),
           "gemm_qkv_prompt", "matmul", _nbytes(x, w, bias, q_out) + m * 2 * nkv * hd * 2)


# 65 to 128 tokens (decoding above batch 64): a CTA per tile of 128 features x 128 tokens with both
# accumulators, 96 CTAs at 8B layer sizes, takes 42 us with cold weights where the prompt kernel's
# 192 tiles of 64 features take 54 (30.8 us of bytes); above 128 tokens the prompt kernel is ahead.
GATED_TILE_128_MAX_TOKENS = 128


def gemm_swiglu(x, w_gate_up, out):
    """out[M, N] = silu(x @ gate.T) * (x @ up.T) for w_gate_up = [gate; up] of 2N rows: one
    tensor-core kernel in bfloat16; two kernels (product, then activation) otherwise.  ``x`` may
    be UnscaledRows (a norm taken into this product)."""
    link = x if isinstance(x, UnscaledRows) else None
    if link is not None:
        if norm_link_usable(link.rows, w_gate_up, link.rows.shape[0]):
            gemm_tc(link.rows, w_gate_up, out, swiglu=True, link_in=link)
            return
        x = link.materialize()
    if x.dtype == torch.bfloat16 and gemm_tc_usable(x, w_gate_up):
        if x.shape[0] > GATED_TILE_128_MAX_TOKENS:
            gemm_tc_persistent(x, w_gate_up, out, swiglu=True)
        elif x.shape[0] > 64:
            gemm_tc(x, w_gate_up, out, swiglu=True, bn=128, splits=1)
        else:
            gemm_tc(x, w_gate_up, out, swiglu=True)
        return
    gu = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
    gemm(x, w_gate_up, gu)
    silu_mul(gu, out)


def gemm_gated(x, w_gate_up, out, act: str = "silu"):
    """out = act(x @ gate.T) * (x @ up.T) for the stacked [gate; up], act one of GATED_ACTS: in
    bfloat16 one tensor-core kernel with the activation in its epilogue (a build of the product unit
    per activation); else the product followed by ``gated_act``."""
    if act == "silu":
        gemm_swiglu(x, w_gate_up, out)
        return
    if isinstance(x, UnscaledRows):
        x = x.materialize()
    if x.dtype == torch.bfloat16 and gemm_tc_usable(x, w_gate_up) and act in GATED_ACT_DEFINES:
        if x.shape[0] > GATED_TILE_128_MAX_TOKENS:
            gemm_tc_persistent(x, w_gate_up, out, swiglu=True, act=act)
        elif x.shape[0] > 64:
            gemm_tc(x, w_gate_up, out, swiglu=True, bn=128, splits=1, act=act)
        else:
            gemm_tc(x, w_gate_up, out, swiglu=True, act=act)
        return
    gu = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
    gemm(x, w_gate_up, gu)
    gated_act(gu, out, act)


def gated_units(compute: str, act: str):
    """The units ``gemm_gated`` may launch."""
    units = gemm_units(compute) + [("rows", ())]
    if compute == "bfloat16" and GATED_ACT_DEFINES.get(act):
        units.append(("gemm_tc", GATED_ACT_DEFINES[act]))
    return units


_STATUS_ENTRIES = ("gb_gemm_tc_status", "gb_attention_prefill_tc_status", "gb_attention_decode_stream_status")


def _status(entry: str, reset: bool) -> int:
    """First non-zero status word among the loaded libraries that export ``entry`` (every build of
    a unit keeps a word of its own)."""
    first = 0
    for lib in build.loaded().values():
        try:
            f = getattr(lib, entry)
        except AttributeError:
            continue
        f.argtypes, f.restype = [c_int], c_int
        v = f(1 if reset else 0)
        first = first or v
    return first


def gemm_tc_status(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in a gemm_tc launch (synchronizes)."""
    return _status("gb_gemm_tc_status", reset)


def check_status() -> None:
    """Raises if a bounded wait ran out in any tensor-core kernel since the last check: such a
    kernel gives up and leaves its output unfinished, so what was computed since must not be used.
    Synchronizes; the engine calls it before results leave it."""
    for entry in _STATUS_ENTRIES:
        v = _status(entry, True)
        if v:
            for flags in _part_flags.values():   # a kernel that gave up may have left a part's word set
                flags.zero_()
            raise KernelError(f"{entry[3:-7]}: a bounded wait ran out on the device (code {v}); "
                              "the results computed since the last check are not valid")


# --------------------------------------------------------------------------- attention

def attention_ref(q, out, nh, kcache, vcache, page_table, page_size, tok_pos, tok_seq, seq_slot, window=None, cache_bytes: int = 0):
    """Causal grouped-query attention of q [T, nh*hd] (row stride free) over the paged cache."""
    _cuda(q, out, kcache, vcache, page_table, tok_pos, tok_seq, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and q.dtype == out.dtype == kcache.dtype
    f = _fn("attention_ref", "gb_attention_ref",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), dtype_code(q.dtype), kcache.data_ptr(),
             vcache.data_ptr(), page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, tok_pos.data_ptr(),
             tok_seq.data_ptr(), seq_slot.data_ptr(), q.shape[0], nh, window or 0, _stream()), "attention_ref",
           "attention", _nbytes(q, out) + cache_bytes)


def decode_shares(ntok: int, nh: int, nkv: int, longest: int) -> int:
    """CTAs along the keys per (token, kv head) for the decode attention kernel: about one CTA per
    SM in all (a CTA's fixed work, loading q and merging its warps, is paid once per share; measured
    at 8,192 keys: 16 shares are best for one sequence, 2 for eight, 1 for sixty-four), and never
    so many that a warp is left without a 32-key block."""
    rep = nh // nkv
    chunks = -(-rep // 16)
    base = max(1, ntok * nkv * chunks)
    blocks = -(-max(longest, 1) // 32)
    want = (sm_count() + base // 2) // base
    return max(1, min(want, blocks // 8, 64))


def attention_decode(q, out, nh, kcache, vcache, page_table, page_size, tok_pos, tok_seq, seq_slot, window=None,
                     shares=1, scratch=None, cache_bytes: int = 0):
    """bfloat16 attention of single positions (one CTA per token, kv head and share of the keys)
    over the paged cache; the unit is compiled for the cache's head size."""
    _cuda(q, out, kcache, vcache, page_table, tok_pos, tok_seq, seq_slot, scratch)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    ntok = q.shape[0]
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    if shares > 1:
        need = ntok * nh * shares * (hd + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        assert scratch.dtype == torch.float32 and scratch.numel() >= need
    f = _fn("attention_decode", "gb_attention_decode",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
            defines=(("GB_HEAD_DIM", hd),))
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, tok_pos.data_ptr(), tok_seq.data_ptr(),
             seq_slot.data_ptr(), ntok, nh, window or 0, shares, _ptr(scratch), _stream()), "attention_decode",
           "attention", _nbytes(q, out) + cache_bytes)
    if shares > 1:
        count_launches(1)   # the merge kernel


STREAM_DECODE_HEAD_DIMS = (64, 128)
STREAM_DECODE_MAX_TOKENS = 4096
_decode_stream_scratch = {}
_outgrown = []


def attention_decode_stream_usable(ntok: int, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    return (hd in STREAM_DECODE_HEAD_DIMS and page_size == 64 and nh % nkv == 0 and nh // nkv <= 16
            and ntok <= STREAM_DECODE_MAX_TOKENS)


def attention_decode_stream(q, out, nh, kcache, vcache, page_table, page_size, tok_pos, tok_seq, seq_slot,
                            window=None, ctas=None, skip_slot=None, cache_bytes: int = 0):
    """bfloat16 attention of single positions with the cache streamed through shared memory by
    TMA: the pages that the step reads are dealt evenly to the CTAs as one flat list, whatever the
    lengths of the sequences; parts of a (token, kv head) that fall to different CTAs are added
    in key order by a second kernel.  Tokens of ``skip_slot`` (rows that pad a captured step) read
    nothing and get zeros."""
    _cuda(q, out, kcache, vcache, page_table, tok_pos, tok_seq, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    ntok = q.shape[0]
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    assert kcache.is_contiguous() and vcache.is_contiguous()
    if not attention_decode_stream_usable(ntok, nh, nkv, hd, page_size):
        raise KernelError(f"attention_decode_stream: head size {hd} (64 or 128), page size {page_size} (64), "
                          f"{nh // max(nkv, 1)} query heads per kv head (at most 16) or {ntok} tokens "
                          f"(at most {STREAM_DECODE_MAX_TOKENS}) not supported")
    defines = (("GB_HEAD_DIM", hd),)
    sig = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int,
           c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    f = _fn("attention_decode_stream", "gb_attention_decode_stream", sig, defines=defines)
    if ctas is None:
        ctas = sm_count(q.device)   # one per SM; measured at 8,192 keys, batch 1 / 8 / 64: 17 / 54 / 323 us; two per SM: 24 / 58 / 329
    need = ctas * 2 * (nh // nkv) * (hd + 2) + ntok + 1
    scratch = _decode_stream_scratch.get(q.device.index)
    if scratch is None or scratch.numel() < need:
        if scratch is not None:
            _outgrown.append(scratch)     # a captured step may still point at it: never freed
        scratch = _decode_stream_scratch[q.device.index] = torch.empty(max(need, 1 << 20), dtype=torch.float32,
                                                                       device=q.device)
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             kcache.shape[0], page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, tok_pos.data_ptr(),
             tok_seq.data_ptr(), seq_slot.data_ptr(), ntok, nh, window or 0, -1 if skip_slot is None else skip_slot,
             ctas, scratch.data_ptr(), _stream()),
           "attention_decode_stream", "attention", _nbytes(q, out) + cache_bytes)
    count_launches(1)   # the merge kernel


def attention_decode_stream_status(reset: bool = True) -> int:
    return _status("gb_attention_decode_stream_status", reset)


def attention_prefill(q, out, nh, kcache, vcache, page_table, page_size, cu_seqlens, seq_start, seq_slot, window=None, cache_bytes: int = 0):
    """bfloat16 causal attention of packed prompt tokens (sequence b owns tokens cu_seqlens[b] to
    cu_seqlens[b + 1], at positions from seq_start[b]) over the paged cache, which already holds
    the step's own keys and values."""
    _cuda(q, out, kcache, vcache, page_table, cu_seqlens, seq_start, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    f = _fn("attention_prefill", "gb_attention_prefill",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
            defines=(("GB_HEAD_DIM", hd),))
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, cu_seqlens.data_ptr(),
             seq_start.data_ptr(), seq_slot.data_ptr(), seq_slot.numel(), q.shape[0], nh, window or 0, _stream()),
           "attention_prefill", "attention", _nbytes(q, out) + cache_bytes)


TC_PREFILL_HEAD_DIMS = (64, 128)


def attention_prefill_tc(q, out, nh, kcache, vcache, page_table, page_size, cu_seqlens, seq_start, seq_slot,
                         window=None, cache_bytes: int = 0):
    """As attention_prefill, on the tcgen05 tensor cores (TMA-fed, S and O in tensor memory); head
    sizes 64 and 128."""
    _cuda(q, out, kcache, vcache, page_table, cu_seqlens, seq_start, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    if hd not in TC_PREFILL_HEAD_DIMS:
        raise KernelError(f"attention_prefill_tc: head size {hd} is not supported (64 or 128)")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[0] == vcache.shape[0]
    f = _fn("attention_prefill_tc", "gb_attention_prefill_tc",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int,
             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
            defines=(("GB_HEAD_DIM", hd),))
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             kcache.shape[0], page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, cu_seqlens.data_ptr(),
             seq_start.data_ptr(), seq_slot.data_ptr(), seq_slot.numel(), q.shape[0], nh, window or 0, _stream()),
           "attention_prefill_tc", "attention", _nbytes(q, out) + cache_bytes)


def attention_prefill_tc_status(head_dim: int = 0, reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in attention_prefill_tc (synchronizes)."""
    return _status("gb_attention_prefill_tc_status", reset)


# --------------------------------------------------------------------------- latent attention

def latent_prepare(q_in, kv_in, g_in, norm_w, eps, inv_freq, rot, q_scale, q_nope, q_lat, gate, cache, page_table,
                   page_size, tok_pos, tok_seq, seq_slot, heads, dim, rd, rank, dense=None):
    """From the float32 projections of a latent attention layer: the cache row of every token
    (RMS-normed latent ``kv_in[:, :rank]``, then the key part ``kv_in[:, rank:]`` with its first
    ``rot`` dims rotated as interleaved pairs) into the paged ``cache`` [pages, page_size, rank + rd];
    the queries' unrotated dims times ``q_scale`` into ``q_nope`` [T, heads * dim], their rotated
    dims (rotated, scaled) into the last ``rd`` columns of each head of ``q_lat``
    [T, heads * (rank + rd)]; ``gate`` [T, heads] = sigmoid(g_in) (float32; None: no gate).  ``dense``
    [T, rank + rd] (None: not wanted) receives the same rows as the cache, token by token."""
    _cuda(q_in, kv_in, g_in, norm_w, inv_freq, q_nope, q_lat, gate, cache, page_table, tok_pos, tok_seq, seq_slot)
    t = q_in.shape[0]
    assert q_in.dtype == torch.float32 and kv_in.dtype == torch.float32 and q_in.stride(1) == 1 and kv_in.stride(1) == 1
    assert q_in.shape[1] == heads * (dim + rd) and kv_in.shape == (t, rank + rd) and norm_w.numel() == rank
    assert q_nope.shape == (t, heads * dim) and q_lat.shape == (t, heads * (rank + rd)) and q_nope.dtype == q_lat.dtype
    assert q_nope.stride(1) == 1 and q_lat.stride(1) == 1 and norm_w.dtype == torch.float32
    if g_in is not None:
        assert g_in.dtype == torch.float32 and g_in.shape == (t, heads) and g_in.stride(1) == 1
        assert gate.dtype == torch.float32 and gate.shape == (t, heads) and gate.is_contiguous()
    if cache is not None:
        assert cache.dtype == q_lat.dtype and cache.is_contiguous() and cache.shape[-2:] == (page_size, rank + rd)
    if rot:
        assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rot // 2
    f = _fn("latent_attention", "gb_latent_prepare",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_float, c_void_p, c_int, c_float,
             c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_void_p])
    if dense is not None:
        assert dense.dtype == q_lat.dtype and dense.shape == (t, rank + rd) and dense.stride(1) == 1
    _check(f(q_in.data_ptr(), q_in.stride(0), kv_in.data_ptr(), kv_in.stride(0), _ptr(g_in),
             g_in.stride(0) if g_in is not None else 0, norm_w.data_ptr(), eps, _ptr(inv_freq), rot, q_scale,
             q_nope.data_ptr(), q_nope.stride(0), q_lat.data_ptr(), q_lat.stride(0), _ptr(gate), _ptr(cache),
             dtype_code(q_lat.dtype), _ptr(page_table), page_table.shape[1] if page_table is not None else 1, page_size,
             tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), t, heads, dim, rd, rank, _ptr(dense),
             dense.stride(0) if dense is not None else 0, _stream()),
           "latent_prepare", "elementwise", _nbytes(q_in, kv_in, q_nope) + t * (rank + 2 * rd) * q_lat.element_size())


def heads_gemm(x, w, y, heads, scale=None):
    """y[t, h, :] = scale[t, h] * w[h] @ x[t, h, :] for every head: x [T, heads, K] and y [T, heads, N]
    as views of 2-D tensors (the head stride may be wider than K or N), w [heads, N, K] contiguous,
    scale float32 [T, heads] or None.  Float32 accumulation in ascending k."""
    _cuda(x, w, y, scale)
    t, _, k = x.shape
    n = w.shape[1]
    assert x.shape[1] == heads and w.shape == (heads, n, k) and y.shape == (t, heads, n) and w.is_contiguous()
    assert x.stride(2) == 1 and y.stride(2) == 1 and x.dtype == w.dtype == y.dtype
    if scale is not None:
        assert scale.dtype == torch.float32 and scale.shape == (t, heads) and scale.is_contiguous()
    if (x.dtype == torch.bfloat16 and k % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0
            and x.data_ptr() % 16 == 0 and t >= HEADS_GEMM_TC_MIN_TOKENS):
        grouped_gemm(x, x.stride(0), x.stride(1), None, 1, w, n * k, y, y.stride(0), y.stride(1), scale, None, heads, 1,
                     None, heads, t, t, n, k, what="heads_gemm_tc", nbytes=_nbytes(w) + t * heads * (n + k) * 2)
        return
    f = _fn("latent_attention", "gb_heads_gemm",
            [c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), x.stride(1), w.data_ptr(), y.data_ptr(), y.stride(0), y.stride(1), _ptr(scale),
             dtype_code(x.dtype), t, heads, n, k, _stream()), "heads_gemm", "matmul",
           _nbytes(w) + t * heads * (n + k) * x.element_size())


# the tensor-core kernel from the first token on: inside a replayed decode step of 8 tokens the FFMA
# kernel took 20 and 58 us for the two products of a layer (16 heads, 128 -> 512 and 512 -> 128), one
# scalar load per element and 64 x 16 blocks in turn; a nearly empty 128-row tile costs nothing here
HEADS_GEMM_TC_MIN_TOKENS = 1


def grouped_gemm(a, lda, a_gstride, a_rows, a_div, w, w_gstride, c, ldc, c_gstride, scale, scale_rows, s_rstride, s_gstride,
                 offsets, groups, rows, max_rows, n, k, gated=False, limit=0.0, alpha=0.0, shift=0.0, what="grouped_gemm",
                 nbytes=0):
    """Many bfloat16 products C_g = A_g W_g^T of unequal row counts in one tensor-core launch (see
    csrc/grouped_gemm.cu): group g's rows are offsets[g]..offsets[g+1] (None: ``rows`` each), an A
    row is a_rows[i] // a_div (None: i), C is bfloat16 or float32 by its dtype; ``gated``: W_g stacks
    gate rows over up rows and C = min(g, limit) * sigmoid(alpha g) * (clamp(u) + shift); ``gated`` 2:
    no gate rows, C = gelu(A W_g^T) in the exact (erf) form."""
    _cuda(a, w, c, scale, scale_rows, offsets, a_rows)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and c.dtype in (torch.bfloat16, torch.float32)
    f = _fn("grouped_gemm", "gb_grouped_gemm",
            [c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_longlong,
             c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
             c_float, c_float, c_void_p])
    _check(f(a.data_ptr(), lda, a_gstride, _ptr(a_rows), a_div, w.data_ptr(), w_gstride, c.data_ptr(), ldc, c_gstride,
             _ptr(scale), _ptr(scale_rows), s_rstride, s_gstride, _ptr(offsets), groups, rows, max_rows, n, k,
             int(gated), 1 if c.dtype == torch.float32 else 0, limit, alpha, shift, _stream()), what, "matmul", nbytes)


def latent_attention_ref(qa, out, heads, rank, rd, cache, page_table, page_size, tok_pos, tok_seq, seq_slot, window=None,
                         cache_bytes: int = 0):
    """Causal attention of the absorbed queries qa [T, heads * (rank + rd)] over the cached rows
    [pages, page_size, rank + rd]; out [T, heads * rank] = the softmax-weighted sums of the rows'
    first ``rank`` dims.  One block per (token, head), float32 arithmetic, any precision."""
    _cuda(qa, out, cache, page_table, tok_pos, tok_seq, seq_slot)
    assert qa.stride(-1) == 1 and out.stride(-1) == 1 and qa.dtype == out.dtype == cache.dtype and cache.is_contiguous()
    assert qa.shape[1] == heads * (rank + rd) and out.shape[1] == heads * rank and cache.shape[-1] == rank + rd
    f = _fn("latent_attention", "gb_latent_attention_ref",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(qa.data_ptr(), qa.stride(0), out.data_ptr(), out.stride(0), dtype_code(qa.dtype), cache.data_ptr(),
             page_table.data_ptr(), page_table.shape[1], page_size, tok_pos.data_ptr(), tok_seq.data_ptr(),
             seq_slot.data_ptr(), qa.shape[0], heads, rank, rd, window or 0, _stream()), "latent_attention_ref",
           "attention", _nbytes(qa, out) + cache_bytes)


def rope_pairs(x, tok_pos, inv_freq, rot):
    """Rotates, in place, the first ``rot`` dims of every head of x [T, heads, hd] as interleaved
    pairs (2i, 2i + 1) by the angle float32(position) * inv_freq[i]."""
    _cuda(x, tok_pos, inv_freq)
    t, heads, hd = x.shape
    assert x.stride(2) == 1 and x.stride(1) == hd and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot // 2
    f = _fn("latent_attention", "gb_rope_pairs", [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                                  c_int, c_void_p])
    _check(f(x.data_ptr(), x.stride(0), dtype_code(x.dtype), tok_pos.data_ptr(), inv_freq.data_ptr(), t, heads, hd, rot,
             _stream()), "rope_pairs", "elementwise", 2 * t * heads * rot * x.element_size())


def latent_attention_mma_usable(dtype, rank: int, rd: int, page_size: int) -> bool:
    """Whether the tensor-core kernel takes these sizes: bfloat16, the latent and the rotated part
    multiples of 16 (the latent a multiple of 32 above 128 and of 64 above 256, up to 512: its
    columns are dealt to 2 or 4 warps), pages of 64."""
    if dtype != torch.bfloat16 or page_size != 64 or rank % 16 or rd % 16 or not 16 <= rank <= 512:
        return False
    return rank % (16 if rank <= 128 else (32 if rank <= 256 else 64)) == 0


_latent_scratch = {}


def latent_attention_mma(qa, out, heads, rank, rd, cache, page_table, page_size, cu_seqlens, seq_start, seq_slot,
                         max_new: int, window=None, ksplits: int = 1, cache_bytes: int = 0, head_stride: int = 0,
                         out_scale=None):
    """bfloat16 latent attention on the tensor cores (mma.sync) for packed sequences that bring any
    number of tokens each; with ``ksplits`` > 1 the keys of a tile of rows are dealt to that many
    CTAs and a second kernel adds their parts.  ``head_stride`` > 0: every head has rows of its own,
    ``cache`` [heads, packed tokens + 64, rank + rd] (elements ``head_stride`` apart), a sequence's rows
    from its first packed token on, every sequence from position 0, no page table; ``out_scale``
    float32 [T, heads] multiplies the output."""
    _cuda(qa, out, cache, page_table, cu_seqlens, seq_start, seq_slot, out_scale)
    if not latent_attention_mma_usable(qa.dtype, rank, rd, page_size):
        raise KernelError(f"latent_attention_mma: latent {rank} + {rd}, pages of {page_size} or {qa.dtype} not supported")
    assert qa.stride(-1) == 1 and out.stride(-1) == 1 and out.dtype == cache.dtype == torch.bfloat16 and cache.is_contiguous()
    assert qa.shape[1] == heads * (rank + rd) and out.shape[1] == heads * rank and cache.shape[-1] == rank + rd
    ntok = qa.shape[0]
    if head_stride:
        assert ksplits == 1 and cache.shape[0] == heads and cache.shape[1] >= ntok + 64 and head_stride == cache.stride(0)
    defines = (("GB_LATENT_RANK", rank), ("GB_LATENT_ROT", rd))
    part = None
    if ksplits > 1:
        need = ntok * heads * ksplits * (rank + 4)
        part = _latent_scratch.get(qa.device.index)
        if part is None or part.numel() < need:
            if part is not None:
                _outgrown.append(part)        # a captured step may still point at it: never freed
            part = _latent_scratch[qa.device.index] = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=qa.device)
    f = _fn("latent_attention_mma", "gb_latent_attention_mma",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_longlong, c_void_p, c_void_p], defines=defines)
    _check(f(qa.data_ptr(), qa.stride(0), out.data_ptr(), out.stride(0), _ptr(part), cache.data_ptr(), _ptr(page_table),
             page_table.shape[1] if page_table is not None else 1, page_size, cu_seqlens.data_ptr(), seq_start.data_ptr(),
             seq_slot.data_ptr(), seq_slot.numel(), ntok, heads, rank, rd, max_new * (1 if head_stride else heads),
             window or 0, ksplits, head_stride, _ptr(out_scale), _stream()),
           "latent_attention_mma", "attention", _nbytes(qa, out) + cache_bytes)
    if ksplits > 1:
        count_launches(1)   # the merge kernel


def latent_decode_splits(n_seqs: int, heads: int) -> int:
    """CTAs along the keys for each sequence of a decode step: about two CTAs per SM in all (a CTA is
    one group of 16 rows, few warps; two to an SM hide each other's waits)."""
    tiles = n_seqs * -(-heads // 32)
    return max(1, min(64, (2 * sm_count()) // max(tiles, 1)))


def latent_attention(ctx, qa, out, heads, rank, rd, cache, page_table, page_size, window=None):
    """Latent attention of the step's queries over the cache; picks the kernel for the precision
    and the sizes.  float32 always takes the plain kernel, whose arithmetic for a position does not
    depend on the batch; so do sizes the tensor-core kernel does not take."""
    cached = 0
    if _profile["on"] and ctx.host is not None:
        per_pos = (rank + rd) * cache.element_size()
        for start, n in zip(ctx.host["seq_start"], ctx.host["seq_len"]):
            cached += per_pos * (min(start + n, window + n - 1) if window else start + n)
    if latent_attention_mma_usable(qa.dtype, rank, rd, page_size) and qa.stride(0) % 8 == 0:
        ksplits = latent_decode_splits(ctx.n_seqs, heads) if ctx.max_new <= 1 else 1
        latent_attention_mma(qa, out, heads, rank, rd, cache, page_table, page_size, ctx.cu_seqlens, ctx.seq_start,
                             ctx.seq_slot, ctx.max_new, window, ksplits, cache_bytes=cached)
        return
    latent_attention_ref(qa, out, heads, rank, rd, cache, page_table, page_size, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                         window, cache_bytes=cached)


# prompt steps of at least this many tokens whose sequences all start at position 0 expand keys and
# values per head and run attention over heads of dim + rot_dim with values of vdim, instead of over
# the latent rows: (2 rank + rot_dim) / (2 vdim + dim + rot_dim) times less arithmetic
LATENT_EXPAND_MIN_TOKENS = 256


def latent_expand_usable(dtype, rank: int, dim: int, rd: int, vd: int) -> bool:
    """Whether a prompt step may run attention over expanded heads: the same kernel with the value
    in front of the key ([v | k_nope | k_rot] rows, so vdim plays the latent and dim + rot_dim the
    rest), rows the grouped product can write, and an expansion that saves arithmetic."""
    return (latent_attention_mma_usable(dtype, vd, dim + rd, 64) and rank % 8 == 0 and rd % 8 == 0 and dim > 0
            and 2 * vd + dim + rd < 2 * rank + rd)


def latent_attention_units(compute: str, rank: int, rd: int, dim: int = 0, vd: int = 0):
    units = [("latent_attention", ())]
    if compute != "float32" and latent_attention_mma_usable(torch.bfloat16, rank, rd, 64):
        units.append(("latent_attention_mma", (("GB_LATENT_RANK", rank), ("GB_LATENT_ROT", rd))))
    if compute != "float32" and vd and latent_expand_usable(torch.bfloat16, rank, dim, rd, vd):
        units.append(("latent_attention_mma", (("GB_LATENT_RANK", vd), ("GB_LATENT_ROT", dim + rd))))
    return units


# --------------------------------------------------------------------------- routed feed-forward

def moe_topk(z, bias, experts, top, has_gate=False, all_softmax=False):
    """(idx int32 [T, top], weights float32 [T, top], shared float32 [T] or None) from the router's
    logits z (float32 [T, experts (+ 1)]): each token's ``top`` largest z + bias (the lower index wins
    a tie), the softmax over those alone (with ``all_softmax``: their shares of the softmax over all
    experts, which do not add up to one), and with ``has_gate`` the sigmoid of column ``experts``."""
    _cuda(z, bias)
    t = z.shape[0]
    assert z.dtype == torch.float32 and z.stride(1) == 1 and z.shape[1] >= experts + (1 if has_gate else 0)
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == experts)
    idx = torch.empty((t, top), dtype=torch.int32, device=z.device)
    wts = torch.empty((t, top), dtype=torch.float32, device=z.device)
    sg = torch.empty((t,), dtype=torch.float32, device=z.device) if has_gate else None
    f = _fn("moe", "gb_moe_topk_mode", [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_int, c_void_p])
    _check(f(z.data_ptr(), z.stride(0), _ptr(bias), idx.data_ptr(), wts.data_ptr(), _ptr(sg), t, experts, top,
             1 if has_gate else 0, 1 if all_softmax else 0, _stream()), "moe_topk", "elementwise", _nbytes(z))
    return idx, wts, sg


def moe_experts(h, idx, wts, sg, w_gate_up, w_down, shared_gate_up, shared_down, residual, limit, shared_limit, alpha,
                shift):
    """residual[t] += sum_k wts[t, k] * expert_{idx[t, k]}(h[t]) + sg[t] * shared(h[t]), token-major
    (two kernels: gate/up with the activation, then down).  w_gate_up [E, 2 ff, width] (gate rows,
    then up rows), w_down [E, width, ff]; the shared expert's [2 ffs, width] and [width, ffs], or None."""
    _cuda(h, idx, wts, sg, w_gate_up, w_down, shared_gate_up, shared_down, residual)
    t, width = h.shape
    e, ff2, _ = w_gate_up.shape
    ff = ff2 // 2
    top = idx.shape[1]
    ffs = shared_down.shape[1] if shared_down is not None else 0
    assert w_gate_up.is_contiguous() and w_down.is_contiguous() and w_down.shape == (e, width, ff)
    assert w_gate_up.dtype == h.dtype == w_down.dtype and residual.dtype == torch.float32 and residual.stride(1) == 1
    assert (shared_gate_up is None) == (shared_down is None) == (sg is None)
    if shared_down is not None:
        assert shared_gate_up.shape == (2 * ffs, width) and shared_gate_up.is_contiguous() and shared_down.is_contiguous()
    slots = top + (1 if shared_down is not None else 0)
    y = torch.empty((t, slots, max(ff, ffs)), dtype=h.dtype, device=h.device)
    f = _fn("moe", "gb_moe_gate_up", [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                      c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_void_p])
    _check(f(h.data_ptr(), h.stride(0), dtype_code(h.dtype), idx.data_ptr(), w_gate_up.data_ptr(), _ptr(shared_gate_up),
             y.data_ptr(), t, width, ff, ffs, top, limit, shared_limit, alpha, shift, _stream()), "moe_gate_up", "matmul",
           _nbytes(h, y) + t * slots * 2 * ff * width * h.element_size())
    rows = torch.empty((t, slots, width), dtype=torch.float32, device=h.device)
    f = _fn("moe", "gb_moe_down", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(y.data_ptr(), dtype_code(h.dtype), idx.data_ptr(), wts.data_ptr(), _ptr(sg), w_down.data_ptr(),
             _ptr(shared_down), rows.data_ptr(), residual.data_ptr(), residual.stride(0), t, width, ff, ffs, top, _stream()),
           "moe_down", "matmul", _nbytes(y) + 2 * _nbytes(rows) + 2 * t * width * 4 + t * slots * ff * width * h.element_size())
    count_launches(1)   # the kernel that adds a token's rows


def moe_experts_plain(h, idx, wts, w_up, w_down, residual):
    """residual[t] += sum_k wts[t, k] * down_{idx[t, k]} gelu(up_{idx[t, k]} h[t]) for experts without a
    gate (exact GELU), token-major.  w_up [E, ff, width], w_down [E, width, ff]."""
    _cuda(h, idx, wts, w_up, w_down, residual)
    t, width = h.shape
    e, ff, _ = w_up.shape
    top = idx.shape[1]
    assert w_up.is_contiguous() and w_down.is_contiguous() and w_down.shape == (e, width, ff) and w_up.shape[2] == width
    assert w_up.dtype == h.dtype == w_down.dtype and residual.dtype == torch.float32 and residual.stride(1) == 1
    y = torch.empty((t, top, ff), dtype=h.dtype, device=h.device)
    f = _fn("moe", "gb_moe_up", [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(h.data_ptr(), h.stride(0), dtype_code(h.dtype), idx.data_ptr(), w_up.data_ptr(), y.data_ptr(), t, width, ff, top,
             _stream()), "moe_up", "matmul", _nbytes(h, y) + t * top * ff * width * h.element_size())
    rows = torch.empty((t, top, width), dtype=torch.float32, device=h.device)
    f = _fn("moe", "gb_moe_down", [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_longlong, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(y.data_ptr(), dtype_code(h.dtype), idx.data_ptr(), wts.data_ptr(), None, w_down.data_ptr(), None,
             rows.data_ptr(), residual.data_ptr(), residual.stride(0), t, width, ff, 0, top, _stream()),
           "moe_down", "matmul", _nbytes(y) + 2 * _nbytes(rows) + 2 * t * width * 4 + t * top * ff * width * h.element_size())
    count_launches(1)   # the kernel that adds a token's rows


def moe_experts_plain_grouped(h, idx, wts, w_up, w_down, residual):
    """As moe_experts_plain for a step of many tokens: entries ordered by expert, two grouped
    tensor-core products (up with the GELU in its epilogue, down scaled by the routing weights), a
    token's rows added into the residual in slot order."""
    _cuda(h, idx, wts, w_up, w_down, residual)
    t, width = h.shape
    e, ff, _ = w_up.shape
    top = idx.shape[1]
    entries = t * top
    assert residual.dtype == torch.float32 and residual.stride(1) == 1 and idx.is_contiguous() and wts.is_contiguous()
    meta = torch.empty(e + 1 + 2 * entries, dtype=torch.int32, device=h.device)
    offsets, perm, place = meta[:e + 1], meta[e + 1:e + 1 + entries], meta[e + 1 + entries:]
    f = _fn("grouped_gemm", "gb_moe_sort", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(idx.data_ptr(), entries, e, offsets.data_ptr(), perm.data_ptr(), place.data_ptr(), _stream()), "moe_sort",
           "elementwise", 3 * entries * 4)
    y = torch.empty((entries, ff), dtype=torch.bfloat16, device=h.device)
    grouped_gemm(h, h.stride(0), 0, perm, top, w_up, ff * width, y, ff, 0, None, None, 0, 0, offsets, e, 0, entries,
                 ff, width, gated=2, what="moe_up_tc", nbytes=_nbytes(w_up, y) + entries * width * 2)
    rows = torch.empty((entries, width), dtype=torch.float32, device=h.device)
    grouped_gemm(y, ff, 0, None, 1, w_down, width * ff, rows, width, 0, wts.view(-1), perm, 1, 0, offsets, e, 0, entries,
                 width, ff, what="moe_down_tc", nbytes=_nbytes(w_down, y, rows))
    f = _fn("grouped_gemm", "gb_moe_combine", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(rows.data_ptr(), place.data_ptr(), residual.data_ptr(), residual.stride(0), t, width, top, _stream()),
           "moe_combine", "elementwise", _nbytes(rows) + 2 * t * width * 4)


def moe_experts_plain_tc(h, idx, wts, w_up, w_down, residual):
    """As moe_experts_plain_grouped for a prompt step, the two products on the tcgen05 kernel (the
    activations copied into an order in which every expert's rows start at a multiple of the
    tile's tokens; the GELU and the routing weight in the first product's epilogue)."""
    _cuda(h, idx, wts, w_up, w_down, residual)
    t, width = h.shape
    e, ff, _ = w_up.shape
    top, bn = idx.shape[1], MOE_TC_TILE
    entries = t * top
    rows = (-(-entries // bn) + e) * bn
    meta = torch.empty(rows // bn + entries + rows, dtype=torch.int32, device=h.device)
    tile_expert, place, row_entry = meta[:rows // bn], meta[rows // bn:rows // bn + entries], meta[rows // bn + entries:]
    f = _fn("grouped_gemm", "gb_moe_sort_padded", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(idx.data_ptr(), entries, e, bn, rows, tile_expert.data_ptr(), place.data_ptr(), row_entry.data_ptr(), _stream()),
           "moe_sort", "elementwise", 3 * entries * 4)
    xp = torch.empty((rows, width), dtype=torch.bfloat16, device=h.device)
    scale = torch.empty((rows,), dtype=torch.float32, device=h.device)
    f = _fn("grouped_gemm", "gb_moe_permute", [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                               c_int, c_int, c_int, c_void_p])
    _check(f(h.data_ptr(), h.stride(0), row_entry.data_ptr(), tile_expert.data_ptr(), wts.data_ptr(), xp.data_ptr(),
             scale.data_ptr(), rows, width, top, bn, _stream()), "moe_permute", "elementwise", 2 * entries * width * 2)
    y = torch.empty((rows, ff), dtype=torch.bfloat16, device=h.device)
    gemm_tc_grouped(xp, w_up.view(e * ff, width), y, ff, e, tile_expert, scale, gelu=True)
    out = torch.empty((rows, width), dtype=torch.float32, device=h.device)
    gemm_tc_grouped(y, w_down.view(e * width, ff), out, width, e, tile_expert)
    f = _fn("grouped_gemm", "gb_moe_combine", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(out.data_ptr(), place.data_ptr(), residual.data_ptr(), residual.stride(0), t, width, top, _stream()),
           "moe_combine", "elementwise", entries * width * 4 + 2 * t * width * 4)


MOE_GROUPED_MIN_TOKENS = 16


def moe_grouped_usable(h, w_gate_up, w_down) -> bool:
    """Whether a step's experts run as grouped tensor-core products: bfloat16, enough tokens that
    experts are shared between them, rows that cp.async can bring in 16-byte pieces."""
    return (h.dtype == torch.bfloat16 and h.shape[0] >= MOE_GROUPED_MIN_TOKENS and h.shape[1] % 8 == 0
            and w_down.shape[2] % 8 == 0 and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0)


def moe_experts_grouped(h, idx, wts, sg, w_gate_up, w_down, shared_gate_up, shared_down, residual, limit, shared_limit,
                        alpha, shift):
    """As moe_experts for a step of many tokens: the (token, slot) entries are ordered by expert on the
    device, each expert's rows run as one product of a grouped tensor-core launch (gate/up with the
    activation, then down scaled by the routing weights), a token's rows are added into the residual
    in slot order, and the shared expert runs as dense products over all tokens."""
    _cuda(h, idx, wts, sg, w_gate_up, w_down, shared_gate_up, shared_down, residual)
    t, width = h.shape
    e, ff2, _ = w_gate_up.shape
    ff, top = ff2 // 2, idx.shape[1]
    entries = t * top
    assert residual.dtype == torch.float32 and residual.stride(1) == 1 and idx.is_contiguous() and wts.is_contiguous()
    meta = torch.empty(e + 1 + 2 * entries, dtype=torch.int32, device=h.device)
    offsets, perm, place = meta[:e + 1], meta[e + 1:e + 1 + entries], meta[e + 1 + entries:]
    f = _fn("grouped_gemm", "gb_moe_sort", [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(idx.data_ptr(), entries, e, offsets.data_ptr(), perm.data_ptr(), place.data_ptr(), _stream()), "moe_sort",
           "elementwise", 3 * entries * 4)
    y = torch.empty((entries, ff), dtype=torch.bfloat16, device=h.device)
    grouped_gemm(h, h.stride(0), 0, perm, top, w_gate_up, ff2 * width, y, ff, 0, None, None, 0, 0, offsets, e, 0, entries,
                 ff, width, gated=True, limit=limit, alpha=alpha, shift=shift, what="moe_gate_up_tc",
                 nbytes=_nbytes(w_gate_up, y) + entries * width * 2)
    rows = torch.empty((entries, width), dtype=torch.float32, device=h.device)
    grouped_gemm(y, ff, 0, None, 1, w_down, width * ff, rows, width, 0, wts.view(-1), perm, 1, 0, offsets, e, 0, entries,
                 width, ff, what="moe_down_tc", nbytes=_nbytes(w_down, y, rows))
    f = _fn("grouped_gemm", "gb_moe_combine", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(rows.data_ptr(), place.data_ptr(), residual.data_ptr(), residual.stride(0), t, width, top, _stream()),
           "moe_combine", "elementwise", _nbytes(rows) + 2 * t * width * 4)
    _shared_expert(h, sg, shared_gate_up, shared_down, residual, shared_limit, alpha, shift)


MOE_TC_MIN_TOKENS = 256
MOE_TC_TILE = 128


def moe_tc_usable(h, w_gate_up, w_down) -> bool:
    """Whether a step's experts run on the tcgen05 product: a prompt's worth of tokens, operands the
    product's TMA loads can address."""
    return (moe_grouped_usable(h, w_gate_up, w_down) and h.shape[0] >= MOE_TC_MIN_TOKENS
            and w_gate_up.data_ptr() % 16 == 0 and w_down.data_ptr() % 16 == 0)


def gemm_tc_grouped(x, w, y, n, experts, tile_expert, row_scale=None, gated=False, limit=0.0, alpha=0.0, shift=0.0,
                    bn=MOE_TC_TILE, gelu=False):
    """The tcgen05 product over groups of rows: x [rows, K] holds the groups one after the other, each
    starting at a multiple of ``bn`` rows; w stacks the groups' matrices ([experts * n, K], or
    [experts * 2 n, K] gated); tile_expert names the group of every tile of ``bn`` rows (-1: none).
    y float32 [rows, n], or with ``gated`` bfloat16 [rows, n] = row_scale * act(gate, up), or with
    ``gelu`` bfloat16 [rows, n] = row_scale * gelu(x w^T) (erf form, no gate rows)."""
    _cuda(x, w, y, tile_expert, row_scale)
    rows, k = x.shape
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous()
    assert not (gated and gelu)
    assert y.shape == (rows, n) and y.is_contiguous() and y.dtype == (torch.bfloat16 if gated or gelu else torch.float32)
    assert tile_expert.dtype == torch.int32 and tile_expert.numel() == rows // bn and rows % bn == 0
    f = _fn("gemm_tc", "gb_gemm_tc_grouped",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int, c_int, c_void_p,
             c_void_p, c_float, c_float, c_float, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), y.data_ptr(), 3 if gated else (0 if gelu else 1), rows, n, k, x.stride(0), y.stride(0), bn,
             sm_count(x.device), experts, tile_expert.data_ptr(), _ptr(row_scale), limit, alpha, shift, _stream()),
           "gemm_tc_grouped", "matmul", _nbytes(x, w, y))


def moe_experts_tc(h, idx, wts, sg, w_gate_up, w_down, shared_gate_up, shared_down, residual, limit, shared_limit, alpha,
                   shift):
    """As moe_experts_grouped for a prompt step, the experts' two products on the tcgen05 kernel: the
    activations are copied into an order in which every expert's rows start at a multiple of the
    tile's tokens (zeros between), the routing weight multiplies the activation's rows, and a token's
    float32 rows are added into the residual in slot order."""
    _cuda(h, idx, wts, sg, w_gate_up, w_down, shared_gate_up, shared_down, residual)
    t, width = h.shape
    e, ff2, _ = w_gate_up.shape
    ff, top, bn = ff2 // 2, idx.shape[1], MOE_TC_TILE
    entries = t * top
    rows = (-(-entries // bn) + e) * bn
    meta = torch.empty(rows // bn + entries + rows, dtype=torch.int32, device=h.device)
    tile_expert, place, row_entry = meta[:rows // bn], meta[rows // bn:rows // bn + entries], meta[rows // bn + entries:]
    f = _fn("grouped_gemm", "gb_moe_sort_padded", [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    _check(f(idx.data_ptr(), entries, e, bn, rows, tile_expert.data_ptr(), place.data_ptr(), row_entry.data_ptr(), _stream()),
           "moe_sort", "elementwise", 3 * entries * 4)
    xp = torch.empty((rows, width), dtype=torch.bfloat16, device=h.device)
    scale = torch.empty((rows,), dtype=torch.float32, device=h.device)
    f = _fn("grouped_gemm", "gb_moe_permute", [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                               c_int, c_int, c_int, c_void_p])
    _check(f(h.data_ptr(), h.stride(0), row_entry.data_ptr(), tile_expert.data_ptr(), wts.data_ptr(), xp.data_ptr(),
             scale.data_ptr(), rows, width, top, bn, _stream()), "moe_permute", "elementwise", 2 * entries * width * 2)
    y = torch.empty((rows, ff), dtype=torch.bfloat16, device=h.device)
    gemm_tc_grouped(xp, w_gate_up.view(e * ff2, width), y, ff, e, tile_expert, scale, gated=True, limit=limit, alpha=alpha,
                    shift=shift)
    out = torch.empty((rows, width), dtype=torch.float32, device=h.device)
    gemm_tc_grouped(y, w_down.view(e * width, ff), out, width, e, tile_expert)
    f = _fn("grouped_gemm", "gb_moe_combine", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p])
    _check(f(out.data_ptr(), place.data_ptr(), residual.data_ptr(), residual.stride(0), t, width, top, _stream()),
           "moe_combine", "elementwise", entries * width * 4 + 2 * t * width * 4)
    _shared_expert(h, sg, shared_gate_up, shared_down, residual, shared_limit, alpha, shift)


def _shared_expert(h, sg, shared_gate_up, shared_down, residual, shared_limit, alpha, shift):
    """residual += sg * shared(h): two dense products of the framework's around the activation."""
    if shared_down is None:
        return
    t, ffs = h.shape[0], shared_down.shape[1]
    gu = torch.empty((t, 2 * ffs), dtype=torch.bfloat16, device=h.device)
    gemm(h, shared_gate_up, gu)
    ys = torch.empty((t, ffs), dtype=torch.bfloat16, device=h.device)
    f = _fn("grouped_gemm", "gb_gated_act", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_float, c_void_p])
    _check(f(gu.data_ptr(), ys.data_ptr(), _ptr(sg), t, ffs, shared_limit, alpha, shift, _stream()), "gated_act",
           "elementwise", _nbytes(gu, ys))
    gemm(ys, shared_down, residual, accumulate=True)


# --------------------------------------------------------------------------- sampling

_sample_scratch = {}
_sample_cut_scratch = {}


def sample(logits, out, temperature=None, top_k=None, top_p=None, uniform=None, wide=False, cap: Optional[int] = None):
    """out[r] = token drawn from logits[r] (float32 [rows, vocab]).  Rows whose temperature is
    <= 0 (or all rows when ``temperature`` is None) take the first maximum.  ``cap``: the largest
    top_k among the rows that have one from 1 to MAX_TOP_K (None: MAX_TOP_K when any row is
    sampled, 1 when all are greedy); a smaller cap is less work.  Rows with top_k = 0 (all tokens)
    or more than MAX_TOP_K candidates need ``wide``: they are sorted in scratch memory of 20 bytes
    per logit."""
    _cuda(logits, out, temperature, top_k, top_p, uniform)
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1 and out.dtype == torch.int32
    rows, vocab = logits.shape
    if cap is None:
        cap = 1 if temperature is None else MAX_TOP_K
    cap = max(1, min(int(cap), MAX_TOP_K))
    sms = sm_count(logits.device)
    size = _fn("sampling", "gb_sample_scratch_bytes", [c_int, c_int, c_int, c_int])
    size.restype = c_longlong
    need = size(rows, vocab, cap, sms)
    if need < 0:
        raise KernelError(f"sample: a vocabulary of {vocab} with up to {cap} candidates a row is not supported "
                          "(at most 64 slices of 16,384 tokens, whose candidates together number at most 16,384)")
    cut = _sample_cut_scratch.get(logits.device.index)
    if cut is None or cut.numel() < need:
        if cut is not None:
            _outgrown.append(cut)         # a captured step may still point at it: never freed
        cut = _sample_cut_scratch[logits.device.index] = torch.empty(max(need, 1 << 20), dtype=torch.uint8,
                                                                     device=logits.device)
    scratch = None
    if wide and temperature is not None:
        need = 5 * rows * vocab
        scratch = _sample_scratch.get(logits.device.index)
        if scratch is None or scratch.numel() < need:
            scratch = _sample_scratch[logits.device.index] = torch.empty(need, dtype=torch.float32, device=logits.device)
    f = _fn("sampling", "gb_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p])
    _check(f(logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(uniform), out.data_ptr(), _ptr(scratch), cut.data_ptr(), cap, sms, _stream()),
           "sample", "sampling", _nbytes(logits))
    count_launches(1 if scratch is None else 2)


# --------------------------------------------------------------------------- choices by precision and shape

def gemm_units(compute: str):
    """The units ``gemm`` may launch for a model computed in ``compute``."""
    return [("gemm_ref", ())] if compute == "float32" else [("gemm_tc", ()), ("gemm_ref", ())]


# Whether the blocks take the RMSNorms of a decode step into the products around them (see
# UnscaledRows).  Measured as an upper bound, by skipping the norm kernels: 2 % of a step at 8B layer
# sizes, 5.6 % at 4B sizes.
NORM_LINKS = True


def gemm(x, w, out, bias=None, accumulate=False, then_norm=None):
    """out = x @ w.T (+ bias) or, with ``accumulate``, out += ...; picks the kernel for the
    precision and the shape: float32 runs on the CUDA cores in a fixed order; bfloat16 runs on the
    tensor cores, except for operands whose rows TMA cannot address (an inner size that is not
    a multiple of 8), which the plain kernel takes.  ``x`` may be UnscaledRows (a norm taken into
    this product).  ``then_norm`` = (weight, eps) of an RMSNorm that follows an accumulating
    product: where the kernel can, it leaves that norm's input as UnscaledRows, which is returned
    (None: the norm has to run by itself)."""
    link = x if isinstance(x, UnscaledRows) else None
    if link is not None:
        if norm_link_usable(link.rows, w, link.rows.shape[0]):
            x = link.rows
        else:
            x, link = link.materialize(), None
    if x.dtype == torch.bfloat16 and gemm_tc_usable(x, w):
        m, n, k = x.shape[0], w.shape[0], x.shape[1]
        if m > 64:
            gemm_tc_persistent(x, w, out, bias, accumulate)
            return None
        if then_norm is not None and not (accumulate and gemm_tc_tiling(m, n, k)[1] >= 2):
            then_norm = None
        return gemm_tc(x, w, out, bias, accumulate, link_in=link, link_out=then_norm)
    gemm_ref(x, w, out, bias, accumulate)
    return None


def attention_units(compute: str, head_dim: int):
    if compute == "float32":
        return [("attention_ref", ())]
    hd = (("GB_HEAD_DIM", head_dim),)
    prefill = "attention_prefill_tc" if head_dim in (64, 128) else "attention_prefill"
    units = [("attention_ref", ()), ("attention_decode", hd), (prefill, hd)]
    if head_dim in STREAM_DECODE_HEAD_DIMS:
        units.append(("attention_decode_stream", hd))
    return units


def attention(ctx, q, out, nh, kcache, vcache, page_table, page_size, window=None):
    """Attention of the step's queries over the cache; picks the kernel for the precision and
    for prompts or single tokens.  float32 always takes the plain kernel, whose arithmetic for a
    position does not depend on the batch."""
    cached = 0
    if _profile["on"] and ctx.host is not None:
        # keys and values the step has to read: each sequence's positions (its window's worth) once
        per_pos = 2 * kcache.shape[1] * kcache.shape[3] * kcache.element_size()
        for start, n in zip(ctx.host["seq_start"], ctx.host["seq_len"]):
            cached += per_pos * (min(start + n, window + n - 1) if window else start + n)
    if q.dtype == torch.bfloat16 and ctx.max_new <= DECODE_KERNEL_MAX_NEW:
        nkv = kcache.shape[1]
        if attention_decode_stream_usable(ctx.n_tokens, nh, nkv, kcache.shape[3], page_size):
            attention_decode_stream(q, out, nh, kcache, vcache, page_table, page_size, ctx.tok_pos, ctx.tok_seq,
                                    ctx.seq_slot, window, skip_slot=ctx.pad_slot, cache_bytes=cached)
            return
        shares = decode_shares(ctx.n_tokens, nh, nkv, ctx.max_total if window is None else min(ctx.max_total, window))
        attention_decode(q, out, nh, kcache, vcache, page_table, page_size, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                         window, shares, cache_bytes=cached)
        return
    if q.dtype == torch.bfloat16:
        prefill = attention_prefill_tc if kcache.shape[3] in TC_PREFILL_HEAD_DIMS else attention_prefill
        prefill(q, out, nh, kcache, vcache, page_table, page_size, ctx.cu_seqlens, ctx.seq_start, ctx.seq_slot, window,
                cache_bytes=cached)
        return
    attention_ref(q, out, nh, kcache, vcache, page_table, page_size, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, window,
                  cache_bytes=cached)


# a step whose sequences bring at most this many tokens each runs the per-position decode kernel
DECODE_KERNEL_MAX_NEW = 1


# --------------------------------------------------------------------------- rows: second tables, norms after a sublayer

ACT_SILU, ACT_GELU_TANH = 0, 1
GATED_ACTS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}


def gather_add(table: torch.Tensor, idx: torch.Tensor, x: torch.Tensor):
    """x[t] += table[idx[t]]; x is the float32 residual stream [T, H]."""
    _cuda(table, idx, x)
    assert idx.dtype == torch.int32 and x.dtype == torch.float32 and x.is_contiguous() and table.is_contiguous()
    assert table.shape[1] == x.shape[1] and idx.numel() == x.shape[0]
    f = _fn("rows", "gb_gather_add", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(table.data_ptr(), dtype_code(table.dtype), idx.data_ptr(), x.data_ptr(), idx.numel(), table.shape[1],
             table.shape[0], _stream()), "gather_add", "embed",
           2 * _nbytes(x) + idx.numel() * table.shape[1] * table.element_size())


def rmsnorm_add(y: torch.Tensor, weight: torch.Tensor, x: torch.Tensor, eps: float, then=None):
    """x[t] += y[t] * (mean(y[t]^2) + eps)^-1/2 * weight: a norm on a sublayer's output, added into
    the float32 residual stream.  ``then`` = (weight2, eps2, out): the norm that reads the stream
    next, taken in the same pass: out[t] = x[t] * (mean(x[t]^2) + eps2)^-1/2 * weight2."""
    _cuda(y, weight, x)
    assert y.dtype == torch.float32 and x.dtype == torch.float32 and weight.dtype == torch.float32
    assert y.is_contiguous() and x.is_contiguous() and y.shape == x.shape and weight.numel() == x.shape[-1]
    n = x.shape[-1]
    w2 = out = None
    eps2 = 0.0
    if then is not None:
        w2, eps2, out = then
        _cuda(w2, out)
        assert w2.dtype == torch.float32 and w2.numel() == n and out.is_contiguous() and out.shape == x.shape
    f = _fn("rows", "gb_rmsnorm_add",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_float, c_void_p])
    _check(f(y.data_ptr(), weight.data_ptr(), x.data_ptr(), x.numel() // n, n, eps, _ptr(w2), _ptr(out),
             dtype_code(out.dtype) if out is not None else F32, eps2, _stream()), "rmsnorm_add", "norm",
           _nbytes(y, weight, out) + 2 * _nbytes(x))


def gated_act(gu: torch.Tensor, out: torch.Tensor, act: str = "silu"):
    """out[t, i] = act(gu[t, i]) * gu[t, I + i], act one of GATED_ACTS."""
    _cuda(gu, out)
    inter = out.shape[-1]
    assert gu.shape[-1] == 2 * inter and gu.dtype == out.dtype and gu.is_contiguous() and out.is_contiguous()
    f = _fn("rows", "gb_gated_act", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(gu.data_ptr(), out.data_ptr(), dtype_code(out.dtype), out.numel() // inter, inter, GATED_ACTS[act],
             _stream()), "gated_act", "elementwise", _nbytes(gu, out))


def scale_rows(y: torch.Tensor, s: float):
    """y *= s in place (float32)."""
    _cuda(y)
    assert y.dtype == torch.float32 and y.is_contiguous()
    f = _fn("rows", "gb_scale_f32", [c_void_p, c_longlong, c_float, c_void_p])
    _check(f(y.data_ptr(), y.numel(), s, _stream()), "scale_rows", "elementwise", 2 * _nbytes(y))


# --------------------------------------------------------------------------- mixers with a state per sequence

def _cols(t: torch.Tensor):
    """A [T, n] tensor or a slice of columns of one: unit stride inside a row."""
    assert t.dim() == 2 and t.stride(1) == 1
    return t.data_ptr(), t.stride(0)


def short_filter(u, taps, bias, state, cu_seqlens, tok_seq, seq_slot, out, act: bool = False, update_state: bool = True):
    """out[t, c] = act(bias[c] + sum_j taps[c, j] u[t - K + 1 + j, c]) along each sequence of the
    packed step; the rows before the step's first come from ``state`` [slots + 1, K - 1, C]
    (float32, oldest first), which then takes the sequence's last K - 1 inputs.  ``u`` and ``out``
    may be slices of columns; ``act``: SiLU."""
    _cuda(u, taps, bias, state, cu_seqlens, tok_seq, seq_slot, out)
    c, k = taps.shape
    assert taps.dtype == torch.float32 and taps.is_contiguous() and u.shape[1] == c and out.shape == u.shape
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (max(k - 1, 0), c)
    up, ldu = _cols(u)
    op, ldo = _cols(out)
    f = _fn("recurrent", "gb_short_filter",
            [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
             c_longlong, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(up, dtype_code(u.dtype), ldu, taps.data_ptr(), _ptr(bias), state.data_ptr(), cu_seqlens.data_ptr(),
             tok_seq.data_ptr(), seq_slot.data_ptr(), op, dtype_code(out.dtype), ldo, u.shape[0], seq_slot.numel(), c, k,
             1 if act else 0, 1 if update_state else 0, _stream()), "short_filter", "elementwise",
           u.numel() * u.element_size() + out.numel() * out.element_size())
    if update_state and k > 1 and u.shape[0] != seq_slot.numel():
        count_launches(1)      # the kernel that shifts the memory (a step of single tokens does both in one)


def short_filter_state(u, state, cu_seqlens, seq_slot, k: int):
    """Only the state's update of ``short_filter``."""
    _cuda(u, state, cu_seqlens, seq_slot)
    if k <= 1:
        return
    c = u.shape[1]
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (k - 1, c)
    up, ldu = _cols(u)
    f = _fn("recurrent", "gb_short_filter_state",
            [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(up, dtype_code(u.dtype), ldu, state.data_ptr(), cu_seqlens.data_ptr(), seq_slot.data_ptr(), seq_slot.numel(),
             c, k, _stream()), "short_filter_state", "elementwise", 0)


def recurrent_state_floats(dims: int, vdim: int) -> int:
    """Floats that ``delta_rule`` and ``ssd_scan`` keep per head for a state matrix [dims, vdim]: the
    dims are padded to 32 lanes' worth (32, 64, 128 or 256) and stored in the order the kernel's
    lanes read them (see csrc/recurrent.cu)."""
    lanes = 1 if dims <= 32 else (2 if dims <= 64 else (4 if dims <= 128 else 8))
    return 32 * lanes * vdim


def recurrent_state_matrix(head_state: torch.Tensor, dims: int, vdim: int) -> torch.Tensor:
    """The state matrix [dims, vdim] that one head's stored floats hold: element (d, col) with
    d = 32 part + 4 r + e lies at ((r * vdim + col) * lanes + part) * 4 + e."""
    lanes = head_state.numel() // (32 * vdim)
    return head_state.reshape(8, vdim, lanes, 4).permute(2, 0, 3, 1).reshape(32 * lanes, vdim)[:dims]


def delta_rule(q, k, v, beta_logit, a_logit, a_log, dt_bias, state, cu_seqlens, seq_slot, y, heads, groups, dim, vdim,
               q_scale):
    """The gated delta rule over each sequence of the packed step (float32 throughout):
    S <- g S; u = beta (v - S^T k^); S <- S + k^ u^T; y = S^T q^, with k^, q^ the unit vectors of k
    and q (q^ times ``q_scale``), beta = sigmoid(beta_logit), g = exp(-exp(a_log) softplus(a_logit +
    dt_bias)).  q, k, v: slices of columns of one [T, *] tensor; ``state`` [slots + 1, heads,
    recurrent_state_floats(dim, vdim)] (see recurrent_state_matrix); dim up to 256."""
    _cuda(q, k, v, beta_logit, a_logit, a_log, dt_bias, state, cu_seqlens, seq_slot, y)
    for t in (q, k, v, beta_logit, a_logit, y, state):
        assert t.dtype == torch.float32
    qp, ld = _cols(q)
    kp, ldk = _cols(k)
    vp, ldv = _cols(v)
    bp, ldg = _cols(beta_logit)
    ap, lda = _cols(a_logit)
    assert ld == ldk == ldv and ldg == lda and y.is_contiguous() and y.shape[1] == heads * vdim
    assert state.is_contiguous() and tuple(state.shape[1:]) == (heads, recurrent_state_floats(dim, vdim))
    f = _fn("recurrent", "gb_delta_rule",
            [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(qp, kp, vp, ld, bp, ap, ldg, a_log.data_ptr(), dt_bias.data_ptr(), state.data_ptr(), cu_seqlens.data_ptr(),
             seq_slot.data_ptr(), y.data_ptr(), seq_slot.numel(), heads, groups, dim, vdim, q_scale, _stream()),
           "delta_rule", "attention", _nbytes(y) * 2 + 2 * seq_slot.numel() * heads * dim * vdim * 4)


def ssd_scan(x, b, c, dt_raw, a_log, dt_bias, skip, state, cu_seqlens, seq_slot, y, heads, groups, n_state, vdim):
    """The state-space recurrence with one decay per head over each sequence of the packed step
    (float32): dt = softplus(dt_raw + dt_bias); S <- exp(-exp(a_log) dt) S + dt B x^T; y = S^T C +
    skip x.  x, b, c: slices of columns of one tensor; ``state`` [slots + 1, heads,
    recurrent_state_floats(n_state, vdim)]; n_state up to 256."""
    _cuda(x, b, c, dt_raw, a_log, dt_bias, skip, state, cu_seqlens, seq_slot, y)
    for t in (x, b, c, dt_raw, y, state):
        assert t.dtype == torch.float32
    xp, ld = _cols(x)
    bp, ldb = _cols(b)
    cp, ldc = _cols(c)
    dp, ldd = _cols(dt_raw)
    assert ld == ldb == ldc and y.is_contiguous() and y.shape[1] == heads * vdim
    assert state.is_contiguous() and tuple(state.shape[1:]) == (heads, recurrent_state_floats(n_state, vdim))
    f = _fn("recurrent", "gb_ssd_scan",
            [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(xp, bp, cp, ld, dp, ldd, a_log.data_ptr(), dt_bias.data_ptr(), skip.data_ptr(), state.data_ptr(),
             cu_seqlens.data_ptr(), seq_slot.data_ptr(), y.data_ptr(), seq_slot.numel(), heads, groups, n_state, vdim,
             _stream()), "ssd_scan", "attention", _nbytes(y) * 2 + 2 * seq_slot.numel() * heads * n_state * vdim * 4)


GATE_ACTS = {"silu": 0, "sigmoid": 1}


def gated_group_norm(y, gate, weight, out, group_size: int, eps: float, gate_first: bool, out_scale: float = 1.0,
                     gate_act: str = "silu"):
    """Rows of float32 ``y`` [T, n] in groups of ``group_size`` channels, each group divided by its
    root mean square, channel i times weight[i % len(weight)] and silu(gate[t, i]) (or, with
    ``gate_act`` "sigmoid", sigmoid(gate[t, i])); with ``gate_first`` the gate goes in before the
    statistics.  ``gate``: float32, may be a slice."""
    _cuda(y, gate, weight, out)
    assert y.dtype == torch.float32 and gate.dtype == torch.float32 and weight.dtype == torch.float32
    assert y.is_contiguous() and out.is_contiguous() and out.shape == y.shape and gate.shape == y.shape
    gp, ldg = _cols(gate)
    f = _fn("recurrent", "gb_gated_group_norm_act",
            [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_float,
             c_int, c_void_p])
    _check(f(y.data_ptr(), gp, ldg, weight.data_ptr(), weight.numel(), out.data_ptr(), dtype_code(out.dtype), y.shape[0],
             y.shape[1], group_size, eps, 1 if gate_first else 0, out_scale, GATE_ACTS[gate_act], _stream()),
           "gated_group_norm", "norm",
           _nbytes(y, out) + y.numel() * 4)


def shift_mix(x, mu, state, cu_seqlens, tok_seq, seq_slot):
    """[n_mix, T, C] in x's type: out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s] along each sequence of
    the packed step, in float32 before the rounding.  The row before a sequence's first row of
    the step is ``state`` [slots + 1, C] (float32; zeros for a new sequence), which then takes the
    sequence's last row."""
    _cuda(x, mu, state, cu_seqlens, tok_seq, seq_slot)
    n_mix, c = mu.shape
    assert mu.dtype == torch.float32 and mu.is_contiguous() and x.shape[1] == c
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (c,)
    xp, ldx = _cols(x)
    out = torch.empty((n_mix, x.shape[0], c), dtype=x.dtype, device=x.device)
    f = _fn("recurrent", "gb_shift_mix", [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(f(xp, dtype_code(x.dtype), ldx, mu.data_ptr(), state.data_ptr(), cu_seqlens.data_ptr(), tok_seq.data_ptr(),
             seq_slot.data_ptr(), out.data_ptr(), x.shape[0], seq_slot.numel(), c, n_mix, _stream()), "shift_mix",
           "elementwise", _nbytes(x, out))
    if x.shape[0] != seq_slot.numel():
        count_launches(1)      # the kernel that keeps each sequence's last row
    return out


def lowrank_decay(z, w2, base):
    """float32 [T, C]: exp(-exp(base + tanh(z) @ w2.T)), all of it float32 arithmetic.  ``z``: float32
    [T, rank]; ``w2``: [C, rank] float32 or bfloat16; ``base``: float32 [C]."""
    _cuda(z, w2, base)
    c, rank = w2.shape
    assert z.dtype == torch.float32 and z.is_contiguous() and z.shape[1] == rank and w2.is_contiguous()
    assert base.dtype == torch.float32 and base.numel() == c
    out = torch.empty((z.shape[0], c), dtype=torch.float32, device=z.device)
    f = _fn("recurrent", "gb_lowrank_decay", [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(z.data_ptr(), rank, w2.data_ptr(), dtype_code(w2.dtype), base.data_ptr(), out.data_ptr(), z.shape[0], c,
             _stream()), "lowrank_decay", "elementwise", _nbytes(z, out, w2))
    return out


LOWRANK_MODES = {"tanh_expexp": 0, "rate": 1, "sigmoid_root": 2, "plain": 3}


def lowrank_map(z, w2, base, mode: str, rate=None, rate_group: int = 1, tau: float = 1.0):
    """float32 [T, C] from the second half of a two-matrix projection, a = z @ w2.T + base in float32
    (``z`` float32 [T, rank], may be a slice of columns; ``base`` float32 [C] or None), by ``mode``:
    "rate": exp(-exp(rate[c // rate_group]) * softplus(a)); "sigmoid_root": sigmoid(a) ** (1 / tau);
    "plain": a; "tanh_expexp": exp(-exp(tanh(z) @ w2.T + base)) (lowrank_decay)."""
    _cuda(z, w2, base, rate)
    c, rank = w2.shape
    assert z.dtype == torch.float32 and z.shape[1] == rank and w2.is_contiguous()
    assert base is None or (base.dtype == torch.float32 and base.numel() == c)
    assert rate is None or (rate.dtype == torch.float32 and rate.is_contiguous() and rate.numel() * rate_group == c)
    zp, ldz = _cols(z)
    out = torch.empty((z.shape[0], c), dtype=torch.float32, device=z.device)
    f = _fn("recurrent", "gb_lowrank_map", [c_void_p, c_longlong, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_void_p, c_int, c_float, c_void_p])
    _check(f(zp, ldz, rank, w2.data_ptr(), dtype_code(w2.dtype), _ptr(base), out.data_ptr(), z.shape[0], c,
             LOWRANK_MODES[mode], _ptr(rate), rate_group, float(tau), _stream()), "lowrank_map", "elementwise",
           _nbytes(out, w2) + z.shape[0] * rank * 4)
    return out


def channel_delta_rule(q, k, v, beta_logit, decay, state, cu_seqlens, seq_slot, y, heads, groups, dim, vdim, q_scale):
    """The delta rule with a decay per head and key channel over each sequence of the packed step
    (float32 throughout): S <- diag(g) S; u = beta (v - S^T k^); S <- S + k^ u^T; y = S^T q^, with k^,
    q^ the unit vectors of k and q (q^ times ``q_scale``), beta = sigmoid(beta_logit), g = ``decay``
    [T, heads * dim] as given.  q, k, v: slices of columns of one [T, *] tensor, q/k head
    i // (heads / groups) for head i; ``state`` as for delta_rule; dim up to 256."""
    _cuda(q, k, v, beta_logit, decay, state, cu_seqlens, seq_slot, y)
    for t in (q, k, v, beta_logit, decay, y, state):
        assert t.dtype == torch.float32
    qp, ld = _cols(q)
    kp, ldk = _cols(k)
    vp, ldv = _cols(v)
    bp, ldb = _cols(beta_logit)
    dp, ldd = _cols(decay)
    assert ld == ldk == ldv and y.is_contiguous() and y.shape[1] == heads * vdim and decay.shape[1] == heads * dim
    assert state.is_contiguous() and tuple(state.shape[1:]) == (heads, recurrent_state_floats(dim, vdim))
    f = _fn("recurrent", "gb_channel_delta_rule",
            [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(qp, kp, vp, ld, bp, ldb, dp, ldd, state.data_ptr(), cu_seqlens.data_ptr(), seq_slot.data_ptr(), y.data_ptr(),
             seq_slot.numel(), heads, groups, dim, vdim, q_scale, _stream()),
           "channel_delta_rule", "attention", _nbytes(y) * 2 + _nbytes(decay) + 2 * seq_slot.numel() * heads * dim * vdim * 4)


def wkv_scan(r, k, w, v, bonus, state, cu_seqlens, seq_slot, y, heads, dim, vdim, out_scale: float = 1.0):
    """Linear attention with a decay per key channel over each sequence of the packed step (float32):
    y = S^T r + (sum_d r_d bonus_d k_d) v, then S <- diag(w) S + k v^T, per head.  r, k: [T, heads *
    dim] with equal row strides; w: [T, heads * dim]; v: [T, heads * vdim]; ``bonus`` [heads, dim]; ``state`` [slots + 1,
    heads, recurrent_state_floats(dim, vdim)] (see recurrent_state_matrix); dim up to 256.
    ``bonus`` None: the read-out follows the write, S <- diag(w) S + k v^T; y = S^T r (gated linear
    attention).  ``out_scale`` multiplies y (a factor on r, which y is linear in)."""
    _cuda(r, k, w, v, bonus, state, cu_seqlens, seq_slot, y)
    for t in (r, k, w, v, bonus, state, y):
        assert t is None or t.dtype == torch.float32
    rp, ld = _cols(r)
    kp, ldk = _cols(k)
    wp, ldw = _cols(w)
    vp, ldv = _cols(v)
    assert ld == ldk and y.is_contiguous() and y.shape[1] == heads * vdim
    assert bonus is None or (bonus.is_contiguous() and bonus.numel() == heads * dim)
    assert state.is_contiguous() and tuple(state.shape[1:]) == (heads, recurrent_state_floats(dim, vdim))
    f = _fn("recurrent", "gb_wkv_scan_scaled", [c_void_p, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p,
                                                c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                                c_void_p])
    _check(f(rp, kp, wp, ld, ldw, vp, ldv, _ptr(bonus), state.data_ptr(), cu_seqlens.data_ptr(), seq_slot.data_ptr(),
             y.data_ptr(), seq_slot.numel(), heads, dim, vdim, float(out_scale), _stream()), "wkv_scan", "attention",
           _nbytes(y) * 5 + 2 * seq_slot.numel() * heads * dim * vdim * 4)


# --------------------------------------------------------------------------- attention with capped scores

def filter_rope_cache(u, taps, state, inv_freq, rot, ctx_pos, tok_seq, seq_slot, cu_seqlens, page_table, page_size, q_out,
                      kcache, vcache, heads, groups, dim, vdim, q_norm=None, k_norm=None, norm_eps: float = 0.0,
                      rot_magnitude: float = 1.0, q_temper=None, values_are_keys: bool = False):
    """The columns [q | k | v] of ``u`` through a short causal filter (``taps`` [channels, K] or
    None), the first ``rot`` dims of each q and k head rotated (pairs i, i + rot/2), then q into
    ``q_out`` [T, heads * dim] and keys and values into their pages (None: not kept).
    ``q_norm`` / ``k_norm`` (float32 [dim]): every q / k head is divided by its root mean square
    (``norm_eps``) and multiplied by the weight before the rotation.  ``rot_magnitude`` multiplies
    the cosines and sines.  ``q_temper`` (coef, every): q at position p times 1 + coef ln(floor((p +
    1) / every) + 1).  ``values_are_keys``: the rows hold [q | k] alone and a value head is its key
    head as projected and filtered, before norm and rotation (vdim == dim)."""
    _cuda(u, taps, state, inv_freq, ctx_pos, tok_seq, seq_slot, cu_seqlens, page_table, q_out, kcache, vcache, q_norm, k_norm)
    channels = (heads + groups) * dim + (0 if values_are_keys else groups * vdim)
    for w in (q_norm, k_norm):
        assert w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == dim)
    assert not values_are_keys or vdim == dim
    qt_coef, qt_every = (float(q_temper[0]), int(q_temper[1])) if q_temper else (0.0, 0)
    k = 0 if taps is None else taps.shape[1]
    up, ldu = _cols(u)
    qp, ldq = _cols(q_out)
    assert u.shape[1] == channels and q_out.dtype == u.dtype
    if taps is not None:
        assert taps.dtype == torch.float32 and taps.is_contiguous() and taps.shape[0] == channels
    if k > 1:
        assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (k - 1, channels)
    if kcache is not None:
        assert kcache.dtype == u.dtype and vcache.dtype == u.dtype and kcache.is_contiguous() and vcache.is_contiguous()
        assert tuple(kcache.shape[1:]) == (groups, page_size, dim) and tuple(vcache.shape[1:]) == (groups, vdim, page_size)
    f = _fn("attention_capped", "gb_filter_rope_cache_ext",
            [c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
             c_void_p, c_float, c_float, c_float, c_int, c_int, c_void_p])
    _check(f(up, dtype_code(u.dtype), ldu, _ptr(taps), _ptr(state) if k > 1 else None, k, _ptr(inv_freq) if rot else None,
             rot, ctx_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), cu_seqlens.data_ptr(), _ptr(page_table),
             page_table.shape[1] if page_table is not None else 1, page_size, qp, ldq, _ptr(kcache), _ptr(vcache),
             u.shape[0], heads, groups, dim, vdim, _ptr(q_norm), _ptr(k_norm), float(norm_eps), float(rot_magnitude), qt_coef,
             qt_every, 1 if values_are_keys else 0, _stream()), "filter_rope_cache", "elementwise",
           2 * u.numel() * u.element_size())


#: whether bfloat16 steps take the tensor-core kernel where its sizes allow (tests turn it off to
#: run the plain kernel on the same inputs)
CAPPED_ATTENTION_MMA = True


def attention_capped_mma_usable(dtype, dim: int, vdim: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and dim % 16 == 0 and 16 <= dim <= 256 and vdim % 8 == 0 and 8 <= vdim <= 256
            and page_size % 32 == 0)


def attention_capped_units(compute: str, dim: int, vdim: int, page_size: int = 64):
    units = [("attention_capped", ())]
    if compute == "bfloat16" and attention_capped_mma_usable(torch.bfloat16, dim, vdim, page_size):
        units.append(("attention_capped_mma", (("GB_HEAD_DIM", dim), ("GB_VALUE_DIM", vdim))))
    return units


def attention_capped(ctx, q, out, heads, kcache, vcache, page_table, page_size, window, scale, cap, gate=None,
                     out_scale: float = 1.0, keep_first: int = 0, sink=None):
    """Attention of the step's queries [T, heads * dim] over the cache with keys of ``dim`` and
    values of ``vdim``: score = (q . k) * scale, capped as cap * tanh(score / cap) when ``cap``;
    a window of ``window`` keys when given, beside which the first ``keep_first`` keys of the
    sequence stay visible; ``sink`` (float32 [heads]): exp(sink[head]) is one more term of the
    softmax's denominator; the output times sigmoid(gate) * out_scale.  bfloat16
    steps run on the tensor cores where the sizes allow (keys a multiple of 16, values of 8, up to
    256), prompts and single tokens alike; float32 and other sizes run the plain kernel."""
    _cuda(q, out, kcache, vcache, page_table, gate, sink)
    groups, dim, vdim = kcache.shape[1], kcache.shape[3], vcache.shape[2]
    assert sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == heads)
    keep_first = int(keep_first or 0)
    qp, ldq = _cols(q)
    op, ldo = _cols(out)
    gp, ldg = _cols(gate) if gate is not None else (None, 0)
    assert q.dtype == out.dtype == kcache.dtype == vcache.dtype and (gate is None or gate.dtype == q.dtype)
    assert q.shape[1] == heads * dim and out.shape[1] == heads * vdim
    if (CAPPED_ATTENTION_MMA and attention_capped_mma_usable(q.dtype, dim, vdim, page_size)
            and getattr(ctx, "cu_seqlens", None) is not None and qp % 16 == 0 and ldq % 8 == 0 and op % 4 == 0
            and ldo % 2 == 0 and (gp or 0) % 4 == 0 and ldg % 2 == 0):
        f = _fn("attention_capped_mma", "gb_attention_capped_mma",
                [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_float, c_void_p,
                 c_longlong, c_float, c_int, c_void_p], (("GB_HEAD_DIM", dim), ("GB_VALUE_DIM", vdim)))
        _check(f(qp, ldq, op, ldo, kcache.data_ptr(), vcache.data_ptr(), page_table.data_ptr(), page_table.shape[1], page_size,
                 groups, dim, vdim, ctx.cu_seqlens.data_ptr(), ctx.seq_start.data_ptr(), ctx.seq_slot.data_ptr(), ctx.n_seqs,
                 q.shape[0], heads, int(window or 0), keep_first, _ptr(sink), scale, float(cap or 0.0), gp, ldg, out_scale,
                 1 if q.shape[0] == ctx.n_seqs else 0, _stream()),
               "attention_capped_mma", "attention", 2 * q.numel() * q.element_size())
        return
    f = _fn("attention_capped", "gb_attention_capped",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_float, c_void_p, c_longlong, c_float,
             c_void_p])
    _check(f(qp, ldq, op, ldo, dtype_code(q.dtype), kcache.data_ptr(), vcache.data_ptr(), page_table.data_ptr(),
             page_table.shape[1], page_size, groups, dim, vdim, ctx.tok_pos.data_ptr(), ctx.tok_seq.data_ptr(),
             ctx.seq_slot.data_ptr(), q.shape[0], heads, int(window or 0), keep_first, _ptr(sink), scale, float(cap or 0.0),
             gp, ldg, out_scale, _stream()), "attention_capped", "attention", 2 * q.numel() * q.element_size())
