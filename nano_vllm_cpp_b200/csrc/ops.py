"""ctypes binding of the CUDA library: one Python function per launcher.

Every function takes torch CUDA tensors, checks what the kernel assumes (dtype, contiguity,
sizes), launches on torch's current stream and raises ``KernelError`` on a refusal or a
CUDA error.  There is no CPU fallback: on a machine without the library (and without nvcc to
build it) importing the ops fails with the reason.
"""
from __future__ import annotations

import ctypes
import os
import re

import torch

from . import build as _build


# The launchers' prototypes are read from the sources (every ``NV_API`` function of csrc/*.cu) and given to ctypes,
# which then converts plain Python numbers and addresses itself and refuses a call with the wrong number of arguments.
_C_TYPES = {"int": ctypes.c_int, "long long": ctypes.c_longlong, "unsigned long long": ctypes.c_ulonglong,
            "float": ctypes.c_float, "double": ctypes.c_double, "void": None, "cudaStream_t": ctypes.c_void_p,
            "const char*": ctypes.c_char_p}


def _c_type(text: str):
    text = " ".join(text.replace("*", " * ").split())
    if "*" in text:
        return ctypes.c_char_p if text.replace("const ", "").startswith("char") else ctypes.c_void_p
    text = text.replace("const ", "")
    try:
        return _C_TYPES[text]
    except KeyError:
        raise KernelError(f"cannot read the C type {text!r} of a launcher's prototype") from None


def _declare(lib: ctypes.CDLL) -> None:
    """Sets ``argtypes`` and ``restype`` of every exported launcher from its definition in the sources."""
    proto = re.compile(r"NV_API\s+([\w\s\*]+?)\s*\b(nv_\w+)\s*\(([^)]*)\)\s*\{", re.S)
    for name in sorted(os.listdir(_build.CSRC)):
        if not name.endswith(".cu"):
            continue
        with open(os.path.join(_build.CSRC, name)) as f:
            text = f.read()
        for ret, fn, args in proto.findall(text):
            types = []
            for a in (x.strip() for x in args.split(",")):
                if not a or a == "void":
                    continue
                m = re.match(r"(.*?)(\w+)$", a, re.S)              # the type is what stands before the name
                types.append(_c_type(m.group(1)))
            f_ = getattr(lib, fn)
            f_.argtypes = types
            f_.restype = _c_type(ret)

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}
_ERR = {-2: "unsupported dtype", -3: "bad size", -4: "size not supported by this kernel",
        -5: "kernel set-up failed"}


class KernelError(RuntimeError):
    pass


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.library_path()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the CUDA library {path}: {e}") from None
        _declare(_lib)
        _lib.nv_set_dependent_launch(_early())
    return _lib


_launches = 0


def launch_count() -> int:
    """How many launcher calls have been made so far (each launches this library's kernels)."""
    return _launches


def add_launches(n: int) -> None:
    """Launches replayed from a CUDA graph, counted at its capture."""
    global _launches
    _launches += n


class KernelTimes:
    """CUDA-event timers per kernel class, off unless asked for:

        with ops.KernelTimes() as kt:
            runner.step(...)
        rows = kt.summary()        # [{"name", "calls", "ms", "flops", "bytes"}], largest first

    While it is active every launcher call records an event behind its launch; the time between two consecutive
    events of a stream is booked to the later launch (so a gap before a kernel counts as its own).  Steps must run
    outside CUDA graphs to be seen.  ``flops`` and ``bytes`` are what the launcher knows from its arguments (matrix
    sizes); 0 where it knows nothing."""

    def __init__(self):
        self.records = []           # (name, start event, end event, flops, bytes)
        self.last = {}

    def __enter__(self):
        global _timer
        torch.cuda.synchronize()
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        self.last = {}
        _timer = self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = None
        torch.cuda.synchronize()

    def mark(self) -> None:
        """The next launch's time starts here (the model calls this when a step's kernels begin, so that the host's
        preparation of the step is not booked to its first kernel)."""
        stream = torch.cuda.current_stream()
        e = torch.cuda.Event(enable_timing=True)
        e.record(stream)
        self.last[stream.cuda_stream] = e

    def note(self, name: str, flops: float, nbytes: float) -> None:
        stream = torch.cuda.current_stream()
        e = torch.cuda.Event(enable_timing=True)
        e.record(stream)
        self.records.append((name, self.last.get(stream.cuda_stream, self.start), e, flops, nbytes))
        self.last[stream.cuda_stream] = e

    def summary(self) -> list:
        torch.cuda.synchronize()
        rows = {}
        for name, a, b, flops, nbytes in self.records:
            r = rows.setdefault(name, {"name": name, "calls": 0, "ms": 0.0, "flops": 0.0, "bytes": 0.0})
            r["calls"] += 1
            r["ms"] += a.elapsed_time(b)
            r["flops"] += flops
            r["bytes"] += nbytes
        return sorted(rows.values(), key=lambda r: -r["ms"])


_timer = None


def timing() -> bool:
    """True while a ``KernelTimes`` is active: work that would run on a second stream stays on the first then, so
    that every kernel's time is its own."""
    return _timer is not None


def mark_step() -> None:
    if _timer is not None:
        _timer.mark()


def _check(code: int, what: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
    global _launches
    _launches += 1
    if _timer is not None and code == 0:
        _timer.note(what, flops, nbytes)
    if code == 0:
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERR.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def _cuda_error_name(code: int) -> str:
    try:
        f = lib().nv_error_string
        f.restype = ctypes.c_char_p
        return f(code).decode()
    except Exception:
        return "?"


# torch's own fast accessors of the current device and its current stream (a step makes some four hundred
# launches, and ``torch.cuda.current_stream()`` costs ten microseconds a time); the public call where they are missing
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    """The address of a tensor's first element (None: a null pointer)."""
    return None if t is None else t.data_ptr()


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda_contig(*ts) -> None:
    for t in ts:
        if t is None:
            continue
        _need(t.is_cuda, "tensor is not on a CUDA device")
        _need(t.is_contiguous(), "tensor is not contiguous")


def _i32(*ts) -> None:
    for t in ts:
        if t is not None:
            _need(t.dtype == torch.int32, f"index tensor must be int32, found {t.dtype}")


# ----------------------------------------------------------------------------- error flag
class ErrorFlag:
    """A device int that kernels set (to 1 + the offending row) instead of trapping."""

    def __init__(self, device):
        self.t = torch.zeros(1, dtype=torch.int32, device=device)

    def check(self, what: str) -> None:
        v = int(self.t.item())
        if v:
            self.t.zero_()
            if v >= 0x7000:
                raise KernelError(f"{what}: a kernel gave up waiting on a barrier (code {v:#x}); its output is invalid")
            raise KernelError(f"{what}: a kernel reported a bad index at row/pair {v - 1}")


# ----------------------------------------------------------------------------- plain ops
def random_fill(out, key: int, mean: float, std: float) -> None:
    """``out[i] = mean + z_i * std`` with z_i a function of (key, i) alone (see weights/random_values.py, whose
    host function gives the same bits)."""
    _cuda_contig(out)
    _check(lib().nv_random_fill(_p(out), dt(out), out.numel(), ctypes.c_ulonglong(key & (2**64 - 1)),
                                mean, std, _stream()), "random_fill")


def embedding(ids, table, out, err: ErrorFlag, feed=None) -> None:
    """``feed``: int32 tokens that negative ids point into (id ``-(r + 1)`` reads ``feed[r]``)."""
    _cuda_contig(ids, table, out, feed)
    _i32(ids, feed)
    T, (V, H) = ids.numel(), table.shape
    _need(out.dtype == torch.float32 and out.shape == (T, H), "embedding: out must be float32 [T, H]")
    _check(lib().nv_embedding(_p(ids), _p(feed), _p(table), dt(table), _p(out), T, H, V,
                              _p(err.t), _stream()), "embedding")


def add_rmsnorm(x, branch, w, eps: float, out, out32=None, *, mix=None) -> None:
    """x (+= branch); out = rmsnorm(x) * w; optional float32 copy of out.

    ``mix`` = (rows, index, weight, dense, gate_logit) gives the branch as a sum that has not been taken yet:
    ``sigmoid(gate_logit[t]) * dense[t] + sum_r weight[t, r] * rows[index[t, r]]`` (dense and gate_logit may be
    None); it is summed inside the kernel instead of by ``moe_combine`` first."""
    _cuda_contig(x, branch, w, out, out32)
    T, H = x.shape
    _need(x.dtype == torch.float32, "add_rmsnorm: the residual stream is float32")
    _need(branch is None or (branch.dtype == torch.float32 and branch.shape == x.shape),
          "add_rmsnorm: branch must be float32 and shaped like x")
    _need(w.numel() == H and out.shape == x.shape, "add_rmsnorm: shape mismatch")
    _need(out32 is None or (out32.dtype == torch.float32 and out32.shape == x.shape), "add_rmsnorm: out32")
    rows = index = weight = dense = gate = None
    R, gate_ld = 0, 1
    if mix is not None:
        _need(branch is None, "add_rmsnorm: a branch or a mix, not both")
        rows, index, weight, dense, gate = mix
        _cuda_contig(rows, index, weight, dense)
        R = index.shape[1]
        _need(R <= ADD_RMSNORM_MAX_MIX, f"add_rmsnorm: at most {ADD_RMSNORM_MAX_MIX} rows are mixed per token")
        _need(rows.dtype == torch.float32 and rows.shape[1] == H and weight.dtype == torch.float32
              and index.dtype == torch.int32 and index.shape == (T, R) and weight.shape == (T, R),
              "add_rmsnorm: mix shapes")
        _need(dense is None or (dense.dtype == torch.float32 and dense.shape == x.shape), "add_rmsnorm: mix dense term")
        if gate is not None:
            _need(gate.dtype == torch.float32, "add_rmsnorm: gate logits are float32")
            gate_ld = gate.stride(0) if gate.dim() >= 1 else 1
    if H % 4 == 0:
        for t_ in (x, branch, out, out32, rows, dense):
            _need(t_ is None or t_.data_ptr() % 16 == 0, "add_rmsnorm: rows must start on 16-byte boundaries")
    _check(lib().nv_add_rmsnorm(_p(x), _p(branch), _p(w), dt(w), eps, _p(out), dt(out),
                                _p(out32), T, H, _p(rows), _p(index), _p(weight), R, _p(dense),
                                _p(gate), gate_ld, _stream()), "add_rmsnorm")


ADD_RMSNORM_MAX_MIX = 64


def gemm_plain(a, w, out, *, bias=None, a_rows=None, swiglu=False, M=None, tiles=None) -> None:
    """out[m, :] = a[a_rows[m] or m, :] @ w.T (+ bias), or silu(gate) * up with ``swiglu``.

    ``tiles`` = (tile_expert, tile_row0, tile_rows, num_tiles) selects the grouped form, where w is
    [E, rows, K]."""
    _cuda_contig(w, bias, a_rows)
    _need(a.stride(-1) == 1 and out.stride(-1) == 1, "gemm: rows must be dense")
    K = a.shape[1]
    grouped = tiles is not None
    n_rows_w = w.shape[-2]
    _need(w.shape[-1] == K, f"gemm: inner sizes differ ({K} vs {w.shape[-1]})")
    N = n_rows_w // 2 if swiglu else n_rows_w
    _need(not swiglu or n_rows_w % 2 == 0, "gemm: swiglu needs an even number of weight rows")
    if M is None:
        M = a_rows.numel() if a_rows is not None else a.shape[0]
    _need(out.shape[0] >= M and out.shape[1] == N, f"gemm: out is {tuple(out.shape)}, need [{M}, {N}]")
    _i32(a_rows)
    if grouped:
        te, tr0, tr, nt = tiles
        _i32(te, tr0, tr, nt)
        stride = w.stride(0)
        max_tiles = te.numel()
    else:
        te = tr0 = tr = nt = None
        stride = 0
        max_tiles = 0
    if bias is not None:
        _need(bias.numel() == N, "gemm: bias length")
    _check(lib().nv_gemm_plain(_p(a), dt(a), a.stride(0), _p(a_rows),
                               _p(w), dt(w), stride,
                               _p(bias), (dt(bias) if bias is not None else 0),
                               _p(out), dt(out), out.stride(0),
                               M, N, K, (1 if swiglu else 0),
                               _p(te), _p(tr0), _p(tr), _p(nt), max_tiles, _stream()), "gemm_plain")


def rowdot(a, w, out, wide: bool = False) -> None:
    """out[t, n] = a[t, :] . w[n, :] for float32 rows and a short matrix (float32 or bfloat16), float32 out.
    ``wide``: the many-rows kernel (another summation order; see small_ops.cu)."""
    _cuda_contig(w)
    _need(a.dtype == torch.float32 and out.dtype == torch.float32 and a.stride(1) == 1 and out.stride(1) == 1,
          "rowdot: float32 rows")
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (T, N), "rowdot: shapes")
    scratch = None
    if wide:        # a long K is cut into ranges whose sums a second kernel adds
        n = int(lib().nv_rowdot_scratch_floats(T, N, K, 1))
        if n:
            scratch = torch.empty(n, dtype=torch.float32, device=a.device)
    _check(lib().nv_rowdot(_p(a), a.stride(0), _p(w), dt(w), _p(out), out.stride(0),
                           T, N, K, (1 if wide else 0), _p(scratch), _stream()), "rowdot")


def attention_decode_usable(k_cache, D: int) -> bool:
    return bool(lib().nv_attention_decode_usable(D, k_cache.shape[2], dt(k_cache)))


def attention_decode(qkv, k_cache, v_cache, block_table, row_entry, positions, scale: float, window: int, out,
                     Hq: int, Hkv: int, D: int, max_context: int, rows=None, err=None) -> None:
    """One query row per request (``rows``: which batch rows; None = all) against its paged keys."""
    _cuda_contig(qkv, k_cache, v_cache, block_table, row_entry, positions, out, rows)
    _i32(block_table, row_entry, positions, rows)
    R = qkv.shape[0] if rows is None else rows.numel()
    page = k_cache.shape[2]
    L = lib()
    splits = L.nv_attention_decode_splits(R, Hq, Hkv, max_context, num_sms())
    scratch = counts = None
    if splits > 1:
        scratch = torch.empty(R * Hq * splits * (D + 2), dtype=torch.float32, device=qkv.device)
        counts = _split_counts(qkv.device)
    _check(L.nv_attention_decode(_p(qkv), dt(qkv), qkv.shape[1], _p(k_cache), _p(v_cache),
                                 dt(k_cache), _p(block_table), block_table.shape[1], _p(row_entry),
                                 _p(positions), _p(rows), R, scale, window, _p(out),
                                 dt(out), Hq, Hkv, D, page, k_cache.shape[0],
                                 splits, _p(scratch), _p(err.t if err is not None else _global_err().t),
                                 _p(counts), (counts.numel() if counts is not None else 0), _stream()),
           "attention_decode")


_counts = {}


def _split_counts(device):
    """Zeros that the decode attention kernel counts finished splits in (and sets back to zero itself): one array
    per device, for kernels that run one after the other, as a step's do."""
    key = torch.device(device)
    if key not in _counts:
        _counts[key] = torch.zeros(1 << 16, dtype=torch.int32, device=key)
    return _counts[key]


def attention_prefill_tile_rows() -> int:
    return int(lib().nv_attention_prefill_tile_rows())


def attention_prefill(qkv, k_cache, v_cache, block_table, cu_rows, entry_pos0, max_tiles: int, scale: float,
                      window: int, out, Hq: int, Hkv: int, D: int, err=None, min_rows: int = 1,
                      kernel: str = "auto") -> None:
    """bfloat16 rows of any mix of portions against their paged keys: the tcgen05 kernel for head sizes 64 and
    128 and pages of 16, 32 or 64 keys, else the mma.sync kernel (``kernel="mma"`` asks for that one).  Entries
    with fewer than ``min_rows`` rows are skipped and their rows of ``out`` left as they are."""
    _cuda_contig(qkv, k_cache, v_cache, block_table, cu_rows, entry_pos0, out)
    _i32(block_table, cu_rows, entry_pos0)
    _need(qkv.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_prefill: bfloat16 only")
    _need(out.shape == (qkv.shape[0], Hq * D), "attention_prefill: out shape")
    S = entry_pos0.numel()
    L = lib()
    page = k_cache.shape[2]
    _need(kernel in ("auto", "mma"), "attention_prefill: kernel is 'auto' or 'mma'")
    if kernel == "auto" and L.nv_attention_prefill_tc_usable(D, page):
        _check(L.nv_attention_prefill_tc(_p(qkv), qkv.shape[1], qkv.shape[0], _p(k_cache), _p(v_cache),
                                         k_cache.shape[0], _p(block_table), block_table.shape[1],
                                         _p(cu_rows), _p(entry_pos0), S, max_tiles, scale,
                                         window, _p(out), Hq, Hkv, D, page,
                                         min_rows, _p(err.t if err is not None else _global_err().t),
                                         _stream()),
               "attention_prefill_tc")
        return
    _check(L.nv_attention_prefill(_p(qkv), qkv.shape[1], _p(k_cache), _p(v_cache), _p(block_table),
                                  block_table.shape[1], _p(cu_rows), _p(entry_pos0), S,
                                  max_tiles, scale, window, _p(out), Hq, Hkv,
                                  D, page, min_rows, _stream()), "attention_prefill")


def gemm_plain_tile_m() -> int:
    return int(lib().nv_gemm_plain_tile_m())


def rope_store(qkv, positions, inv_freq, rotary_dim: int, k_cache, v_cache, block_table, row_entry,
               Hq: int, Hkv: int, D: int, write_kv: bool, err: ErrorFlag, rot_positions=None, pair_axis=None) -> None:
    """Turns q and k by their positions and writes k and v to their pages.  ``positions`` [T] are the rows' places
    in their sequences (they pick the cache slot, and the angle unless ``rot_positions`` is given).
    ``rot_positions`` [T] or [T, axes] int32: the coordinates that the pairs are turned by instead, and
    ``pair_axis`` [rotary_dim / 2] int32: which coordinate turns which pair (None: the first)."""
    _cuda_contig(qkv, positions, inv_freq, k_cache, v_cache, block_table, row_entry, rot_positions, pair_axis)
    _i32(positions, block_table, row_entry, rot_positions, pair_axis)
    T = qkv.shape[0]
    axes = 0
    if rot_positions is not None:
        axes = 1 if rot_positions.dim() == 1 else rot_positions.shape[1]
        _need(rot_positions.shape[0] == T and axes >= 1, "rope_store: one row of coordinates per row")
    _need(pair_axis is None or (rot_positions is not None and pair_axis.numel() >= rotary_dim // 2),
          "rope_store: pair_axis needs rot_positions and one entry per pair")
    _need(qkv.shape[1] == (Hq + 2 * Hkv) * D, "rope_store: qkv width")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() >= rotary_dim // 2, "rope_store: inv_freq")
    page = k_cache.shape[2]
    _need(k_cache.shape[1:] == (Hkv, page, D) and v_cache.shape == k_cache.shape, "rope_store: cache shape")
    _check(lib().nv_rope_store(_p(qkv), dt(qkv), _p(positions), _p(rot_positions), axes, _p(pair_axis),
                               _p(inv_freq), rotary_dim,
                               _p(k_cache), _p(v_cache), dt(k_cache), _p(block_table),
                               block_table.shape[1], _p(row_entry), T, Hq, Hkv,
                               D, page, (1 if write_kv else 0), _p(err.t), _stream()),
           "rope_store")


def paged_attention_plain(qkv, k_cache, v_cache, block_table, row_entry, positions, scale: float, window: int,
                          out, Hq: int, Hkv: int, D: int) -> None:
    _cuda_contig(qkv, k_cache, v_cache, block_table, row_entry, positions, out)
    _i32(block_table, row_entry, positions)
    T = qkv.shape[0]
    page = k_cache.shape[2]
    _need(out.shape == (T, Hq * D), "attention: out shape")
    _check(lib().nv_paged_attention_plain(_p(qkv), dt(qkv), qkv.shape[1], _p(k_cache), _p(v_cache),
                                          dt(k_cache), _p(block_table), block_table.shape[1],
                                          _p(row_entry), _p(positions), scale, window, _p(out),
                                          dt(out), T, Hq, Hkv, D, page,
                                          _stream()), "paged_attention_plain")


def router_topk(logits, K: int, renorm: bool, idx, score, C: int = 0, gate_logit=None) -> None:
    """``logits`` may be a column slice of a wider float32 matrix (rows ``stride(0)`` apart).  With ``C`` the
    rows of ``idx``/``score`` are K + C wide: C always-on experts E..E+C-1 weighted sigmoid(gate_logit)."""
    _cuda_contig(idx, score)
    _need(logits.is_cuda and logits.stride(1) == 1, "router: logits rows must be dense")
    T, E = logits.shape
    _need(logits.dtype == torch.float32 and score.dtype == torch.float32, "router: float32 logits and scores")
    _i32(idx)
    _need(idx.shape == (T, K + C) and score.shape == (T, K + C), "router: output shapes")
    _need(C == 0 or (gate_logit is not None and gate_logit.dtype == torch.float32), "router: gate logits")
    _check(lib().nv_router_topk(_p(logits), logits.stride(0), T, E, K,
                                (1 if renorm else 0), _p(idx), _p(score), C, _p(gate_logit),
                                (gate_logit.stride(0) if gate_logit is not None else 0), _stream()),
           "router_topk")


class TileList:
    """Tiles (expert, first row, rows) over an expert-sorted row list, cut by ``tile_m`` rows."""

    def __init__(self, TK: int, E: int, tile_m: int, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.tile_m = tile_m
        self.max_tiles = max(1, min(TK, (TK + tile_m - 1) // tile_m + E))
        self.tile_expert = torch.empty(self.max_tiles, **i32)
        self.tile_row0 = torch.empty(self.max_tiles, **i32)
        self.tile_rows = torch.empty(self.max_tiles, **i32)
        self.num_tiles = torch.zeros(1, **i32)

    @property
    def arrays(self):
        return (self.tile_expert, self.tile_row0, self.tile_rows, self.num_tiles)


class MoeAlignment:
    """Device buffers of one expert permutation (sizes fixed by T*K and E): counts and offsets per expert,
    the sorted pairs, and one or two tile lists over them (``tile_m2``: a second list cut by another tile
    size, for a product that prefers it; 0 = none)."""

    def __init__(self, TK: int, E: int, tile_m: int, device, tile_m2: int = 0):
        i32 = dict(dtype=torch.int32, device=device)
        self.TK, self.E = TK, E
        self.primary = TileList(TK, E, tile_m, device)
        self.secondary = TileList(TK, E, tile_m2, device) if tile_m2 and tile_m2 != tile_m else None
        self.counts = torch.empty(E, **i32)
        self.offsets = torch.empty(E + 1, **i32)
        self.sorted_token = torch.empty(max(TK, 1), **i32)
        self.pair_pos = torch.empty(max(TK, 1), **i32)

    # the primary list under the names the kernels' wrappers use
    tile_m = property(lambda self: self.primary.tile_m)
    max_tiles = property(lambda self: self.primary.max_tiles)
    tile_expert = property(lambda self: self.primary.tile_expert)
    tile_row0 = property(lambda self: self.primary.tile_row0)
    tile_rows = property(lambda self: self.primary.tile_rows)
    num_tiles = property(lambda self: self.primary.num_tiles)

    @property
    def tiles(self):
        return self.primary.arrays

    def list_for(self, tile_m: int) -> TileList:
        if self.secondary is not None and self.secondary.tile_m == tile_m:
            return self.secondary
        return self.primary


def moe_align(idx, K: int, al: MoeAlignment, err: ErrorFlag, spread_last: int = 0, static_last: int = 0,
              zero=None) -> None:
    """``spread_last``: the tiles of the last so many experts (ones that every row visits) are spread evenly through
    the tile lists instead of standing at their end.  ``static_last`` instead: those experts' pairs sit in row order
    at the end of the permutation and get no tiles (``StaticTiles`` lists them; they can run before the routing).
    ``zero``: a few int32 that the kernel also sets to 0 (the tile counters of the products that follow it)."""
    _cuda_contig(idx)
    _i32(idx)
    T = idx.numel() // K
    _need(T * K == al.TK, "moe_align: buffers were sized for another batch")
    s2 = al.secondary
    _check(lib().nv_moe_align(_p(idx), T, K, al.E, al.tile_m, _p(al.counts),
                              _p(al.offsets), _p(al.sorted_token), _p(al.pair_pos),
                              _p(al.tile_expert), _p(al.tile_row0), _p(al.tile_rows), _p(al.num_tiles), _p(err.t),
                              (s2.tile_m if s2 else 0), _p(s2.tile_expert if s2 else None), _p(s2.tile_row0 if s2 else None),
                              _p(s2.tile_rows if s2 else None), _p(s2.num_tiles if s2 else None), spread_last,
                              static_last, _p(zero), (zero.numel() if zero is not None else 0), _stream()),
           "moe_align")


def moe_route_small_usable(T: int, E: int, K: int, C: int, H: int) -> bool:
    return bool(lib().nv_moe_route_small_usable(T, E, K, C, H))


def moe_route_small(logits, K: int, renorm: bool, C: int, gate_logit, idx, score, al: "MoeAlignment", err, x=None,
                    static: bool = False, zero=None):
    """Top-k, expert permutation and (with ``x``, bfloat16 rows) the expert-sorted copy of x, in one launch.
    Returns the sorted copy or None.  ``static``: the C always-on experts' pairs sit in row order at the end of
    the permutation and get no tiles (``static_tiles`` lists them; they can then run before the routing).
    ``zero``: a few int32 that the kernel also sets to 0 (the tile counters of the products that follow it)."""
    T, E = logits.shape
    KT = K + C
    _need(idx.shape == (T, KT) and score.shape == (T, KT) and al.TK == T * KT and al.E == E + C, "route: sizes")
    _need(al.secondary is None, "route: the one-launch routing builds one tile list")
    xs = None
    H = 8
    if x is not None:
        _need(x.dtype == torch.bfloat16 and x.is_contiguous(), "route: bfloat16 rows")
        H = x.shape[1]
        xs = torch.empty((T * KT, H), dtype=x.dtype, device=x.device)
    _check(lib().nv_moe_route_small(_p(logits), logits.stride(0), T, E, K,
                                    (1 if renorm else 0), C, _p(gate_logit),
                                    (gate_logit.stride(0) if gate_logit is not None else 0), _p(idx),
                                    _p(score), al.tile_m, _p(al.counts), _p(al.offsets), _p(al.sorted_token),
                                    _p(al.pair_pos), _p(al.tile_expert), _p(al.tile_row0), _p(al.tile_rows),
                                    _p(al.num_tiles), _p(err.t), _p(x), _p(xs), H, (C if static else 0),
                                    _p(zero), (zero.numel() if zero is not None else 0), _stream()), "moe_route_small")
    return xs


class StaticTiles:
    """The tiles of C experts E .. E + C - 1 that each take all T rows, in row order, their segments behind the
    T * K routed pairs: what ``moe_route_small(static=True)`` leaves out of its list."""

    def __init__(self, T: int, K: int, E: int, C: int, device):
        self.tile_m = 16 if T <= 16 else (32 if T <= 32 else (64 if T <= 64 else 128))
        experts, row0, rows = [], [], []
        for c in range(C):
            for r in range(0, T, self.tile_m):
                experts.append(E + c)
                row0.append(T * K + c * T + r)
                rows.append(min(self.tile_m, T - r))
        i32 = dict(dtype=torch.int32, device=device)
        self.max_tiles = len(experts)
        self.tile_expert = torch.tensor(experts, **i32)
        self.tile_row0 = torch.tensor(row0, **i32)
        self.tile_rows = torch.tensor(rows, **i32)
        self.num_tiles = torch.tensor([len(experts)], **i32)
        self.x_rows = (T * K, T)


def moe_combine(y, pair_pos, score, shared, gate_logit, out) -> None:
    """``gate_logit``: [T] or a [T, 1] column slice of a wider float32 matrix."""
    _cuda_contig(y, pair_pos, score, shared, out)
    T, K = score.shape
    gate_ld = 1 if gate_logit is None else (gate_logit.stride(0) if gate_logit.dim() >= 1 else 1)
    H = out.shape[1]
    for t in (y, score, shared, gate_logit, out):
        _need(t is None or t.dtype == torch.float32, "moe_combine: float32 tensors")
    _check(lib().nv_moe_combine(_p(y), _p(pair_pos), _p(score), _p(shared), _p(gate_logit), gate_ld,
                                _p(out), T, K, H, _stream()), "moe_combine")


def silu_mul(gu, out) -> None:
    _cuda_contig(gu, out)
    rows, I2 = gu.shape
    _need(out.shape == (rows, I2 // 2), "silu_mul: out shape")
    _check(lib().nv_silu_mul(_p(gu), dt(gu), _p(out), dt(out), rows, I2 // 2,
                             _stream()), "silu_mul")


def gather_rows(src, rows, dst) -> None:
    _cuda_contig(src, rows, dst)
    _i32(rows)
    _need(src.dtype == dst.dtype and dst.shape == (rows.numel(), src.shape[1]), "gather_rows: shapes")
    _check(lib().nv_gather_rows(_p(src), dt(src), _p(rows), _p(dst), rows.numel(),
                                src.shape[1], _stream()), "gather_rows")


def reset_fresh_state(state, entry_slot, entry_pos0) -> None:
    """Zeroes ``state[slot]`` (``state``: [slots, ...]) for every entry whose first position is 0."""
    _cuda_contig(state, entry_slot, entry_pos0)
    _i32(entry_slot, entry_pos0)
    slots = state.shape[0]
    slot_bytes = (state.numel() // max(slots, 1)) * state.element_size()
    _need(slot_bytes % 4 == 0, "reset_fresh_state: a slot's bytes must be a multiple of four")
    _check(lib().nv_reset_fresh_state(_p(state), slot_bytes, slots, _p(entry_slot), _p(entry_pos0),
                                      entry_slot.numel(), _stream()), "reset_fresh_state")


def sync_block_tables(src, lens, rows, entry_slot, tables, step_tables, S: int) -> None:
    """``tables`` [slots, max_blocks] takes in the rows that travelled with the step (``rows[src[e]]`` for the
    entries with ``src[e]`` >= 0) and ``step_tables[e, :lens[e]]`` becomes entry e's table, for e < S."""
    _cuda_contig(src, lens, rows, entry_slot, tables, step_tables)
    _i32(src, lens, rows, entry_slot, tables, step_tables)
    slots, max_blocks = tables.shape
    _need(step_tables.shape == tables.shape and src.numel() >= S and lens.numel() >= S and entry_slot.numel() >= S,
          "sync_block_tables: shapes")
    _check(lib().nv_sync_block_tables(_p(src), _p(lens), _p(rows), _p(entry_slot), _p(tables), _p(step_tables),
                                      S, max_blocks, slots, _stream()), "sync_block_tables")


def delay(micros: int) -> None:
    """Keeps the current stream busy for about ``micros`` microseconds (at most 200,000); for measurements that
    want a step's launches queued before the GPU starts on them."""
    code = lib().nv_delay(int(micros), _stream())
    if code:
        raise KernelError(f"delay: {_ERR.get(code, code)}")


def sample(logits, temperature, u, out) -> None:
    """One token per row: greedy where temperature <= 0, else inverse-CDF with the given u in [0,1)."""
    _cuda_contig(logits, temperature, u, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and temperature.dtype == torch.float32 and u.dtype == torch.float64,
          "sample: logits/temperature float32, u float64")
    _i32(out)
    _need(temperature.numel() == R and u.numel() == R and out.numel() == R, "sample: one entry per row")
    _check(lib().nv_sample(_p(logits), R, V, _p(temperature), _p(u), _p(out), _stream()), "sample")


def sample_nucleus(logits, params, recent, recent_off, out) -> None:
    """One token per row by nucleus (top-p) sampling with a repetition penalty (include/nanovllm/sampler.hpp:46-88).
    ``params``: float64 [R, 4] = (temperature, top_p, penalty, u) per row; ``recent``: int32 ids whose scores are
    divided by the row's penalty, row r's being ``recent[recent_off[r]:recent_off[r + 1]]``."""
    _cuda_contig(logits, params, recent, recent_off, out)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and params.dtype == torch.float64 and params.shape == (R, 4),
          "sample_nucleus: logits float32 [R, V], params float64 [R, 4]")
    _i32(recent, recent_off, out)
    _need(recent_off.numel() == R + 1 and out.numel() == R, "sample_nucleus: one entry per row")
    work = torch.empty_like(logits)
    _check(lib().nv_sample_nucleus(_p(logits), _p(work), R, V, _p(params), _p(recent), _p(recent_off),
                                   _p(out), _stream()), "sample_nucleus")


# ----------------------------------------------------------------------------- fast products
_num_sms = None


def num_sms() -> int:
    global _num_sms
    if _num_sms is None:
        _num_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _num_sms


def _tma_ok(t) -> bool:
    return (t.dtype == torch.bfloat16 and t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all(st % 8 == 0 for st in t.stride()[:-1]))


def gemm_fast_usable(a, w, out, *, bias=None, a_rows=None, swiglu=False, grouped=False) -> bool:
    """Whether the tensor-core product takes these operands; the plain product takes all.

    Both operands bfloat16 with K a multiple of 8 (TMA moves 16-byte units), output float32 or
    bfloat16."""
    if not (_tma_ok(a) and _tma_ok(w) and w.is_contiguous()):
        return False
    if a.shape[-1] % 8 or out.dtype not in _DT or out.stride(-1) != 1:
        return False
    return True


SKINNY_MAX_ROWS = 32               # without SwiGLU; 8 with it
GROUPED_SPLIT_MAX_PAIRS = 16       # grouped products of at most this many (row, expert) pairs may split K


def skinny_usable(a, w, rows: int, swiglu: bool = False) -> bool:
    """Whether the weight-streaming product for a handful of rows (skinny_gemm.cu) takes these operands."""
    return (1 <= rows <= (8 if swiglu else SKINNY_MAX_ROWS) and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and a.stride(-1) == 1 and w.is_contiguous() and a.shape[-1] % 32 == 0 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_gemm(a, w, out, *, bias=None, swiglu=False, rows=None, err=None) -> None:
    """``out[:rows] = a[:rows] @ w.T (+ bias)`` for at most 32 rows (8 with ``swiglu``; default: all rows of ``a``),
    by streaming ``w`` once; ``swiglu`` as in ``gemm_plain``."""
    _cuda_contig(w, bias)
    K = a.shape[-1]
    rows_w = w.shape[0]
    N = rows_w // 2 if swiglu else rows_w
    R = a.shape[0] if rows is None else rows
    _need(skinny_usable(a, w, R, swiglu), "skinny product: operands or row count not supported")
    _need(w.dim() == 2 and w.shape[1] == K and out.shape[1] == N and out.stride(1) == 1 and out.shape[0] >= R,
          "skinny product: shapes")
    _need(bias is None or (not swiglu and bias.numel() == N), "skinny product: bias")
    _check(lib().nv_skinny_gemm(_p(a), a.stride(0), R, _p(w), N, K,
                                _p(bias), (dt(bias) if bias is not None else 0), _p(out), dt(out),
                                out.stride(0), (1 if swiglu else 0), _stream()),
           f"skinny_gemm N={rows_w} K={K}", 0.0, float(w.element_size() * rows_w * K))


def grouped_token_tile(TK: int, E: int, swiglu: bool = False) -> int:
    """Token tile of the grouped tensor-core product for TK (row, expert) pairs over E experts: the most rows of
    one expert that a CTA takes at once.  The product's instruction is as wide as a tile's rows need (in steps
    of 16) and so are its token loads (in boxes of 64 rows), so a short last tile of an expert is cheap.  Tiles
    of 256 rows are accepted but lose (one accumulator set instead of two: 23.9 against 20.5 ms for a prompt of
    2,048 tokens).  ``swiglu`` lets the two products of an expert layer choose differently; they agree."""
    avg = (TK + E - 1) // E
    if avg <= 12:
        return 16
    if avg <= 24:
        return 32
    return 128 if avg >= 96 else 64


def permute_rows(src, rows, R=None):
    """bfloat16 rows of ``src`` gathered in the order of ``rows``."""
    R = rows.numel() if R is None else R
    dst = torch.empty((R, src.shape[1]), dtype=src.dtype, device=src.device)
    _check(lib().nv_permute_rows_bf16(_p(src), _p(rows), _p(dst), R, src.shape[1], _stream()),
           "permute_rows")
    return dst


def gemm_fast(a, w, out, *, bias=None, a_rows=None, swiglu=False, M=None, err=None, splits=None) -> None:
    """Tensor-core form of ``gemm_plain`` (dense)."""
    if a_rows is not None:
        a = permute_rows(a, a_rows, M)
    M = a.shape[0] if M is None else M
    K = a.shape[1]
    rows_w = w.shape[0]
    N = rows_w // 2 if swiglu else rows_w
    L = lib()
    n_tile = L.nv_tc_gemm_token_tile(M, (1 if swiglu else 0))
    if splits is None:
        splits = L.nv_tc_gemm_splits(M, N, K, n_tile, num_sms())
    scratch = None
    if splits > 1:
        scratch = torch.empty((splits, M, 2 * N if swiglu else N), dtype=torch.float32, device=a.device)
    _check(L.nv_tc_gemm(_p(a), a.stride(0), M, _p(w), rows_w, N, K,
                        _p(bias), (dt(bias) if bias is not None else 0), _p(out), dt(out),
                        out.stride(0), (1 if swiglu else 0), n_tile, splits,
                        _p(scratch), _p(None), _p(None), _p(None), _p(None), 0, 0,
                        _p(err.t if err is not None else _global_err().t), _early(), 0, 0,
                        0, _p(None), 0, _stream()), f"tc_gemm N={rows_w} K={K}", 2.0 * M * rows_w * K,
           w.element_size() * rows_w * K + a.element_size() * M * K + out.element_size() * M * N)


def gemm_fast_grouped(a, w, out, align, *, a_rows=None, swiglu=False, err=None, tiles=None, tiles_ready=False,
                      x_rows=None, max_ctas: int = 0, counter=None) -> None:
    """Tensor-core form of the grouped ``gemm_plain``; ``tiles`` (a TileList of ``align``) picks the token tile.

    ``x_rows`` = (sub, mod): a tile whose outputs are rows r.. takes rows ``(r - sub) % mod``.. of ``a`` (several
    experts that all take the same few rows, their outputs one segment after the other).

    ``max_ctas`` > 0 caps the grid, for a product that runs beside other kernels and must leave them room.
    ``counter`` (one int32 on the device, 0 between launches, used by one product at a time): the CTAs take their
    tiles from it instead of by position, so a CTA that starts late takes fewer.

    ``tiles_ready``: the tile lists were complete before the kernel that precedes this product on the stream
    started, so the product may start beside that kernel and fetch its first weights (it reads the lists at
    once).  With ``a_rows`` that holds by itself: the row copy comes between the routing and the product."""
    if a_rows is not None:
        a = permute_rows(a, a_rows, align.TK)
        tiles_ready = True
    K = a.shape[1]
    E, rows_w = w.shape[0], w.shape[1]
    N = rows_w // 2 if swiglu else rows_w
    tl = tiles if tiles is not None else align.primary
    _need(tl.tile_m in (16, 32, 64, 128, 256), "grouped product: token tile must be 16, 32, 64, 128 or 256")
    x_sub, x_mod = x_rows if x_rows is not None else (0, 0)
    _need(out.shape[0] >= align.TK and (x_mod or a.shape[0] <= align.TK), "grouped product: row counts")
    # One or two rows: the list has few tiles (an expert's matrix is a dozen tiles of 128 features), which would
    # leave most multiprocessors idle and each CTA with a long stream of its own; K is then split as in a small
    # dense product and a finishing kernel adds the parts.  (Measured per decode step: batch 1 492 -> 504 tokens/s;
    # with more rows the parts' traffic and the crowding of the other stream's product cost more than the split
    # gains: batch 4 1,464 -> 1,420, batch 64 6,219 -> 5,300.)
    splits, scratch = 1, None
    k_steps = (K + 63) // 64
    ctas = tl.max_tiles * ((N + 127) // 128)
    if counter is None and align.TK <= GROUPED_SPLIT_MAX_PAIRS and ctas < num_sms() and k_steps >= 8:
        splits = max(1, min(2 * num_sms() // ctas, k_steps // 4, 16))
        if splits > 1:
            scratch = torch.empty((splits, align.TK, 2 * N if swiglu else N), dtype=torch.float32, device=a.device)
    _check(lib().nv_tc_gemm(_p(a), a.stride(0), a.shape[0], _p(w), E * rows_w, N,
                            K, _p(None), 0, _p(out), dt(out), out.stride(0),
                            (1 if swiglu else 0), tl.tile_m, splits, _p(scratch), _p(tl.tile_expert),
                            _p(tl.tile_row0), _p(tl.tile_rows), _p(tl.num_tiles), tl.max_tiles,
                            rows_w, _p(err.t if err is not None else _global_err().t),
                            (_early() if tiles_ready else 0), x_sub, x_mod, max_ctas,
                            _p(counter), align.TK, _stream()),
           f"tc_gemm_grouped N={rows_w} K={K}")


_dependent_launch = 1


def set_dependent_launch(on: bool) -> None:
    """Whether a step's kernels are launched as programmatic dependents of one another (the default) or the
    ordinary way; for comparisons."""
    global _dependent_launch
    _dependent_launch = 1 if on else 0
    lib().nv_set_dependent_launch(_dependent_launch)


def _early() -> int:
    return _dependent_launch


_gerr = None


def _global_err() -> "ErrorFlag":
    global _gerr
    if _gerr is None:
        _gerr = ErrorFlag(torch.device("cuda", torch.cuda.current_device()))
    return _gerr
