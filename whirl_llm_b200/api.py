"""ctypes bindings of libwhirl_b200.so over torch tensors (device memory and streams only; all arithmetic is in the
library).  Function names and argument meaning follow include/whirl_b200.h, which follows the reference's kernel and
ServerModel interfaces."""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("WHIRL_B200_LIB") or os.path.join(_HERE, "libwhirl_b200.so")

F32, BF16 = 0, 1
ROW_DONE, ROW_ESCALATE, ROW_OPEN_TAIL = 0, 1, 2
CNT_ESCALATED, CNT_OPEN_TAIL, CNT_UNRESOLVED, CNT_TIMEOUT, CNT_REDO, CNT_NAN_ROWS, CNT_WORDS = 0, 1, 2, 3, 4, 5, 8
ERR_TIMEOUT = 5
MAX_K, STREAM_MAX_K, MAX_HIST, Q_WORDS, Q_MAX, CTL_WORDS = 16384, 1024, 4096, 72, 32, 64
STATIC_MAX_ROWS = 256


class WhirlError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"whirl_b200 status {status}: {msg}")
        self.status = status


class SampleParams(C.Structure):
    _fields_ = [("inv_t", C.c_void_p), ("top_k", C.c_void_p), ("top_p", C.c_void_p), ("min_p", C.c_void_p),
                ("greedy", C.c_void_p), ("u", C.c_void_p), ("race_key", C.c_void_p), ("hist", C.c_void_p),
                ("hist_len", C.c_void_p), ("hist_stride", C.c_int64), ("rep", C.c_void_p), ("pres", C.c_void_p),
                ("freq", C.c_void_p)]


class DSampArgs(C.Structure):
    _fields_ = [("on", C.c_void_p), ("top_k", C.c_void_p), ("qoff", C.c_void_p), ("inv_t", C.c_void_p), ("top_p", C.c_void_p),
                ("min_p", C.c_void_p), ("key_lo", C.c_void_p), ("key_hi", C.c_void_p)]


class RelaxParams(C.Structure):
    _fields_ = [("k", C.c_uint32), ("alpha", C.c_float), ("eps", C.c_float), ("delta", C.c_float)]


class AcceptIn(C.Structure):
    _fields_ = [("tokens", C.c_void_p), ("drafts", C.c_void_p), ("draft_stride", C.c_int64), ("nd", C.c_void_p), ("row0", C.c_void_p),
                ("greedy", C.c_void_p), ("relax_on", C.c_void_p), ("next", C.c_void_p), ("hist", C.c_void_p),
                ("hist_stride", C.c_int64), ("hist_len", C.c_void_p), ("rk_ids", C.c_void_p), ("rk_vals", C.c_void_p),
                ("rk_stats", C.c_void_p), ("rk", C.c_int32), ("kept_cap", C.c_int32), ("kept_ids", C.c_void_p),
                ("kept_p", C.c_void_p), ("n_kept", C.c_void_p), ("closed", C.c_void_p), ("stats", C.c_void_p), ("x", C.c_void_p),
                ("dtype", C.c_int32), ("n", C.c_int32), ("inv_t", C.c_void_p)]


class SampleOut(C.Structure):
    _fields_ = [("token", C.c_void_p), ("status", C.c_void_p), ("n_kept", C.c_void_p), ("closed", C.c_void_p),
                ("stats", C.c_void_p), ("kept_ids", C.c_void_p), ("kept_p", C.c_void_p), ("kept_cap", C.c_int32),
                ("counters", C.c_void_p)]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m whirl_llm_b200.build` "
                          "(there is no fallback implementation)")
    lib = C.CDLL(LIB_PATH)
    vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    sigs = {
        "whirl_status_string": (C.c_char_p, [i]),
        "whirl_last_error": (C.c_char_p, []),
        "whirl_version": (i, []),
        "whirl_workspace_bytes": (sz, [i, i]),
        "whirl_argmax": (i, [vp, i, i, vp, vp, vp, i, vp, sz, vp]),
        "whirl_argmax_rows": (i, [vp, i, i, i, vp, vp, sz, vp]),
        "whirl_argmax_rows_to": (i, [vp, i, i, i, vp, vp, vp, sz, vp]),
        "whirl_argmax_rows_static": (i, [vp, i, i, i, vp, vp]),
        "whirl_argmax_prob": (i, [vp, i, i, i, vp, vp, vp, sz, vp]),
        "whirl_draft_pick": (i, [vp, i, i, vp, vp, vp, i, i, f, vp, vp, sz, vp]),
        "whirl_draft_pick_rows": (i, [vp, i, i, i, vp, vp, i, i, f, vp, vp, sz, vp]),
        "whirl_topk_rows": (i, [vp, i, i, i, i, f, vp, vp, vp, vp, vp, sz, vp]),
        "whirl_draft_sample_rows": (i, [vp, i, i, i, vp, vp, i, vp, C.POINTER(DSampArgs), vp, vp]),
        "whirl_accept_tokens": (i, [vp, vp, i, vp, vp, i, vp, vp, vp]),
        "whirl_spec_workspace_bytes": (sz, [i, i]),
        "whirl_spec_accept_residual": (i, [vp, vp, i, i, i, i, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
        "whirl_topk_rows_shard": (i, [vp, i, i, i, i, i, f, vp, vp, vp, vp, vp, sz, vp]),
        "whirl_merge_sample_rows": (i, [vp, vp, vp, i, i, i, i, C.POINTER(SampleParams), C.POINTER(SampleOut), vp]),
        "whirl_sample_rows": (i, [vp, i, i, i, C.POINTER(SampleParams), C.POINTER(SampleOut), vp, sz, vp]),
        "whirl_sample_rows_host": (i, [vp, i, i, i, C.POINTER(SampleParams), C.POINTER(SampleOut), i]),
        "whirl_host_release": (None, []),
        "whirl_host_last_error": (C.c_char_p, []),
        "whirl_launch_counts": (None, [vp, i]),
        "whirl_check": (i, [vp, sz, i, vp, vp]),
        "whirl_shard_block_words": (sz, [i, i]),
        "whirl_merge_sample_rows_packed": (i, [vp, i, i, i, i, C.POINTER(SampleParams), C.POINTER(SampleOut), vp]),
        "whirl_accept_rows": (i, [C.POINTER(AcceptIn), C.POINTER(RelaxParams), i, vp, vp, vp, vp, vp, vp]),
        "whirl_uniform_splitmix": (C.c_double, [C.c_uint64, C.c_uint64, C.c_uint32]),
        "whirl_race_base": (C.c_uint64, [C.c_uint64, C.c_uint64]),
        "whirl_philox4x32_10": (None, [C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
        "whirl_uniform_philox4x32": (C.c_double, [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32]),
        "whirl_fill_draws": (i, [vp, vp, i, i, C.c_uint32, vp, vp, vp]),
        "whirl_test_waits": (None, [C.c_uint32, i]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()
DECLARED = ["whirl_status_string", "whirl_last_error", "whirl_version", "whirl_workspace_bytes", "whirl_argmax",
            "whirl_argmax_rows", "whirl_argmax_rows_static", "whirl_argmax_rows_to", "whirl_argmax_prob", "whirl_draft_pick", "whirl_draft_pick_rows", "whirl_draft_sample_rows", "whirl_accept_tokens", "whirl_spec_workspace_bytes",
            "whirl_spec_accept_residual",
            "whirl_topk_rows", "whirl_topk_rows_shard", "whirl_merge_sample_rows", "whirl_sample_rows", "whirl_sample_rows_host", "whirl_host_release", "whirl_host_last_error",
            "whirl_launch_counts", "whirl_check", "whirl_shard_block_words", "whirl_merge_sample_rows_packed", "whirl_test_waits", "whirl_accept_rows",
            "whirl_uniform_splitmix", "whirl_race_base", "whirl_philox4x32_10", "whirl_uniform_philox4x32", "whirl_fill_draws"]


def _check(status: int):
    if status != 0:
        raise WhirlError(status, (lib.whirl_last_error() or b"").decode())


def _dtype(x: torch.Tensor) -> int:
    if x.dtype == torch.float32:
        return F32
    if x.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"logits must be float32 or bfloat16, got {x.dtype}")


def _rows(x: torch.Tensor):
    if not x.is_cuda:
        raise ValueError("logits must be on a CUDA device (this library has no CPU path)")
    if x.dim() == 1:
        x = x.unsqueeze(0)
    if x.dim() != 2 or x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) != x.shape[1]):
        raise ValueError("logits must be dense rows [rows, n]")
    return x, x.shape[0], x.shape[1]


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(x: torch.Tensor):
    return torch.cuda.current_stream(x.device).cuda_stream


def workspace_bytes(rows: int, n: int) -> int:
    return lib.whirl_workspace_bytes(rows, n)


_ws_cache: dict = {}


def workspace(rows: int, n: int, device) -> torch.Tensor:
    """A cached workspace tensor for (rows, n) on `device` (callers that manage memory pass their own)."""
    device = torch.device(device)
    need = workspace_bytes(rows, n)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _ws_cache[key] = ws
    return ws


def argmax(x, out=None, ids=None, pos=None, advance=0, ws=None):
    x, rows, n = _rows(x)
    assert rows == 1
    out = torch.empty(1, dtype=torch.int32, device=x.device) if out is None else out
    ws = workspace(1, n, x.device) if ws is None else ws
    _check(lib.whirl_argmax(x.data_ptr(), _dtype(x), n, out.data_ptr(), _p(ids), _p(pos), advance, ws.data_ptr(), ws.numel(),
                            _stream(x)))
    return out


def argmax_rows(x, out=None, ws=None):
    x, rows, n = _rows(x)
    out = torch.empty(rows, dtype=torch.int32, device=x.device) if out is None else out
    ws = workspace(rows, n, x.device) if ws is None else ws
    _check(lib.whirl_argmax_rows(x.data_ptr(), _dtype(x), rows, n, out.data_ptr(), ws.data_ptr(), ws.numel(), _stream(x)))
    return out


def argmax_rows_static(x, out=None):
    """The greedy pick with the library's own fixed scratch: no workspace, no allocation by the library (at most
    WHIRL_STATIC_MAX_ROWS rows).  `out` is the caller's."""
    x, rows, n = _rows(x)
    out = torch.empty(rows, dtype=torch.int32, device=x.device) if out is None else out
    _check(lib.whirl_argmax_rows_static(x.data_ptr(), _dtype(x), rows, n, out.data_ptr(), _stream(x)))
    return out


def argmax_rows_to(x, out, dst, ws=None):
    x, rows, n = _rows(x)
    ws = workspace(rows, n, x.device) if ws is None else ws
    _check(lib.whirl_argmax_rows_to(x.data_ptr(), _dtype(x), rows, n, out.data_ptr(), dst.data_ptr(), ws.data_ptr(), ws.numel(),
                                    _stream(x)))
    return out


def argmax_prob(x, ws=None):
    x, rows, n = _rows(x)
    tok = torch.empty(rows, dtype=torch.int32, device=x.device)
    prob = torch.empty(rows, dtype=torch.float32, device=x.device)
    ws = workspace(rows, n, x.device) if ws is None else ws
    _check(lib.whirl_argmax_prob(x.data_ptr(), _dtype(x), rows, n, tok.data_ptr(), prob.data_ptr(), ws.data_ptr(), ws.numel(),
                                 _stream(x)))
    return tok, prob


def draft_pick(x, tok, prob, ctl, r, n_min, p_min, vmap=None, ws=None):
    x, rows, n = _rows(x)
    assert rows == 1
    ws = workspace(1, n, x.device) if ws is None else ws
    _check(lib.whirl_draft_pick(x.data_ptr(), _dtype(x), n, tok.data_ptr(), prob.data_ptr(), ctl.data_ptr(), r, n_min, p_min,
                                _p(vmap), ws.data_ptr(), ws.numel(), _stream(x)))


def draft_pick_rows(x, ctl_all, area, r, n_min, p_min, vmap=None, ws=None):
    x, rows, n = _rows(x)
    ws = workspace(rows, n, x.device) if ws is None else ws
    _check(lib.whirl_draft_pick_rows(x.data_ptr(), _dtype(x), rows, n, ctl_all.data_ptr(), area.data_ptr(), r, n_min, p_min,
                                     _p(vmap), ws.data_ptr(), ws.numel(), _stream(x)))


def draft_sample_rows(x, ctl_all, area, r, on, top_k, qoff, inv_t, top_p, min_p, race_key, qbuf, vmap=None):
    """draft_sample_rows: per-row arrays are device tensors (int32 / float32); race_key int64 holding the uint64 keys."""
    x, rows, n = _rows(x)
    lo = (race_key & 0xFFFFFFFF).to(torch.int32).contiguous()
    hi = ((race_key >> 32) & 0xFFFFFFFF).to(torch.int32).contiguous()
    d = DSampArgs(on=_p(on), top_k=_p(top_k), qoff=_p(qoff), inv_t=_p(inv_t), top_p=_p(top_p), min_p=_p(min_p), key_lo=_p(lo),
                  key_hi=_p(hi))
    _check(lib.whirl_draft_sample_rows(x.data_ptr(), _dtype(x), rows, n, ctl_all.data_ptr(), area.data_ptr(), r, _p(vmap),
                                       C.byref(d), qbuf.data_ptr(), _stream(x)))


def topk_rows(x, K, inv_t=1.0, inv_t_rows=None, ws=None):
    """ids [rows, K] i32, vals [rows, K] f32, stats [rows, 2] f32 (ServerModel::topkRows)."""
    x, rows, n = _rows(x)
    ids = torch.full((rows, K), -1, dtype=torch.int32, device=x.device)
    vals = torch.zeros((rows, K), dtype=torch.float32, device=x.device)
    stats = torch.zeros((rows, 2), dtype=torch.float32, device=x.device)
    ws = workspace(rows, n, x.device) if ws is None else ws
    _check(lib.whirl_topk_rows(x.data_ptr(), _dtype(x), rows, n, K, float(inv_t), _p(inv_t_rows), ids.data_ptr(), vals.data_ptr(),
                               stats.data_ptr(), ws.data_ptr(), ws.numel(), _stream(x)))
    return ids, vals, stats


def shard_block_views(block: torch.Tensor, rows: int, K: int):
    """The ids / vals / stats views of one rank's packed block (int32 tensor of whirl_shard_block_words words)."""
    assert block.dtype == torch.int32 and block.is_contiguous() and block.numel() == lib.whirl_shard_block_words(rows, K)
    ids = block[: rows * K].view(rows, K)
    vals = block[rows * K: 2 * rows * K].view(torch.float32).view(rows, K)
    stats = block[2 * rows * K:].view(torch.float32).view(rows, 2)
    return ids, vals, stats


def topk_rows_shard(x, K, id_offset, inv_t=1.0, inv_t_rows=None, ws=None, out=None):
    """topk_rows of one vocabulary slice with global token ids (ids pre-filled with -1).  out: (ids, vals, stats) to
    write into, e.g. the views of a packed block."""
    x, rows, n = _rows(x)
    if out is None:
        ids = torch.full((rows, K), -1, dtype=torch.int32, device=x.device)
        vals = torch.zeros((rows, K), dtype=torch.float32, device=x.device)
        stats = torch.zeros((rows, 2), dtype=torch.float32, device=x.device)
    else:
        ids, vals, stats = out
        if K > n:
            ids.fill_(-1)
    ws = workspace(rows, n, x.device) if ws is None else ws
    _check(lib.whirl_topk_rows_shard(x.data_ptr(), _dtype(x), rows, n, K, int(id_offset), float(inv_t), _p(inv_t_rows),
                                     ids.data_ptr(), vals.data_ptr(), stats.data_ptr(), ws.data_ptr(), ws.numel(), _stream(x)))
    return ids, vals, stats


@dataclass
class RowParams:
    """Device tensors of per-row sampler settings (None = the library default)."""
    inv_t: Optional[torch.Tensor] = None      # float32
    top_k: Optional[torch.Tensor] = None      # int32
    top_p: Optional[torch.Tensor] = None      # float64
    min_p: Optional[torch.Tensor] = None      # float64
    greedy: Optional[torch.Tensor] = None     # uint8
    u: Optional[torch.Tensor] = None          # float64
    race_key: Optional[torch.Tensor] = None   # int64 holding the uint64 bit pattern
    hist: Optional[torch.Tensor] = None       # int32 [rows, H]
    hist_len: Optional[torch.Tensor] = None   # int32
    rep: Optional[torch.Tensor] = None        # float32
    pres: Optional[torch.Tensor] = None       # float32
    freq: Optional[torch.Tensor] = None       # float32

    _DT = dict(inv_t=torch.float32, top_k=torch.int32, top_p=torch.float64, min_p=torch.float64, greedy=torch.uint8,
               u=torch.float64, race_key=torch.int64, hist=torch.int32, hist_len=torch.int32, rep=torch.float32,
               pres=torch.float32, freq=torch.float32)

    def struct(self, rows: int) -> SampleParams:
        s = SampleParams()
        for k, dt in self._DT.items():
            t = getattr(self, k)
            if t is not None:
                if t.dtype != dt or not t.is_cuda or not t.is_contiguous():
                    raise TypeError(f"{k}: want a contiguous CUDA tensor of {dt}, got {t.dtype} on {t.device}")
                if k != "hist" and t.shape != (rows,):
                    raise ValueError(f"{k}: want shape ({rows},), got {tuple(t.shape)}")
                if k == "hist" and (t.dim() != 2 or t.shape[0] != rows):
                    raise ValueError(f"hist: want [rows, H], got {tuple(t.shape)}")
            setattr(s, k, _p(t))
        s.hist_stride = 0 if self.hist is None else self.hist.shape[1]
        return s


@dataclass
class SampleResult:
    token: torch.Tensor
    status: torch.Tensor
    n_kept: torch.Tensor
    closed: torch.Tensor
    stats: Optional[torch.Tensor]
    kept_ids: Optional[torch.Tensor]
    kept_p: Optional[torch.Tensor]
    counters: torch.Tensor


def sample_rows(x, params: RowParams, kept_cap: int = 0, ws=None, result: Optional[SampleResult] = None,
                want_stats: bool = True) -> SampleResult:
    """One token per row: penalties -> candidates -> top-k / top-p / min-p -> draw (whirl_sample_rows)."""
    x, rows, n = _rows(x)
    dev = x.device
    if result is None:
        result = SampleResult(
            token=torch.empty(rows, dtype=torch.int32, device=dev), status=torch.empty(rows, dtype=torch.int32, device=dev),
            n_kept=torch.empty(rows, dtype=torch.int32, device=dev), closed=torch.empty(rows, dtype=torch.int32, device=dev),
            stats=torch.empty((rows, 2), dtype=torch.float32, device=dev) if want_stats else None,
            kept_ids=torch.full((rows, kept_cap), -1, dtype=torch.int32, device=dev) if kept_cap else None,
            kept_p=torch.zeros((rows, kept_cap), dtype=torch.float64, device=dev) if kept_cap else None,
            counters=torch.zeros(CNT_WORDS, dtype=torch.int32, device=dev))
    o = SampleOut(token=_p(result.token), status=_p(result.status), n_kept=_p(result.n_kept), closed=_p(result.closed),
                  stats=_p(result.stats), kept_ids=_p(result.kept_ids), kept_p=_p(result.kept_p),
                  kept_cap=0 if result.kept_ids is None else result.kept_ids.shape[1], counters=_p(result.counters))
    ws = workspace(rows, n, dev) if ws is None else ws
    ps = params.struct(rows)
    _check(lib.whirl_sample_rows(x.data_ptr(), _dtype(x), rows, n, C.byref(ps), C.byref(o), ws.data_ptr(), ws.numel(), _stream(x)))
    return result


def check(ws: torch.Tensor, rows: int) -> int:
    """whirl_check: reads the device error word of the last sample_rows / topk_rows call on `ws` (synchronises the
    stream).  Returns the code of the wait that ran out (0: none)."""
    where = C.c_uint32(0)
    st = lib.whirl_check(ws.data_ptr(), ws.numel(), rows, torch.cuda.current_stream(ws.device).cuda_stream, C.byref(where))
    if st not in (0, ERR_TIMEOUT):
        _check(st)
    return int(where.value)


def test_waits(wait_us: int = 0, lose_copy: bool = False) -> None:
    """whirl_test_waits: a testing aid; see include/whirl_b200.h."""
    lib.whirl_test_waits(wait_us, int(lose_copy))


GEN_SPLITMIX, GEN_PHILOX = 0, 1


def uniform_splitmix(seed: int, pos_idx: int, stream_id: int = 0) -> float:
    """Sampler::uniform / spec::uniform of the reference, on the host."""
    return lib.whirl_uniform_splitmix(seed, pos_idx, stream_id)


def race_base(seed: int, pos_idx: int) -> int:
    return lib.whirl_race_base(seed, pos_idx)


def philox4x32_10(ctr, key):
    c, k, o = (C.c_uint32 * 4)(*ctr), (C.c_uint32 * 2)(*key), (C.c_uint32 * 4)()
    lib.whirl_philox4x32_10(c, k, o)
    return list(o)


def uniform_philox4x32(seed: int, pos_idx: int, row: int, stream_id: int = 0) -> float:
    return lib.whirl_uniform_philox4x32(seed, pos_idx, row, stream_id)


def fill_draws(seed: torch.Tensor, pos_idx: torch.Tensor, generator: int = GEN_SPLITMIX, stream_id: int = 0, want_u: bool = True,
               want_race_key: bool = True):
    """seed, pos_idx: int64 CUDA tensors holding the u64 bit patterns -> (u f64, race_key int64 bit patterns)."""
    rows = seed.numel()
    u = torch.empty(rows, dtype=torch.float64, device=seed.device) if want_u else None
    rk = torch.empty(rows, dtype=torch.int64, device=seed.device) if want_race_key else None
    _check(lib.whirl_fill_draws(seed.data_ptr(), pos_idx.data_ptr(), rows, generator, stream_id, _p(u), _p(rk),
                                torch.cuda.current_stream(seed.device).cuda_stream))
    return u, rk


def launch_counts() -> dict:
    """Kernel launches made through the library by this process so far, per family."""
    a = (C.c_uint64 * 4)()
    lib.whirl_launch_counts(a, 4)
    return dict(rowscan=a[0], select_generic=a[1], single_pass=a[2], aux=a[3])


def sample_rows_host(x_host, params: dict, rows: int, n: int, dtype: int, out: dict, kept_cap: int = 0, device: int = 0):
    """whirl_sample_rows_host on host buffers: `x_host`, the values of `params` and of `out` are CPU tensors (pinned for
    full copy speed) or None.  Blocks until the tokens are in out['token']."""
    ps = SampleParams()
    for k, _ in SampleParams._fields_:
        if k == "hist_stride":
            continue
        t = params.get(k)
        setattr(ps, k, None if t is None else t.data_ptr())
    ps.hist_stride = 0 if params.get("hist") is None else params["hist"].shape[1]
    o = SampleOut(kept_cap=kept_cap)
    for k, _ in SampleOut._fields_:
        if k == "kept_cap":
            continue
        t = out.get(k)
        setattr(o, k, None if t is None else t.data_ptr())
    st = lib.whirl_sample_rows_host(x_host.data_ptr(), dtype, rows, n, C.byref(ps), C.byref(o), device)
    if st != 0:
        raise WhirlError(st, (lib.whirl_host_last_error() or b"").decode())


def merge_sample_rows(ids, vals, stats, n_total: int, params: RowParams, kept_cap: int = 0) -> SampleResult:
    """ids / vals [shards, rows, K_s], stats [shards, rows, 2] (all-gathered slices) -> one token per row."""
    shards, rows, ks = ids.shape
    dev = ids.device
    res = SampleResult(
        token=torch.empty(rows, dtype=torch.int32, device=dev), status=torch.empty(rows, dtype=torch.int32, device=dev),
        n_kept=torch.empty(rows, dtype=torch.int32, device=dev), closed=torch.empty(rows, dtype=torch.int32, device=dev),
        stats=torch.empty((rows, 2), dtype=torch.float32, device=dev),
        kept_ids=torch.full((rows, kept_cap), -1, dtype=torch.int32, device=dev) if kept_cap else None,
        kept_p=torch.zeros((rows, kept_cap), dtype=torch.float64, device=dev) if kept_cap else None,
        counters=torch.zeros(CNT_WORDS, dtype=torch.int32, device=dev))
    o = SampleOut(token=_p(res.token), status=_p(res.status), n_kept=_p(res.n_kept), closed=_p(res.closed), stats=_p(res.stats),
                  kept_ids=_p(res.kept_ids), kept_p=_p(res.kept_p), kept_cap=kept_cap, counters=_p(res.counters))
    ps = params.struct(rows)
    assert ids.is_contiguous() and vals.is_contiguous() and stats.is_contiguous()
    _check(lib.whirl_merge_sample_rows(ids.data_ptr(), vals.data_ptr(), stats.data_ptr(), shards, rows, ks, n_total, C.byref(ps),
                                       C.byref(o), torch.cuda.current_stream(dev).cuda_stream))
    return res


def merge_sample_rows_packed(blocks: torch.Tensor, shards: int, rows: int, ks: int, n_total: int, params: RowParams,
                             kept_cap: int = 0) -> SampleResult:
    """blocks: int32 tensor of `shards` packed blocks (the all-gather of every rank's block) -> one token per row."""
    dev = blocks.device
    assert blocks.is_contiguous() and blocks.numel() == shards * lib.whirl_shard_block_words(rows, ks)
    res = SampleResult(
        token=torch.empty(rows, dtype=torch.int32, device=dev), status=torch.empty(rows, dtype=torch.int32, device=dev),
        n_kept=torch.empty(rows, dtype=torch.int32, device=dev), closed=torch.empty(rows, dtype=torch.int32, device=dev),
        stats=torch.empty((rows, 2), dtype=torch.float32, device=dev),
        kept_ids=torch.full((rows, kept_cap), -1, dtype=torch.int32, device=dev) if kept_cap else None,
        kept_p=torch.zeros((rows, kept_cap), dtype=torch.float64, device=dev) if kept_cap else None,
        counters=torch.zeros(CNT_WORDS, dtype=torch.int32, device=dev))
    o = SampleOut(token=_p(res.token), status=_p(res.status), n_kept=_p(res.n_kept), closed=_p(res.closed), stats=_p(res.stats),
                  kept_ids=_p(res.kept_ids), kept_p=_p(res.kept_p), kept_cap=kept_cap, counters=_p(res.counters))
    ps = params.struct(rows)
    _check(lib.whirl_merge_sample_rows_packed(blocks.data_ptr(), shards, rows, ks, n_total, C.byref(ps), C.byref(o),
                                              torch.cuda.current_stream(dev).cuda_stream))
    return res


def accept_tokens(tokens, drafts, nd, row0):
    """Device accept loop: tokens [rows] i32, drafts [seqs, D] i32, nd / row0 [seqs] i32 -> (acc, chosen) [seqs] i32."""
    seqs = drafts.shape[0]
    acc = torch.empty(seqs, dtype=torch.int32, device=tokens.device)
    chosen = torch.empty(seqs, dtype=torch.int32, device=tokens.device)
    _check(lib.whirl_accept_tokens(tokens.data_ptr(), drafts.data_ptr(), drafts.shape[1], nd.data_ptr(), row0.data_ptr(), seqs,
                                   acc.data_ptr(), chosen.data_ptr(), torch.cuda.current_stream(tokens.device).cuda_stream))
    return acc, chosen


def accept_rows(tokens, drafts, nd, row0, relax: RelaxParams, greedy=None, relax_on=None, next_tok=None, hist=None, hist_len=None,
                rk_ids=None, rk_vals=None, rk_stats=None, kept: Optional[SampleResult] = None, x=None, inv_t=None):
    """whirl_accept_rows: the accept step with the relaxed rules.  tokens [rows] i32; drafts [seqs, D] i32; nd / row0 / next_tok
    [seqs] i32; greedy / relax_on [seqs] u8; hist [seqs, H] i32 + hist_len [seqs] i32; rk_* the outputs of topk_rows with
    K = rk; kept: a SampleResult with kept_ids / kept_p (the typical rule); x / inv_t the verify logits for open rows.
    Returns (acc, chosen, relaxed, relax_gap, flags)."""
    seqs = drafts.shape[0]
    dev = tokens.device
    a = AcceptIn(tokens=_p(tokens), drafts=_p(drafts), draft_stride=drafts.shape[1], nd=_p(nd), row0=_p(row0), greedy=_p(greedy),
                 relax_on=_p(relax_on), next=_p(next_tok), hist=_p(hist), hist_stride=0 if hist is None else hist.shape[1],
                 hist_len=_p(hist_len), rk_ids=_p(rk_ids), rk_vals=_p(rk_vals), rk_stats=_p(rk_stats),
                 rk=0 if rk_ids is None else rk_ids.shape[1])
    if kept is not None:
        a.kept_cap = 0 if kept.kept_ids is None else kept.kept_ids.shape[1]
        a.kept_ids, a.kept_p, a.n_kept, a.closed, a.stats = _p(kept.kept_ids), _p(kept.kept_p), _p(kept.n_kept), _p(kept.closed), _p(kept.stats)
    if x is not None:
        x, _, n = _rows(x)
        a.x, a.dtype, a.n = x.data_ptr(), _dtype(x), n
    a.inv_t = _p(inv_t)
    acc = torch.empty(seqs, dtype=torch.int32, device=dev)
    chosen = torch.empty(seqs, dtype=torch.int32, device=dev)
    relaxed = torch.zeros(seqs, dtype=torch.int32, device=dev)
    gap = torch.zeros(seqs, dtype=torch.float64, device=dev)
    flags = torch.zeros(seqs, dtype=torch.int32, device=dev)
    _check(lib.whirl_accept_rows(C.byref(a), C.byref(relax), seqs, acc.data_ptr(), chosen.data_ptr(), relaxed.data_ptr(), gap.data_ptr(),
                                 flags.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
    return acc, chosen, relaxed, gap, flags


def spec_accept_residual(target, draft, draft_tok, inv_t, u_acc, u_res):
    """target [seqs, L + 1, n], draft [seqs, L, n] logits; draft_tok [seqs, L] i32; inv_t [seqs] f32 or None;
    u_acc [seqs, L], u_res [seqs, L + 1] f64 -> (n_acc, next_tok) [seqs] i32."""
    seqs, L1, n = target.shape
    L = L1 - 1
    dev = target.device
    n_acc = torch.empty(seqs, dtype=torch.int32, device=dev)
    nxt = torch.empty(seqs, dtype=torch.int32, device=dev)
    ws = torch.empty(lib.whirl_spec_workspace_bytes(seqs, L), dtype=torch.uint8, device=dev)
    _check(lib.whirl_spec_accept_residual(target.data_ptr(), _p(draft), _dtype(target), seqs, L, n, _p(draft_tok), _p(inv_t), _p(u_acc),
                                          u_res.data_ptr(), n_acc.data_ptr(), nxt.data_ptr(), ws.data_ptr(), ws.numel(),
                                          torch.cuda.current_stream(dev).cuda_stream))
    return n_acc, nxt
