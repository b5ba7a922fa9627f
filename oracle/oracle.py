"""ctypes bindings of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

``Oracle()``     -> oracle/liboracle.so, the plain-C restatement (oracle/whirl_oracle.c), prefix ``orc_``.
``Reference()``  -> oracle/_ref/libwhirl_ref.so, the reference's own sampling sources behind oracle/ref_shim.cpp,
                    prefix ``ref_`` (present only where it was built from a reference checkout).

Both expose the same methods where the reference has the function, so a test can run one body against either.
Only tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this module; the shipped package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libwhirl_ref.so")
DEFAULT_REF = os.environ.get("WHIRL_REF", "/root/reference")


class Sampler(C.Structure):
    _fields_ = [("inv_t", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_double), ("min_p", C.c_double),
                ("seed", C.c_uint64), ("pos_idx", C.c_uint64), ("race", C.c_int32), ("n", C.c_uint32),
                ("closed", C.c_int32), ("m", C.c_float), ("sum", C.c_float), ("full_used", C.c_uint32),
                ("big_used", C.c_uint32), ("use_u", C.c_int32), ("u_given", C.c_double)]


class RowOut(C.Structure):
    _fields_ = [("token", C.c_uint32), ("n", C.c_uint32), ("closed", C.c_int32), ("m", C.c_float), ("sum", C.c_float),
                ("big_used", C.c_uint32), ("full_used", C.c_uint32)]


class Batch(C.Structure):
    _fields_ = [("inv_t", C.c_void_p), ("top_k", C.c_void_p), ("top_p", C.c_void_p), ("min_p", C.c_void_p),
                ("greedy", C.c_void_p), ("race", C.c_void_p), ("seed", C.c_void_p), ("pos_idx", C.c_void_p),
                ("u", C.c_void_p), ("hist", C.c_void_p), ("hist_len", C.c_void_p), ("hist_stride", C.c_uint64),
                ("rep", C.c_void_p), ("pres", C.c_void_p), ("freq", C.c_void_p), ("ks", C.c_uint32), ("kb", C.c_uint32)]


class QDist(C.Structure):
    _fields_ = [("n", C.c_uint32), ("id", C.c_uint32 * 32), ("p", C.c_float * 32)]


class Accepted(C.Structure):
    _fields_ = [("acc", C.c_uint32), ("chosen", C.c_uint32), ("relaxed", C.c_uint32), ("relax_gap", C.c_double),
                ("pos_idx", C.c_uint64), ("full_used", C.c_uint32), ("big_used", C.c_uint32)]


class Relax(C.Structure):
    _fields_ = [("on", C.c_int32), ("k", C.c_uint32), ("alpha", C.c_float), ("eps", C.c_float), ("delta", C.c_float)]


class CaseInfo(C.Structure):
    _fields_ = [("greedy", C.c_int32), ("relax", C.c_int32), ("race", C.c_int32), ("temp", C.c_double),
                ("top_k", C.c_uint32), ("top_p", C.c_double), ("min_p", C.c_double), ("seed", C.c_uint64),
                ("n_gen", C.c_uint32), ("nd", C.c_uint32), ("row0", C.c_uint32), ("V", C.c_uint32),
                ("n_rows", C.c_uint32), ("next", C.c_uint32), ("hist_n", C.c_uint32)]


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _arr(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def build_oracle(force: bool = False) -> str:
    """Compile oracle/liboracle.so (gcc) if missing or older than its source."""
    src = os.path.join(HERE, "whirl_oracle.c")
    if force or not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, "oracle"], stdout=subprocess.DEVNULL)
    return ORACLE_SO


def build_reference(ref_root: str = DEFAULT_REF) -> str | None:
    """Compile oracle/_ref from a reference checkout when one is present; returns the .so path or None."""
    if os.path.isdir(os.path.join(ref_root, "src", "sampling")):
        subprocess.check_call(["make", "-C", HERE, "ref", f"WHIRL_REF={ref_root}"], stdout=subprocess.DEVNULL)
    return REF_SO if os.path.exists(REF_SO) else None


class _Lib:
    prefix = ""

    def __init__(self, path):
        self.lib = C.CDLL(path)
        self.path = path
        f = self._f
        f("uniform", C.c_double, [C.c_uint64, C.c_uint64, C.c_uint32])
        f("race_base", C.c_uint64, [C.c_uint64, C.c_uint64])
        f("race_e", C.c_double, [C.c_uint64, C.c_uint32])
        f("filter_cands", C.c_int, [C.POINTER(Sampler), C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_int])
        f("sample_rows", None if self.prefix == "orc_" else C.c_int,
          [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(Batch), C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
           C.c_int])
        f("draft_dist", None, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_float, C.c_float, C.c_float, C.c_uint32, C.c_float,
                               C.c_float, C.POINTER(QDist)])
        f("spec_sample_race", C.c_uint32, [C.POINTER(QDist), C.c_uint64])
        f("relax_accept_greedy", C.c_int, [C.POINTER(Relax), C.c_void_p, C.c_void_p, C.c_uint32, C.c_float, C.c_uint32])
        f("relax_extends_repeat", C.c_int, [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t])
        f("relax_accept_typical", C.c_int, [C.POINTER(Relax), C.c_double, C.c_double])
        f("accept_greedy", None, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_int, C.POINTER(Relax), C.c_void_p,
                                  C.c_uint32, C.c_void_p, C.c_size_t, C.c_uint32, C.POINTER(Accepted)])

    def _f(self, name, restype, argtypes):
        fn = getattr(self.lib, self.prefix + name)
        fn.restype = restype
        fn.argtypes = argtypes
        setattr(self, "_" + name, fn)

    # ---- scalars
    def uniform(self, seed, pos, stream=0):
        return self._uniform(seed, pos, stream)

    def race_base(self, seed, pos):
        return self._race_base(seed, pos)

    def race_e(self, base, token):
        return self._race_e(base, token)

    # ---- candidate filter
    def filter_cands(self, ids, logits, *, inv_t=1.0, top_k=0, top_p=1.0, min_p=0.0, m=None, sum_=None, complete=False):
        ids = np.array(ids, dtype=np.uint32)
        lg = np.array(logits, dtype=np.float32)
        p = np.zeros(len(ids), dtype=np.float64)
        s = Sampler(inv_t=inv_t, top_k=top_k, top_p=top_p, min_p=min_p, m=0 if m is None else m,
                    sum=1 if sum_ is None else sum_)
        ok = self._filter_cands(C.byref(s), _ptr(ids), _ptr(lg), _ptr(p), len(ids), int(complete))
        return dict(ok=bool(ok), n=s.n, closed=bool(s.closed), m=s.m, sum=s.sum, ids=ids, logits=lg, p=p)

    # ---- batch of rows
    def _batch(self, rows, *, inv_t=None, top_k=None, top_p=None, min_p=None, greedy=None, race=None, seed=None,
               pos_idx=None, u=None, hist=None, hist_len=None, rep=None, pres=None, freq=None, ks=0, kb=0):
        keep = dict(inv_t=_arr(inv_t, np.float32), top_k=_arr(top_k, np.uint32), top_p=_arr(top_p, np.float64),
                    min_p=_arr(min_p, np.float64), greedy=_arr(greedy, np.uint8), race=_arr(race, np.uint8),
                    seed=_arr(seed, np.uint64), pos_idx=_arr(pos_idx, np.uint64), u=_arr(u, np.float64),
                    hist=_arr(hist, np.int32), hist_len=_arr(hist_len, np.uint32), rep=_arr(rep, np.float32),
                    pres=_arr(pres, np.float32), freq=_arr(freq, np.float32))
        for k, v in keep.items():
            if v is not None and k != "hist":
                assert v.shape == (rows,), (k, v.shape)
        b = Batch(ks=ks, kb=kb, hist_stride=0 if keep["hist"] is None else keep["hist"].shape[1])
        for k, v in keep.items():
            setattr(b, k, None if v is None else v.ctypes.data)
        return b, keep

    def sample_rows(self, x, *, kept_cap=0, threads=1, **params):
        """x: [rows, V] float32, or uint16 (bf16 bit patterns).  Returns dict of per-row arrays."""
        x = np.ascontiguousarray(x)
        rows, V = x.shape
        b, keep = self._batch(rows, **params)
        out = (RowOut * rows)()
        kept_ids = np.zeros((rows, kept_cap), dtype=np.uint32) if kept_cap else None
        kept_p = np.zeros((rows, kept_cap), dtype=np.float64) if kept_cap else None
        xf = _ptr(x) if x.dtype == np.float32 else None
        xb = _ptr(x) if x.dtype == np.uint16 else None
        assert xf or xb, x.dtype
        rc = self._sample_rows(xf, xb, rows, V, C.byref(b), out, _ptr(kept_ids), _ptr(kept_p), kept_cap, threads)
        if rc not in (None, 0):
            raise RuntimeError(f"{self.prefix}sample_rows refused the batch (rc={rc})")
        o = np.frombuffer(out, dtype=np.dtype([("token", "u4"), ("n", "u4"), ("closed", "i4"), ("m", "f4"), ("sum", "f4"),
                                               ("big_used", "u4"), ("full_used", "u4")]))
        res = {k: o[k].copy() for k in o.dtype.names}
        res["kept_ids"], res["kept_p"] = kept_ids, kept_p
        del keep
        return res

    # ---- speculative pieces
    def draft_dist(self, ids, logits, m, sum_, inv_t, top_k, top_p, min_p):
        ids = np.array(ids, dtype=np.uint32)
        lg = np.array(logits, dtype=np.float32)
        q = QDist()
        self._draft_dist(_ptr(ids), _ptr(lg), len(ids), m, sum_, inv_t, top_k, top_p, min_p, C.byref(q))
        return q

    def spec_sample_race(self, q, base):
        return self._spec_sample_race(C.byref(q), base)

    def relax_accept_greedy(self, rp, ids, logits, m, draft):
        ids = np.array(ids, dtype=np.int32)
        lg = np.array(logits, dtype=np.float32)
        return bool(self._relax_accept_greedy(C.byref(rp), _ptr(ids), _ptr(lg), len(ids), m, draft))

    def relax_extends_repeat(self, hist, tail, ng=6, window=4096):
        h = np.array(hist, dtype=np.uint32)
        t = np.array(tail, dtype=np.uint32)
        return bool(self._relax_extends_repeat(_ptr(h), len(h), _ptr(t), len(t), ng, window))

    def relax_accept_typical(self, rp, pd, h):
        return bool(self._relax_accept_typical(C.byref(rp), pd, h))

    def accept_greedy(self, argmax, dr, nd, row0, relax, rp, relax_host, max_rows, hist, nxt):
        am = np.array(argmax, dtype=np.int32)
        d = np.array(dr, dtype=np.uint32)
        rh = np.ascontiguousarray(relax_host, dtype=np.uint8)
        h = np.array(hist, dtype=np.uint32)
        a = Accepted()
        self._accept_greedy(_ptr(am), _ptr(d), nd, row0, int(relax), C.byref(rp), _ptr(rh), max_rows, _ptr(h), len(h), nxt,
                            C.byref(a))
        return a


class Oracle(_Lib):
    prefix = "orc_"

    def __init__(self):
        super().__init__(build_oracle())
        f = self._f
        f("philox4x32_10", None, [C.c_void_p, C.c_void_p, C.c_void_p])
        f("philox_uniform", C.c_double, [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32])
        f("apply_penalties", C.c_int, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_float, C.c_float, C.c_float])
        f("first_max", C.c_int32, [C.c_void_p, C.c_uint32])
        f("softmax_top", C.c_double, [C.c_void_p, C.c_uint32])
        f("draft_pick", None, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_float,
                               C.c_void_p])
        f("topk_rows", None, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p])
        f("draft_sample_row", C.c_uint32, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_float, C.c_float, C.c_float,
                                          C.c_uint64, C.c_void_p])
        f("accept_sample", None, [C.c_void_p, C.c_uint32, C.POINTER(Sampler), C.c_void_p, C.c_uint32, C.c_uint32, C.c_int,
                                  C.c_uint32, C.POINTER(Relax), C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32, C.c_uint32,
                                  C.POINTER(Accepted)])
        f("spec_accept_residual", None, [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p, C.c_float, C.c_void_p,
                                         C.c_void_p, C.c_void_p, C.c_void_p])
        f("merge_shards", None, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float,
                                 C.c_void_p, C.c_void_p, C.c_void_p])
        f("bf16_to_f32", None, [C.c_void_p, C.c_void_p, C.c_size_t])

    def philox4x32_10(self, ctr, key):
        c = np.array(ctr, dtype=np.uint32)
        k = np.array(key, dtype=np.uint32)
        o = np.zeros(4, dtype=np.uint32)
        self._philox4x32_10(_ptr(c), _ptr(k), _ptr(o))
        return o

    def philox_uniform(self, seed, pos, row, stream=0):
        return self._philox_uniform(seed, pos, row, stream)

    def apply_penalties(self, x, hist, rep, pres, freq):
        x = np.array(x, dtype=np.float32)
        h = np.ascontiguousarray(hist, dtype=np.int32)
        skipped = self._apply_penalties(_ptr(x), len(x), _ptr(h), len(h), rep, pres, freq)
        return x, skipped

    def first_max(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return self._first_max(_ptr(x), len(x))

    def softmax_top(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return self._softmax_top(_ptr(x), len(x))

    def draft_pick(self, x, tok, prob, ctl, r, n_min, p_min, vmap=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        mp = _arr(vmap, np.int32)
        self._draft_pick(_ptr(x), len(x), _ptr(tok), _ptr(prob), _ptr(ctl), r, n_min, p_min, _ptr(mp))

    def topk_rows(self, x, k, inv_t):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, n = x.shape
        ids = np.full((rows, k), -1, dtype=np.int32)
        vals = np.zeros((rows, k), dtype=np.float32)
        stats = np.zeros((rows, 2), dtype=np.float32)
        self._topk_rows(_ptr(x), rows, n, k, inv_t, _ptr(ids), _ptr(vals), _ptr(stats))
        return ids, vals, stats

    def draft_sample_row(self, x, top_k, inv_t, top_p, min_p, race_key, vmap=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        mp = _arr(vmap, np.int32)
        words = np.zeros(72, dtype=np.int32)
        tok = self._draft_sample_row(_ptr(x), len(x), _ptr(mp), top_k, inv_t, top_p, min_p, race_key, _ptr(words))
        return tok, words

    def accept_sample(self, rows, sm, dr, nd, row0, typ, n_gen, rp, hist, nxt, ks=4, kb=16):
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        d = np.array(dr, dtype=np.uint32)
        h = np.array(hist, dtype=np.uint32)
        a = Accepted()
        self._accept_sample(_ptr(rows), rows.shape[1], C.byref(sm), _ptr(d), nd, row0, int(typ), n_gen, C.byref(rp), _ptr(h),
                            len(h), nxt, ks, kb, C.byref(a))
        return a

    def spec_accept_residual(self, target, draft, draft_tok, inv_t, u_acc, u_res):
        t = np.ascontiguousarray(target, dtype=np.float32)
        d = np.ascontiguousarray(draft, dtype=np.float32)
        L, V = d.shape
        assert t.shape == (L + 1, V)
        tok = np.ascontiguousarray(draft_tok, dtype=np.int32)
        ua = np.ascontiguousarray(u_acc, dtype=np.float64)
        ur = np.ascontiguousarray(u_res, dtype=np.float64)
        na = C.c_uint32()
        nt = C.c_uint32()
        self._spec_accept_residual(_ptr(t), _ptr(d), V, L, _ptr(tok), inv_t, _ptr(ua), _ptr(ur), C.byref(na), C.byref(nt))
        return na.value, nt.value

    def merge_shards(self, ids, vals, stats, k, inv_t):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        vals = np.ascontiguousarray(vals, dtype=np.float32)
        stats = np.ascontiguousarray(stats, dtype=np.float32)
        shards, ks = ids.shape
        kk = min(k, shards * ks)
        oi = np.zeros(kk, dtype=np.int32)
        ov = np.zeros(kk, dtype=np.float32)
        os_ = np.zeros(2, dtype=np.float32)
        self._merge_shards(_ptr(ids), _ptr(vals), _ptr(stats), shards, ks, k, inv_t, _ptr(oi), _ptr(ov), _ptr(os_))
        return oi, ov, os_

    def bf16_to_f32(self, xb):
        xb = np.ascontiguousarray(xb, dtype=np.uint16)
        out = np.zeros(xb.shape, dtype=np.float32)
        self._bf16_to_f32(_ptr(xb), _ptr(out), xb.size)
        return out


class Reference(_Lib):
    prefix = "ref_"

    def __init__(self, path: str = REF_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        super().__init__(path)
        f = self._f
        f("sampler_uniform", C.c_double, [C.c_uint64, C.c_uint64])
        f("sample_rows_small", C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(Batch), C.c_void_p, C.c_void_p,
                                         C.c_void_p, C.c_uint32])
        f("sample_row_excluding", C.c_uint32, [C.c_void_p, C.c_uint32, C.POINTER(Sampler), C.c_uint32, C.c_double])
        f("prob_of", C.c_double, [C.c_void_p, C.c_uint32, C.POINTER(Sampler), C.c_uint32])
        f("draft_cands", C.c_uint32, [C.c_uint32])
        f("accept_sample", None, [C.c_void_p, C.c_uint32, C.POINTER(Sampler), C.c_void_p, C.c_uint32, C.c_uint32, C.c_int,
                                  C.c_uint32, C.POINTER(Relax), C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint32,
                                  C.POINTER(Accepted)])
        f("case_count", C.c_uint32, [])
        f("case_name", C.c_char_p, [C.c_uint32])
        f("case_inputs", None, [C.c_uint32, C.POINTER(CaseInfo), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32,
                                C.c_void_p])
        f("case_relax_bytes", C.c_uint32, [C.c_uint32])
        f("case_max_rows", C.c_uint32, [])
        f("bench_rows", C.c_int, [C.c_void_p, C.c_uint32, C.c_uint32, C.POINTER(Batch), C.c_int, C.c_int, C.POINTER(C.c_double),
                                  C.c_void_p])

    def bench_rows(self, x, *, threads=1, reps=1, **params):
        """The timed CPU arm: persistent workers over the reference's real SampleBuffers -> filterCands -> sampleRow (this
        repository's penalty rule applied to each row first).  Returns (seconds for rows * reps samplings, first-pass tokens)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, V = x.shape
        b, keep = self._batch(rows, **params)
        sec = C.c_double(0.0)
        tok = np.zeros(rows, dtype=np.uint32)
        rc = self._bench_rows(_ptr(x), rows, V, C.byref(b), threads, reps, C.byref(sec), _ptr(tok))
        if rc != 0:
            raise RuntimeError("ref_bench_rows refused the batch")
        del keep
        return sec.value, tok

    def sampler_uniform(self, seed, pos):
        return self._sampler_uniform(seed, pos)

    def sample_rows_small(self, x, *, kept_cap=0, **params):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, V = x.shape
        b, keep = self._batch(rows, **params)
        out = (RowOut * rows)()
        kept_ids = np.zeros((rows, kept_cap), dtype=np.uint32) if kept_cap else None
        kept_p = np.zeros((rows, kept_cap), dtype=np.float64) if kept_cap else None
        rc = self._sample_rows_small(_ptr(x), rows, V, C.byref(b), out, _ptr(kept_ids), _ptr(kept_p), kept_cap)
        if rc != 0:
            raise RuntimeError("ref_sample_rows_small refused the batch")
        o = np.frombuffer(out, dtype=np.dtype([("token", "u4"), ("n", "u4"), ("closed", "i4"), ("m", "f4"), ("sum", "f4"),
                                               ("big_used", "u4"), ("full_used", "u4")]))
        res = {k: o[k].copy() for k in o.dtype.names}
        res["kept_ids"], res["kept_p"] = kept_ids, kept_p
        del keep
        return res

    def sample_row_excluding(self, x, sm, ex, p_ex):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return self._sample_row_excluding(_ptr(x), len(x), C.byref(sm), ex, p_ex)

    def prob_of(self, x, sm, t):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return self._prob_of(_ptr(x), len(x), C.byref(sm), t)

    def accept_sample(self, rows, sm, dr, nd, row0, typ, n_gen, rp, hist, nxt):
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        d = np.array(dr, dtype=np.uint32)
        h = np.array(hist, dtype=np.uint32)
        a = Accepted()
        self._accept_sample(_ptr(rows), rows.shape[1], C.byref(sm), _ptr(d), nd, row0, int(typ), n_gen, C.byref(rp), _ptr(h),
                            len(h), nxt, rows.shape[0], C.byref(a))
        return a

    def cases(self):
        """The reference's fixed acceptance cases with their inputs, as plain Python / numpy."""
        out = []
        for i in range(self._case_count()):
            info = CaseInfo()
            rb = self._case_relax_bytes(i)
            rows = np.zeros((16, 96), dtype=np.float32)
            dr = np.zeros(15, dtype=np.uint32)
            am = np.zeros(16, dtype=np.int32)
            rh = np.zeros(rb, dtype=np.uint8)
            hist = np.zeros(16, dtype=np.uint32)
            # V is 64 for every fixed case; rows are returned packed [n_rows][V]
            self._case_inputs(i, C.byref(info), _ptr(rows), _ptr(dr), _ptr(am), _ptr(rh), rb, _ptr(hist))
            V = info.V
            flat = rows.reshape(-1)[: info.n_rows * V].reshape(info.n_rows, V).copy()
            out.append(dict(name=self._case_name(i).decode(), greedy=bool(info.greedy), relax=bool(info.relax),
                            race=bool(info.race), temp=info.temp, top_k=info.top_k, top_p=info.top_p, min_p=info.min_p,
                            seed=info.seed, n_gen=info.n_gen, nd=info.nd, row0=info.row0, V=V, rows=flat, dr=dr.copy(),
                            argmax=am.copy(), relax_host=rh.copy(), hist=hist[: info.hist_n].copy(), next=info.next,
                            max_rows=self._case_max_rows()))
        return out


def have_reference() -> bool:
    return os.path.exists(REF_SO)
