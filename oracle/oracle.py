"""TEST INFRASTRUCTURE — ctypes access to the two CPU checkers (see oracle_api.h).

    Oracle("port")       the CPU restatement, oracle/liboracle_port.so (built by `make -C oracle`)
    Oracle("reference")  the reference's own sampler.cpp compiled unmodified, oracle/_ref/liboracle_ref.so
    Oracle("best")       the reference build when present, else the port

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(HERE, "liboracle_port.so")
REF_PATH = os.path.join(HERE, "_ref", "liboracle_ref.so")


class ParamsC(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_uint32), ("top_p", C.c_float), ("min_p", C.c_float),
                ("presence_penalty", C.c_float), ("frequency_penalty", C.c_float), ("repetition_penalty", C.c_float)]


class RowC(C.Structure):
    _fields_ = [("n_vocab", C.c_uint32), ("logits", C.c_void_p), ("history", C.c_void_p), ("n_history", C.c_uint32),
                ("mask", C.c_void_p), ("bias_ids", C.c_void_p), ("bias_vals", C.c_void_p), ("n_bias", C.c_uint32)]


def build(force: bool = False) -> None:
    if force or not os.path.exists(PORT_PATH):
        subprocess.check_call(["make", "-C", HERE, "-s"])


def have_reference() -> bool:
    return os.path.exists(REF_PATH)


def _params(p) -> ParamsC:
    return ParamsC(p.temperature, p.top_k, p.top_p, p.min_p, p.presence_penalty, p.frequency_penalty,
                   p.repetition_penalty)


class Oracle:
    def __init__(self, kind: str = "best"):
        if kind == "best":
            kind = "reference" if have_reference() else "port"
        path = REF_PATH if kind == "reference" else PORT_PATH
        if kind == "port" and not os.path.exists(path):
            build()
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.lib.orc_kind.restype = C.c_char_p
        self.lib.orc_time_sample_batch.restype = C.c_double
        self.lib.orc_sample.argtypes = [C.POINTER(ParamsC), C.POINTER(RowC), C.c_float, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]
        self.lib.orc_verify.argtypes = [C.POINTER(ParamsC), C.POINTER(RowC), C.c_int32, C.c_float, C.c_float,
                                        C.c_void_p, C.c_void_p]
        self.lib.orc_verify_pq.argtypes = [C.POINTER(ParamsC), C.POINTER(RowC), C.POINTER(RowC), C.c_float, C.c_float,
                                           C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
        self.lib.orc_sample_rng.argtypes = [C.POINTER(ParamsC), C.POINTER(RowC), C.c_uint64, C.c_uint32, C.c_void_p]
        self.lib.orc_time_sample_batch.argtypes = [C.POINTER(ParamsC), C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint64,
                                                   C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64, C.c_void_p,
                                                   C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p]
        self.kind = self.lib.orc_kind().decode()
        assert self.kind == kind

    @staticmethod
    def _row(logits, history=None, mask=None, bias_ids=None, bias_vals=None):
        keep = []

        def arr(a, dt):
            a = np.ascontiguousarray(a, dtype=dt)
            keep.append(a)
            return a

        l = arr(logits, np.float32)
        r = RowC()
        r.n_vocab = l.size
        r.logits = l.ctypes.data
        if history is not None and len(history):
            h = arr(history, np.int32)
            r.history, r.n_history = h.ctypes.data, h.size
        if mask is not None:
            m = arr(mask, np.uint32)
            assert m.size * 32 >= l.size
            r.mask = m.ctypes.data
        if bias_ids is not None and len(bias_ids):
            bi, bv = arr(bias_ids, np.int32), arr(bias_vals, np.float32)
            r.bias_ids, r.bias_vals, r.n_bias = bi.ctypes.data, bv.ctypes.data, bi.size
        return r, keep

    def sample(self, params, logits, u, *, history=None, mask=None, bias_ids=None, bias_vals=None, cap=0):
        """Returns dict(token, prob, n_cand, near_boundary, cand_ids, cand_q)."""
        r, keep = self._row(logits, history, mask, bias_ids, bias_vals)
        p = _params(params)
        tok, prob, n, nb = C.c_int32(), C.c_float(), C.c_uint32(), C.c_uint32()
        ids = np.zeros(max(cap, 1), dtype=np.int32)
        qs = np.zeros(max(cap, 1), dtype=np.float32)
        rc = self.lib.orc_sample(C.byref(p), C.byref(r), float(u), C.addressof(tok), C.addressof(prob),
                                 C.addressof(n), ids.ctypes.data, qs.ctypes.data, cap, C.addressof(nb))
        if rc != 0:
            raise ValueError("oracle: bad argument")
        k = min(n.value, cap)
        return dict(token=tok.value, prob=prob.value, n_cand=n.value, near_boundary=nb.value, cand_ids=ids[:k].copy(),
                    cand_q=qs[:k].copy())

    def verify(self, params, logits, draft, u1, u2, *, history=None, mask=None, bias_ids=None, bias_vals=None):
        r, keep = self._row(logits, history, mask, bias_ids, bias_vals)
        p = _params(params)
        tok, acc = C.c_int32(), C.c_int32()
        rc = self.lib.orc_verify(C.byref(p), C.byref(r), int(draft), float(u1), float(u2), C.addressof(tok),
                                 C.addressof(acc))
        if rc != 0:
            raise ValueError("oracle: bad argument")
        return tok.value, bool(acc.value)

    def verify_pq(self, params, target_logits, draft_logits, u_draft, u_accept, u_resample, *, history=None,
                  mask=None, bias_ids=None, bias_vals=None):
        rt, k1 = self._row(target_logits, history, mask, bias_ids, bias_vals)
        rd, k2 = self._row(draft_logits, history, mask, bias_ids, bias_vals)
        p = _params(params)
        d, acc, tok = C.c_int32(), C.c_int32(), C.c_int32()
        rc = self.lib.orc_verify_pq(C.byref(p), C.byref(rt), C.byref(rd), float(u_draft), float(u_accept),
                                    float(u_resample), C.addressof(d), C.addressof(acc), C.addressof(tok))
        if rc != 0:
            raise ValueError("oracle: bad argument")
        return d.value, bool(acc.value), tok.value

    def sample_rng(self, params, logits, seed, n_draws, *, history=None):
        r, keep = self._row(logits, history)
        p = _params(params)
        out = np.zeros(n_draws, dtype=np.int32)
        rc = self.lib.orc_sample_rng(C.byref(p), C.byref(r), int(seed), n_draws, out.ctypes.data)
        if rc != 0:
            raise ValueError("oracle: bad argument")
        return out

    def uniforms(self, seed, n):
        out = np.zeros(n, dtype=np.float32)
        self.lib.orc_uniforms.argtypes = [C.c_uint64, C.c_uint32, C.c_void_p]
        self.lib.orc_uniforms(int(seed), n, out.ctypes.data)
        return out

    def time_sample_batch(self, params, logits, u, *, history=None, mask=None, bias_ids=None, bias_vals=None,
                          n_threads=1):
        """Returns (seconds, tokens). logits [B, ld] float32 C-contiguous rows."""
        assert logits.dtype == np.float32 and logits.ndim == 2 and logits.strides[1] == 4
        b, v = logits.shape
        p = _params(params)
        tokens = np.zeros(b, dtype=np.int32)
        u = np.ascontiguousarray(u, dtype=np.float32)
        h = np.ascontiguousarray(history, dtype=np.int32) if history is not None else None
        m = np.ascontiguousarray(mask, dtype=np.uint32) if mask is not None else None
        bi = np.ascontiguousarray(bias_ids, dtype=np.int32) if bias_ids is not None else None
        bv = np.ascontiguousarray(bias_vals, dtype=np.float32) if bias_vals is not None else None
        sec = self.lib.orc_time_sample_batch(
            C.byref(p), b, v, logits.ctypes.data, logits.strides[0] // 4,
            h.ctypes.data if h is not None else None, h.shape[1] if h is not None else 0,
            m.ctypes.data if m is not None else None, m.shape[1] if m is not None else 0,
            bi.ctypes.data if bi is not None else None, bv.ctypes.data if bv is not None else None,
            bi.shape[1] if bi is not None else 0, u.ctypes.data, n_threads, tokens.ctypes.data)
        if sec < 0:
            raise ValueError("oracle: bad argument")
        return sec, tokens
