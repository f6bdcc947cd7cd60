"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(csrc/synth.cpp): logits N(0, 2^2) plus 8 spikes U(8, 15), Zipf(1.1) token histories, 2 % allowed-token masks,
64-entry sparse biases, PCG uniforms. numpy arrays out; nothing here touches the GPU."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(HERE, "libmk_synth.so")
if not os.path.exists(_PATH):
    raise ImportError(f"{_PATH} is missing: build it with `python -m mako_b200.build`")
_lib = C.CDLL(_PATH)
_vp = C.c_void_p
_lib.mk_synth_logits.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_float,
                                 C.c_uint32, C.c_float, C.c_float, _vp, _vp, C.c_uint32]
_lib.mk_synth_history_zipf.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                       C.c_double, _vp, C.c_uint32]
_lib.mk_synth_mask.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, C.c_double,
                               _vp, C.c_uint32, _vp, C.c_uint32]
_lib.mk_synth_bias.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float,
                               C.c_float, _vp, _vp, C.c_uint32]
_lib.mk_synth_uniforms.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, _vp]
_lib.mk_synth_add_noise.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64,
                                    C.c_float, _vp, C.c_uint32]

_THREADS = max(1, min(32, os.cpu_count() or 1))


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


def logits(seed: int, rows: int, n_vocab: int, *, step: int = 0, row0: int = 0, ld: int | None = None,
           sigma: float = 2.0, n_spikes: int = 8, spike_lo: float = 8.0, spike_hi: float = 15.0,
           out: np.ndarray | None = None):
    """Returns (logits [rows, ld] float32, spike_ids [rows, n_spikes] int32)."""
    ld = ld or n_vocab
    if out is None:
        out = np.zeros((rows, ld), dtype=np.float32)
    assert out.dtype == np.float32 and out.shape == (rows, ld) and out.flags.c_contiguous
    spikes = np.full((rows, max(n_spikes, 1)), -1, dtype=np.int32)
    _lib.mk_synth_logits(seed, step, row0, rows, n_vocab, ld, sigma, n_spikes, spike_lo, spike_hi, _p(out),
                         _p(spikes), _THREADS)
    return out, spikes[:, :n_spikes]


def history_zipf(seed: int, rows: int, n_vocab: int, n_history: int, *, s: float = 1.1, step: int = 0,
                 row0: int = 0) -> np.ndarray:
    out = np.zeros((rows, n_history), dtype=np.int32)
    _lib.mk_synth_history_zipf(seed, step, row0, rows, n_vocab, n_history, s, _p(out), _THREADS)
    return out


def mask(seed: int, rows: int, n_vocab: int, *, fraction: float = 0.02, spike_ids: np.ndarray | None = None,
         step: int = 0, row0: int = 0) -> np.ndarray:
    """Packed uint32 words [rows, mask_ld], mask_ld = ceil(V/32) rounded up to a multiple of 4."""
    ld = ((n_vocab + 31) // 32 + 3) // 4 * 4
    out = np.zeros((rows, ld), dtype=np.uint32)
    ns = 0 if spike_ids is None else spike_ids.shape[1]
    sp = None if spike_ids is None else np.ascontiguousarray(spike_ids, dtype=np.int32)
    _lib.mk_synth_mask(seed, step, row0, rows, n_vocab, ld, fraction, _p(sp) if sp is not None else None, ns,
                       _p(out), _THREADS)
    return out


def bias(seed: int, rows: int, n_vocab: int, n_bias: int, *, lo: float = -5.0, hi: float = 5.0, step: int = 0,
         row0: int = 0):
    """Returns (ids [rows, n_bias] int32, values [rows, n_bias] float32), ids distinct within a row."""
    ids = np.zeros((rows, n_bias), dtype=np.int32)
    vals = np.zeros((rows, n_bias), dtype=np.float32)
    _lib.mk_synth_bias(seed, step, row0, rows, n_vocab, n_bias, lo, hi, _p(ids), _p(vals), _THREADS)
    return ids, vals


def uniforms(seed: int, n: int, *, purpose: int = 0, step: int = 0, row0: int = 0) -> np.ndarray:
    out = np.zeros(n, dtype=np.float32)
    _lib.mk_synth_uniforms(seed, step, purpose, row0, n, _p(out))
    return out


def add_noise(seed: int, x: np.ndarray, n_vocab: int, *, sigma: float = 1.0, step: int = 0, row0: int = 0) -> np.ndarray:
    y = np.ascontiguousarray(x.copy(), dtype=np.float32)
    _lib.mk_synth_add_noise(seed, step, row0, y.shape[0], n_vocab, y.shape[1], sigma, _p(y), _THREADS)
    return y
