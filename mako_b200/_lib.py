"""ctypes binding of libmako_b200.so (the C ABI declared in include/mako_b200.h).

The library is the product; there is no Python or CPU implementation behind these names. If the shared object is
missing the import fails with the build command to run, and every call fails when no CUDA device is present.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MAKO_B200_LIB") or os.path.join(HERE, "libmako_b200.so")

MK_OK = 0
MK_ERR_INVALID_ARGUMENT = 1
MK_ERR_CUDA = 2
MK_ERR_UNSUPPORTED = 3
MK_ERR_NO_DEVICE = 4

FLAG_NEAR_CDF_BOUNDARY = 0x001
FLAG_GUARD_BAND = 0x002
FLAG_NO_CANDIDATE = 0x004
FLAG_ALL_MASKED = 0x008
FLAG_OVERFLOW = 0x010
FLAG_VP_TRUNCATED = 0x020
FLAG_TIMEOUT = 0x040
FLAG_HISTORY_FULL = 0x100

OVERLAP_OFF, OVERLAP_LAUNCH, OVERLAP_STABLE_SIDE_INPUTS = 0, 1, 2


class SamplingParamsC(C.Structure):
    _fields_ = [
        ("temperature", C.c_float),
        ("top_k", C.c_uint32),
        ("top_p", C.c_float),
        ("min_p", C.c_float),
        ("presence_penalty", C.c_float),
        ("frequency_penalty", C.c_float),
        ("repetition_penalty", C.c_float),
    ]


class RowsC(C.Structure):
    _fields_ = [
        ("logits", C.c_void_p),
        ("ld", C.c_uint64),
        ("batch", C.c_uint32),
        ("n_vocab", C.c_uint32),
        ("id_offset", C.c_int32),
        ("n_history", C.c_uint32),
        ("history", C.c_void_p),
        ("history_ld", C.c_uint64),
        ("history_len", C.c_void_p),
        ("mask", C.c_void_p),
        ("mask_ld", C.c_uint64),
        ("bias", C.c_void_p),
        ("n_bias", C.c_uint32),
        ("params_dev", C.c_void_p),
        ("params", SamplingParamsC),
    ]


class SampleOutC(C.Structure):
    _fields_ = [
        ("token", C.c_void_p),
        ("prob", C.c_void_p),
        ("flags", C.c_void_p),
        ("n_cand", C.c_void_p),
        ("cand_ids", C.c_void_p),
        ("cand_q", C.c_void_p),
        ("cand_cap", C.c_uint32),
    ]


class MakoError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"mako_b200 error {code}: {message}")
        self.code = code


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m mako_b200.build` "
            "(nvcc, sm_100a). There is no fallback implementation."
        )
    try:  # libcudart comes with torch's CUDA wheels; loading torch first makes it resolvable
        import torch  # noqa: F401
    except Exception:
        pass
    lib = C.CDLL(LIB_PATH)
    vp = C.c_void_p
    lib.mk_version.restype = C.c_char_p
    lib.mk_last_error.restype = C.c_char_p
    lib.mk_row_bytes.restype = C.c_uint64
    lib.mk_row_bytes.argtypes = [C.c_uint32, C.c_uint32, C.c_int, C.c_uint32, C.c_uint32]
    lib.mk_check_sampling.argtypes = [C.POINTER(SamplingParamsC)]
    lib.mk_sampler_create.argtypes = [C.POINTER(vp), C.c_int, C.c_uint32, C.c_uint32]
    lib.mk_sampler_destroy.argtypes = [vp]
    lib.mk_sampler_destroy.restype = None
    lib.mk_sampler_sample_batch.argtypes = [vp, C.POINTER(RowsC), vp, C.POINTER(SampleOutC), vp]
    lib.mk_sample_rows_static.argtypes = [C.c_int, C.POINTER(RowsC), vp, C.POINTER(SampleOutC), vp]
    lib.mk_sampler_verify_batch.argtypes = [vp, C.POINTER(RowsC), vp, vp, vp, C.POINTER(SampleOutC), vp, vp]
    lib.mk_sampler_verify_pq_batch.argtypes = [vp, C.POINTER(RowsC), vp, C.c_uint64, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.mk_spec_resolve.argtypes = [vp, C.c_uint32, C.c_uint32, vp, vp, vp, vp, vp]
    lib.mk_sampler_spec_round.argtypes = [vp, C.POINTER(RowsC), C.c_uint32, vp, vp, vp, C.POINTER(SampleOutC), vp, vp,
                                          vp, vp]
    lib.mk_spec_commit.argtypes = [vp, C.c_uint32, C.c_uint32, vp, vp, vp, vp, C.c_uint64, C.c_uint32, vp, vp, vp, vp]
    lib.mk_draft_pick.argtypes = [vp, vp, C.c_uint64, vp, vp, vp, C.c_uint64, vp, vp, C.c_uint32, C.c_uint32, C.c_uint32,
                                  C.c_uint32, C.c_uint32, vp, vp, vp]
    lib.mk_draft_pick_plain.argtypes = [vp, vp, C.c_uint64, C.c_uint32, C.c_uint32, vp, C.c_uint64, vp, C.c_uint32,
                                        C.c_float, vp, vp, vp, vp]
    lib.mk_rank_force.argtypes = [vp, vp, C.c_uint64, C.c_uint32, C.c_uint32, vp, C.c_uint32, vp, vp, vp]
    lib.mk_decode_commit.argtypes = [vp, C.c_uint32, vp, vp, vp, C.c_uint64, C.c_uint32, vp, vp, vp, vp, vp]
    lib.mk_vp_record_bytes.restype = C.c_uint32
    lib.mk_vp_record_bytes.argtypes = [C.c_uint32]
    lib.mk_sampler_vp_local.argtypes = [vp, C.POINTER(RowsC), C.c_uint32, vp, vp]
    lib.mk_sampler_vp_merge.argtypes = [vp, vp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                        C.POINTER(SamplingParamsC), vp, C.POINTER(SampleOutC), vp]
    lib.mk_sampler_sample_host.argtypes = [vp, C.POINTER(RowsC), vp, C.POINTER(SampleOutC)]
    lib.mk_row_sampler_create.argtypes = [C.POINTER(vp), C.POINTER(SamplingParamsC), C.c_uint32, C.c_uint64, C.c_int]
    lib.mk_row_sampler_destroy.argtypes = [vp]
    lib.mk_row_sampler_destroy.restype = None
    lib.mk_row_sampler_greedy.argtypes = [vp]
    lib.mk_row_sampler_accept.argtypes = [vp, C.c_int32]
    lib.mk_row_sampler_sample.argtypes = [vp, vp, C.POINTER(C.c_int32)]
    lib.mk_row_sampler_verify.argtypes = [vp, vp, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]
    lib.mk_debug_expf.argtypes = [vp, vp, C.c_uint64, vp]
    lib.mk_debug_set_timing.argtypes = [vp, vp]
    lib.mk_sampler_set_overlap.argtypes = [vp, C.c_int]
    lib.mk_sampler_set_split.argtypes = [vp, C.c_int]
    lib.mk_debug_withhold_tile.argtypes = [vp, C.c_int, C.c_uint32]
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != MK_OK:
        raise MakoError(rc, lib.mk_last_error().decode())
