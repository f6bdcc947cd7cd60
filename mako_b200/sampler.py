"""Host-side mirror of the reference sampler's interface over the C ABI.

`SamplingParams` and `Sampler` carry the names, argument meaning and error behaviour of mako::gen::SamplingParams and
mako::gen::Sampler (src/gen/sampler.hpp:12-45): one row, own state, own generator. `BatchSampler` is the batched
form the GPU is built for: torch CUDA tensors in, torch CUDA tensors out, one kernel launch per call. Torch is used
for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import RowsC, SampleOutC, check, lib
from .params import SamplingParams


def check_sampling(p: SamplingParams) -> None:
    """The range checks the reference applies upstream (src/server/openai.cpp:316-328); raises ValueError."""
    c = p.to_c()
    if lib.mk_check_sampling(C.byref(c)) != 0:
        raise ValueError(lib.mk_last_error().decode())


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class Sampler:
    """One row at a time, as the reference: Sampler(params, n_vocab, seed); sample(); verify(); accept()."""

    def __init__(self, params: SamplingParams, n_vocab: int, seed: int, device: int = 0):
        if n_vocab == 0:
            raise ValueError("sampler: empty vocabulary")  # std::invalid_argument in the reference
        self._h = C.c_void_p()
        c = params.to_c()
        check(lib.mk_row_sampler_create(C.byref(self._h), C.byref(c), n_vocab, seed, device))
        self.n_vocab = n_vocab
        self.params = params

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.mk_row_sampler_destroy(h)
            self._h = None

    def greedy(self) -> bool:
        return self.params.temperature <= 0.0

    def accept(self, token: int) -> None:
        check(lib.mk_row_sampler_accept(self._h, int(token)))

    @staticmethod
    def _row_ptr(logits, n_vocab: int):
        if isinstance(logits, torch.Tensor):
            assert logits.dtype == torch.float32 and logits.numel() >= n_vocab and logits.is_contiguous()
            return logits.data_ptr(), logits
        a = np.ascontiguousarray(logits, dtype=np.float32)
        assert a.size >= n_vocab
        return a.ctypes.data, a

    def sample(self, logits) -> int:
        p, keep = self._row_ptr(logits, self.n_vocab)
        tok = C.c_int32()
        check(lib.mk_row_sampler_sample(self._h, p, C.byref(tok)))
        del keep
        return tok.value

    def verify(self, logits, draft: int):
        """Returns (token, accepted) — the reference returns the token and sets `accepted` by reference."""
        p, keep = self._row_ptr(logits, self.n_vocab)
        tok, acc = C.c_int32(), C.c_int32()
        check(lib.mk_row_sampler_verify(self._h, p, int(draft), C.byref(acc), C.byref(tok)))
        del keep
        return tok.value, bool(acc.value)


@dataclass
class SampleResult:
    token: torch.Tensor
    prob: torch.Tensor
    flags: torch.Tensor
    n_cand: torch.Tensor
    cand_ids: Optional[torch.Tensor] = None
    cand_q: Optional[torch.Tensor] = None
    accepted: Optional[torch.Tensor] = None
    draft_token: Optional[torch.Tensor] = None


class BatchSampler:
    """Batched sampling on one GPU. All tensors live on `device`; outputs are allocated once and reused."""

    def __init__(self, n_vocab: int, max_batch: int, device: int = 0, cand_cap: int = 0):
        if n_vocab == 0:
            raise ValueError("sampler: empty vocabulary")
        self.device = torch.device("cuda", device)
        self._h = C.c_void_p()
        check(lib.mk_sampler_create(C.byref(self._h), device, n_vocab, max_batch))
        self.n_vocab, self.max_batch, self.cand_cap = n_vocab, max_batch, cand_cap
        d = self.device
        self.token = torch.empty(max_batch, dtype=torch.int32, device=d)
        self.prob = torch.empty(max_batch, dtype=torch.float32, device=d)
        self.flags = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.n_cand = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.accepted = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.draft_token = torch.zeros(max_batch, dtype=torch.int32, device=d)
        self.cand_ids = torch.zeros((max_batch, cand_cap), dtype=torch.int32, device=d) if cand_cap else None
        self.cand_q = torch.zeros((max_batch, cand_cap), dtype=torch.float32, device=d) if cand_cap else None

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.mk_sampler_destroy(h)
            self._h = None

    def set_overlap(self, mode: int) -> None:
        """How the row kernel is launched behind the previous kernel of the stream (mk_sampler_set_overlap):
        0 plain stream order, 1 programmatic dependent launch, 2 the same with the per-row history tables built
        before the wait (the caller promises that the previous kernel writes no parameters, histories or biases)."""
        check(lib.mk_sampler_set_overlap(self._h, int(mode)))

    def set_split(self, on: bool) -> None:
        """Whether a small batch (at most 8 rows, shared parameters, drawing under a top_k of at most 64) has every
        row split over many CTAs and merged (the default) or runs as one CTA per row (mk_sampler_set_split)."""
        check(lib.mk_sampler_set_split(self._h, 1 if on else 0))

    # -- argument marshalling -----------------------------------------------------------------------------------
    def _rows(self, logits: torch.Tensor, params, history=None, history_len=None, mask=None, bias=None,
              n_vocab=None, id_offset: int = 0) -> RowsC:
        assert logits.is_cuda and logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
        r = RowsC()
        r.logits = logits.data_ptr()
        r.ld = logits.stride(0)
        r.batch = logits.shape[0]
        r.n_vocab = n_vocab if n_vocab is not None else logits.shape[1]
        r.id_offset = id_offset
        if history is not None:
            assert history.is_cuda and history.dtype == torch.int32 and history.dim() == 2 and history.stride(1) == 1
            r.history = history.data_ptr()
            r.history_ld = history.stride(0)
            r.n_history = history.shape[1]
            if history_len is not None:
                assert history_len.dtype == torch.int32 and history_len.is_cuda
                r.history_len = history_len.data_ptr()
        if mask is not None:
            assert mask.is_cuda and mask.dtype in (torch.int32, torch.uint32) and mask.dim() == 2
            r.mask = mask.data_ptr()
            r.mask_ld = mask.stride(0)
        if bias is not None:
            # bias: [batch, n_bias, 2] int32 view of (id, float bits) pairs
            assert bias.is_cuda and bias.dtype == torch.int32 and bias.dim() == 3 and bias.shape[2] == 2
            assert bias.is_contiguous()
            r.bias = bias.data_ptr()
            r.n_bias = bias.shape[1]
        if isinstance(params, torch.Tensor):
            assert params.is_cuda and params.dtype == torch.int32 and params.shape == (logits.shape[0], 7)
            r.params_dev = params.data_ptr()
        else:
            r.params = params.to_c()
        return r

    def _out(self, batch: int) -> SampleOutC:
        o = SampleOutC()
        o.token = self.token.data_ptr()
        o.prob = self.prob.data_ptr()
        o.flags = self.flags.data_ptr()
        o.n_cand = self.n_cand.data_ptr()
        if self.cand_cap:
            o.cand_ids = self.cand_ids.data_ptr()
            o.cand_q = self.cand_q.data_ptr()
            o.cand_cap = self.cand_cap
        return o

    def _result(self, b: int, **kw) -> SampleResult:
        return SampleResult(self.token[:b], self.prob[:b], self.flags[:b], self.n_cand[:b],
                            self.cand_ids[:b] if self.cand_cap else None,
                            self.cand_q[:b] if self.cand_cap else None, **kw)

    # -- the operations -----------------------------------------------------------------------------------------
    def sample(self, logits, params, u=None, *, history=None, history_len=None, mask=None, bias=None) -> SampleResult:
        """Sampler::sample for every row (src/gen/sampler.cpp:75-84); u[b] is the row's uniform."""
        r = self._rows(logits, params, history, history_len, mask, bias)
        o = self._out(r.batch)
        check(lib.mk_sampler_sample_batch(self._h, C.byref(r), _ptr(u), C.byref(o), _stream_ptr(self.device)))
        return self._result(r.batch)

    def verify(self, logits, params, draft, u_accept, u_redraw, *, history=None, history_len=None, mask=None,
               bias=None) -> SampleResult:
        """Sampler::verify for every row (src/gen/sampler.cpp:86-107)."""
        r = self._rows(logits, params, history, history_len, mask, bias)
        o = self._out(r.batch)
        check(lib.mk_sampler_verify_batch(self._h, C.byref(r), _ptr(draft), _ptr(u_accept), _ptr(u_redraw),
                                          C.byref(o), self.accepted.data_ptr(), _stream_ptr(self.device)))
        return self._result(r.batch, accepted=self.accepted[: r.batch])

    def verify_pq(self, target_logits, draft_logits, params, u_draft, u_accept, u_resample, *, history=None,
                  history_len=None, mask=None, bias=None) -> SampleResult:
        """Rejection sampling of a drafter's token against max(0, p - q)."""
        r = self._rows(target_logits, params, history, history_len, mask, bias)
        assert draft_logits.is_cuda and draft_logits.dtype == torch.float32 and draft_logits.stride(1) == 1
        b = r.batch
        check(lib.mk_sampler_verify_pq_batch(self._h, C.byref(r), draft_logits.data_ptr(), draft_logits.stride(0),
                                             _ptr(u_draft), _ptr(u_accept), _ptr(u_resample),
                                             self.draft_token.data_ptr(), self.accepted.data_ptr(),
                                             self.token.data_ptr(), self.flags.data_ptr(),
                                             _stream_ptr(self.device)))
        return SampleResult(self.token[:b], self.prob[:b], self.flags[:b], self.n_cand[:b],
                            accepted=self.accepted[:b], draft_token=self.draft_token[:b])

    def draft_pick(self, logits, head, embed, x, w, prev):
        """One step of the drafter pick (src/kernels/dsv41.metal:664-742) for up to 8 sequences: logits [S, V],
        head [V, rank], embed [E, rank], x [S, dim], w [dim + rank], prev [S] int32. Returns (draft [S] int32,
        conf [S] float32)."""
        for t in (logits, head, embed, x, w):
            assert t.is_cuda and t.dtype == torch.float32 and t.stride(-1) == 1
        assert head.is_contiguous() and embed.is_contiguous() and w.is_contiguous()
        n_seq, v = logits.shape
        rank, dim = head.shape[1], x.shape[1]
        assert head.shape[0] == v and embed.shape[1] == rank and w.numel() == dim + rank
        draft = torch.empty(n_seq, dtype=torch.int32, device=self.device)
        conf = torch.empty(n_seq, dtype=torch.float32, device=self.device)
        check(lib.mk_draft_pick(self._h, logits.data_ptr(), logits.stride(0), head.data_ptr(), embed.data_ptr(),
                                x.data_ptr(), x.stride(0), w.data_ptr(), prev.data_ptr(), n_seq, v, rank, dim,
                                embed.shape[0], draft.data_ptr(), conf.data_ptr(), _stream_ptr(self.device)))
        return draft, conf

    def draft_pick_plain(self, logits, h, conf_w, conf_bias: float, next_prev=None):
        """hy4_draft_pick (src/kernels/hy4f.metal:352-397): (argmax of each row with the lowest index on ties,
        sigmoid(conf_w . h[b] + conf_bias)). logits [S, V], h [S, width], conf_w [width]."""
        for t in (logits, h, conf_w):
            assert t.is_cuda and t.dtype == torch.float32 and t.stride(-1) == 1
        n_seq, v = logits.shape
        draft = torch.empty(n_seq, dtype=torch.int32, device=self.device)
        conf = torch.empty(n_seq, dtype=torch.float32, device=self.device)
        check(lib.mk_draft_pick_plain(self._h, logits.data_ptr(), logits.stride(0), n_seq, v, h.data_ptr(), h.stride(0),
                                      conf_w.data_ptr(), conf_w.numel(), float(conf_bias), draft.data_ptr(),
                                      conf.data_ptr(), _ptr(next_prev), _stream_ptr(self.device)))
        return draft, conf

    def rank_force(self, logits: torch.Tensor, token: torch.Tensor, k: int = 3):
        """ReasoningBudget::forced's logit test (src/server/openai.cpp:596-603) for every row: returns (forced [B]
        int32: token[b] if fewer than k raw logits are greater than its own, else -1; above [B]: that count)."""
        assert logits.is_cuda and logits.dtype == torch.float32 and logits.stride(1) == 1
        b, v = logits.shape
        forced = torch.empty(b, dtype=torch.int32, device=self.device)
        above = torch.empty(b, dtype=torch.int32, device=self.device)
        check(lib.mk_rank_force(self._h, logits.data_ptr(), logits.stride(0), b, v, token.data_ptr(), k,
                                forced.data_ptr(), above.data_ptr(), _stream_ptr(self.device)))
        return forced, above

    def decode_commit(self, sampled: torch.Tensor, history: torch.Tensor, history_len: torch.Tensor, *, forced=None,
                      next_input=None, flags=None) -> torch.Tensor:
        """One decode step's bookkeeping on the device (src/gen/session.cpp:416-444): forced tokens replace sampled
        ones, the token is appended to each row's history (history [B, cap] int32, history_len [B] int32, both
        updated in place) and written to next_input. Returns the committed tokens [B]."""
        b = sampled.shape[0]
        assert history.dtype == torch.int32 and history_len.dtype == torch.int32 and history.stride(1) == 1
        committed = torch.empty(b, dtype=torch.int32, device=self.device)
        check(lib.mk_decode_commit(self._h, b, sampled.data_ptr(), _ptr(forced), history.data_ptr(), history.stride(0),
                                   history.shape[1], history_len.data_ptr(), _ptr(next_input), committed.data_ptr(),
                                   _ptr(flags), _stream_ptr(self.device)))
        return committed

    def spec_resolve(self, accepted: torch.Tensor, token: torch.Tensor):
        """accepted/token: [n_seq, n_pos] int32. Returns (n_kept [n_seq], next_token [n_seq])."""
        n_seq, n_pos = accepted.shape
        kept = torch.empty(n_seq, dtype=torch.int32, device=self.device)
        nxt = torch.empty(n_seq, dtype=torch.int32, device=self.device)
        check(lib.mk_spec_resolve(self._h, n_seq, n_pos, accepted.data_ptr(), token.data_ptr(), kept.data_ptr(),
                                  nxt.data_ptr(), _stream_ptr(self.device)))
        return kept, nxt

    def spec_round(self, logits, params, drafts, u, *, history=None, history_len=None, forced=None, mask=None,
                   bias=None):
        """One speculative round of the reference (src/gen/session.cpp:451-506) for every sequence in one launch.
        logits [n_seq * n_pos, V]: row s*n_pos + j follows the round's token and drafts 0..j-1; drafts [n_seq,
        n_pos - 1] int32; u [n_seq, n_pos + 1] the sequence's uniforms in generator order; history [n_seq, cap] and
        history_len [n_seq] per sequence; forced [n_seq, n_pos] int32 (token or -1) or None. Returns (n_kept [n_seq],
        next_token [n_seq], result with per-position token / accepted / flags)."""
        n_seq, n_drafts = drafts.shape
        n_pos = n_drafts + 1
        assert logits.shape[0] == n_seq * n_pos and drafts.dtype == torch.int32 and drafts.is_contiguous()
        assert u.shape == (n_seq, n_pos + 1) and u.dtype == torch.float32 and u.is_contiguous()
        if forced is not None:
            assert forced.shape == (n_seq, n_pos) and forced.dtype == torch.int32 and forced.is_contiguous()
        r = self._rows(logits, params, history, history_len, mask, bias)
        o = self._out(r.batch)
        kept = torch.empty(n_seq, dtype=torch.int32, device=self.device)
        nxt = torch.empty(n_seq, dtype=torch.int32, device=self.device)
        check(lib.mk_sampler_spec_round(self._h, C.byref(r), n_pos, drafts.data_ptr(), _ptr(forced), u.data_ptr(),
                                        C.byref(o), self.accepted.data_ptr(), kept.data_ptr(), nxt.data_ptr(),
                                        _stream_ptr(self.device)))
        return kept, nxt, self._result(r.batch, accepted=self.accepted[: r.batch])

    def spec_commit(self, drafts, n_kept, next_token, history, history_len, *, next_input=None, flags=None) -> None:
        """The round's bookkeeping on the device: kept drafts, then next_token, appended to each sequence's history
        (history [n_seq, cap] and history_len [n_seq] updated in place); next_input receives next_token."""
        n_seq, n_drafts = drafts.shape
        check(lib.mk_spec_commit(self._h, n_seq, n_drafts + 1, drafts.data_ptr(), n_kept.data_ptr(),
                                 next_token.data_ptr(), history.data_ptr(), history.stride(0), history.shape[1],
                                 history_len.data_ptr(), _ptr(next_input), _ptr(flags), _stream_ptr(self.device)))

    def vp_local(self, shard_logits, params, k: int, records: torch.Tensor, *, id_offset: int, history=None,
                 history_len=None, mask=None, bias=None) -> torch.Tensor:
        """Vocab-parallel step 1: this shard's per-row record (max, sum-exp, k best) into `records` (uint8)."""
        r = self._rows(shard_logits, params, history, history_len, mask, bias, id_offset=id_offset)
        rb = lib.mk_vp_record_bytes(k)
        assert records.dtype == torch.uint8 and records.numel() >= r.batch * rb and records.is_cuda
        check(lib.mk_sampler_vp_local(self._h, C.byref(r), k, records.data_ptr(), _stream_ptr(self.device)))
        return records

    def vp_merge(self, gathered: torch.Tensor, n_shards: int, batch: int, k: int, n_vocab_total: int, params, u):
        """Vocab-parallel step 2 on the all-gathered records [n_shards, batch, record_bytes]."""
        o = self._out(batch)
        c = params.to_c()
        check(lib.mk_sampler_vp_merge(self._h, gathered.data_ptr(), n_shards, batch, k, n_vocab_total, C.byref(c),
                                      _ptr(u), C.byref(o), _stream_ptr(self.device)))
        return self._result(batch)

    def sample_host(self, logits: np.ndarray, params: SamplingParams, u: np.ndarray, *, history=None, mask=None,
                    bias=None):
        """Host buffers in, host buffers out (copies inside): the form the reference's callers have."""
        assert logits.dtype == np.float32 and logits.ndim == 2 and logits.strides[1] == 4
        b, v = logits.shape
        r = RowsC()
        r.logits = logits.ctypes.data
        r.ld = logits.strides[0] // 4
        r.batch, r.n_vocab = b, v
        r.params = params.to_c()
        keep = [logits, u]
        if history is not None:
            assert history.dtype == np.int32 and history.ndim == 2
            r.history, r.history_ld, r.n_history = history.ctypes.data, history.strides[0] // 4, history.shape[1]
            keep.append(history)
        if mask is not None:
            assert mask.dtype == np.uint32 and mask.ndim == 2
            r.mask, r.mask_ld = mask.ctypes.data, mask.strides[0] // 4
            keep.append(mask)
        if bias is not None:
            assert bias.dtype == np.int32 and bias.ndim == 3 and bias.flags.c_contiguous
            r.bias, r.n_bias = bias.ctypes.data, bias.shape[1]
            keep.append(bias)
        tok = np.empty(b, dtype=np.int32)
        prob = np.empty(b, dtype=np.float32)
        flags = np.empty(b, dtype=np.uint32)
        o = SampleOutC()
        o.token, o.prob, o.flags = tok.ctypes.data, prob.ctypes.data, flags.ctypes.data
        check(lib.mk_sampler_sample_host(self._h, C.byref(r), u.ctypes.data if u is not None else None, C.byref(o)))
        return tok, prob, flags


def pack_bias(ids: np.ndarray, vals: np.ndarray) -> np.ndarray:
    """(ids int32 [B, nb], values float32 [B, nb]) -> int32 [B, nb, 2] in the layout of mk_bias."""
    out = np.empty(ids.shape + (2,), dtype=np.int32)
    out[..., 0] = ids
    out[..., 1] = vals.astype(np.float32).view(np.int32)
    return out


def pack_params(ps) -> np.ndarray:
    """List of SamplingParams -> int32 [B, 7] in the layout of mk_sampling_params (per-row parameters)."""
    out = np.empty((len(ps), 7), dtype=np.int32)
    for i, p in enumerate(ps):
        f = np.array([p.temperature, 0, p.top_p, p.min_p, p.presence_penalty, p.frequency_penalty,
                      p.repetition_penalty], dtype=np.float32).view(np.int32)
        out[i] = f
        out[i, 1] = np.array([p.top_k], dtype=np.uint32).view(np.int32)[0]
    return out
