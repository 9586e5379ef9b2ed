"""ctypes view of the host sampler, the drafter's device sampler and the H1 cycle engine."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib
from .lib import check, load
from .model import Model

vp, u32, u64, i32, f32 = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_float
TOKEN_LOGIT = np.dtype([("token", np.uint32), ("logit", np.float32)])


class SamplerOptions(C.Structure):
    _fields_ = [("temperature", f32), ("top_k", u32), ("top_p", f32), ("min_p", f32), ("repetition_penalty", f32),
                ("repetition_window", u32), ("seed", u64)]


def sampler_options(temperature=0.7, top_k=40, top_p=0.95, min_p=0.05, repetition_penalty=1.0, seed=0, window=64):
    return SamplerOptions(temperature, top_k, top_p, min_p, repetition_penalty, window, seed)


class GatheredDraft(C.Structure):
    _fields_ = [("proposal", u32), ("count", u32), ("proposal_mass", u64), ("proposal_cdf_begin", u64),
                ("target_mass", u64 * 256)]


class TokenLogitC(C.Structure):
    _fields_ = [("token", u32), ("logit", f32)]


class H1Options(C.Structure):
    _fields_ = [("sampler", SamplerOptions), ("speculative", i32), ("forced_schedule", i32),
                ("forced_accept_probability", f32), ("schedule_seed", u64), ("record_cycles", i32), ("horizon", u32), ("conditional", i32)]


class H1Stats(C.Structure):
    _fields_ = [(n, u64) for n in ("cycles", "accepted", "rejected", "ordinary_steps", "fallback_cycles",
                                   "emitted_tokens", "law_agreements", "sampler_launches", "drafted_tokens",
                                   "accepted_tokens", "full_law_proposals", "verify_passes")]


class CycleRecord(C.Structure):
    _fields_ = [("root", u32), ("proposal", u32), ("word", u32), ("candidate_count", u32),
                ("candidates", TokenLogitC * 384), ("draft", GatheredDraft), ("token", u32), ("accepted", i32),
                ("target_draws", u32), ("status", i32), ("depth", u32), ("horizon", u32)]


class DraftReceipt(C.Structure):
    _fields_ = [("status", u32), ("count", u32), ("token", u32), ("word", u32), ("ids", u32 * 256), ("cdf", u64 * 257)]


lib.register({
    "gf_h1_verification_schedule": (i32, [u32, i32, vp, vp, vp]),
    "gf_draft_receipt_bytes": (C.c_size_t, []),
    "gf_draft_sample_workspace_bytes": (C.c_size_t, [u32]),
    "gf_draft_sample": (i32, [vp, u32, f32, u32, f32, f32, f32, vp, u32, u32, vp, vp, vp, vp]),
    "gf_draft_resolve_overflow": (i32, [u32, f32, u32, f32, f32, u32, vp, vp, vp, vp]),
    "gf_draft_gather_full": (i32, [vp, u32, vp, u32, vp, vp]),
    "gf_selection_base_bytes": (C.c_size_t, []),
    "gf_selection_requests": (i32, [vp, u32, vp, u32, vp, vp]),
    "gf_sampler_create": (i32, [C.POINTER(SamplerOptions), C.POINTER(vp)]),
    "gf_sampler_destroy": (i32, [vp]),
    "gf_sampler_observe": (i32, [vp, vp, u32]),
    "gf_sampler_preview_proposal_word": (i32, [vp, C.POINTER(u32)]),
    "gf_sampler_preview_proposal_words": (i32, [vp, u32, vp]),
    "gf_sampler_prepare": (i32, [vp, vp, u32, vp, u32, vp, vp, C.POINTER(u32), C.POINTER(C.c_double)]),
    "gf_sampler_sample": (i32, [vp, vp, u32, vp, u32, C.POINTER(u32)]),
    "gf_sampler_sample_speculative": (i32, [vp, C.POINTER(GatheredDraft), vp, u32, vp, u32, C.POINTER(u32),
                                            C.POINTER(i32), C.POINTER(u32)]),
    "gf_h1_create": (i32, [vp, vp, C.POINTER(H1Options), C.POINTER(vp)]),
    "gf_h1_destroy": (i32, [vp]),
    "gf_h1_prefill": (i32, [vp, vp, u32]),
    "gf_h1_generate": (i32, [vp, u32, vp, C.POINTER(u32)]),
    "gf_h1_generate_steps": (i32, [vp, u32, u32, vp, C.POINTER(u32)]),
    "gf_h1_stats_read": (i32, [vp, C.POINTER(H1Stats)]),
    "gf_h1_reseed_schedule": (i32, [vp, u64]),
    "gf_h1_cycle_record_read": (i32, [vp, u32, C.POINTER(CycleRecord)]),
    "gf_h1_cycle_record_count": (u32, [vp]),
})


class Sampler:
    """Host sampler (double precision) behind gf_sampler_*."""

    def __init__(self, options: SamplerOptions):
        self.L = load()
        handle = vp()
        check(self.L.gf_sampler_create(C.byref(options), C.byref(handle)))
        self.handle = handle.value

    def observe(self, tokens) -> None:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        check(self.L.gf_sampler_observe(self.handle, tokens.ctypes.data, tokens.size))

    def proposal_word(self) -> int:
        out = u32()
        check(self.L.gf_sampler_preview_proposal_word(self.handle, C.byref(out)))
        return out.value

    def proposal_words(self, count: int) -> np.ndarray:
        out = np.zeros(count, np.uint32)
        check(self.L.gf_sampler_preview_proposal_words(self.handle, count, out.ctypes.data))
        return out

    def prepare(self, candidates, suffix=()):
        candidates = np.ascontiguousarray(candidates, TOKEN_LOGIT)
        suffix = np.ascontiguousarray(np.array(suffix, np.uint32))
        tokens, weights = np.zeros(256, np.uint32), np.zeros(256, np.float64)
        count, total = u32(), C.c_double()
        check(self.L.gf_sampler_prepare(self.handle, candidates.ctypes.data, candidates.size, suffix.ctypes.data,
                                        suffix.size, tokens.ctypes.data, weights.ctypes.data, C.byref(count), C.byref(total)))
        return tokens[:count.value], weights[:count.value], total.value

    def sample(self, candidates, suffix=()) -> int:
        candidates = np.ascontiguousarray(candidates, TOKEN_LOGIT)
        suffix = np.ascontiguousarray(np.array(suffix, np.uint32))
        out = u32()
        check(self.L.gf_sampler_sample(self.handle, candidates.ctypes.data, candidates.size, suffix.ctypes.data,
                                       suffix.size, C.byref(out)))
        return out.value

    def sample_speculative(self, draft: GatheredDraft, candidates, suffix=()):
        candidates = np.ascontiguousarray(candidates, TOKEN_LOGIT)
        suffix = np.ascontiguousarray(np.array(suffix, np.uint32))
        token, accepted, draws = u32(), i32(), u32()
        status = self.L.gf_sampler_sample_speculative(self.handle, C.byref(draft), candidates.ctypes.data, candidates.size,
                                                      suffix.ctypes.data, suffix.size, C.byref(token), C.byref(accepted),
                                                      C.byref(draws))
        return status, token.value, bool(accepted.value), draws.value

    def close(self):
        if getattr(self, "handle", None):
            self.L.gf_sampler_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gathered_draft(proposal, proposal_mass, cdf_begin, target_mass) -> GatheredDraft:
    draft = GatheredDraft()
    draft.proposal, draft.proposal_mass, draft.proposal_cdf_begin = int(proposal), int(proposal_mass), int(cdf_begin)
    draft.count = len(target_mass)
    for i, mass in enumerate(target_mass):
        draft.target_mass[i] = int(mass)
    return draft


def draft_sample_full(logits: np.ndarray, options: SamplerOptions, word: int, history=(), gather=()):
    """The proposal law over the whole vocabulary: runs the device sampler and, when the compact law
    overflows (status 20), resolves it from the same scores.  Returns (receipt, intervals) where
    intervals[i] = (begin, end) of token gather[i] in the full CDF (None for a compact receipt)."""
    L = load()
    logits = np.ascontiguousarray(logits, np.float32)
    history = np.ascontiguousarray(np.array(history, np.uint32))
    src = lib.DeviceBuffer.from_numpy(logits)
    ws = lib.DeviceBuffer(L.gf_draft_sample_workspace_bytes(logits.size))
    receipt = lib.DeviceBuffer(C.sizeof(DraftReceipt))
    token = lib.DeviceBuffer(16)
    check(L.gf_draft_sample(src.ptr, logits.size, options.temperature, options.top_k, options.top_p, options.min_p,
                            options.repetition_penalty, history.ctypes.data if history.size else None, history.size,
                            word, ws.ptr, receipt.ptr, token.ptr, None))
    out = DraftReceipt.from_buffer_copy(receipt.download(np.uint8).tobytes())
    if out.status == 20:
        check(L.gf_draft_resolve_overflow(logits.size, options.temperature, options.top_k, options.top_p, options.min_p,
                                          word, ws.ptr, receipt.ptr, token.ptr, None))
        out = DraftReceipt.from_buffer_copy(receipt.download(np.uint8).tobytes())
    intervals = None
    if out.count == 0xffffffff:
        intervals = []
        tokens = np.ascontiguousarray(np.array(gather, np.uint32))
        for begin in range(0, tokens.size, 256):
            part = np.ascontiguousarray(tokens[begin:begin + 256])
            got = np.zeros(2 * part.size, np.uint64)
            check(L.gf_draft_gather_full(ws.ptr, logits.size, part.ctypes.data, part.size, got.ctypes.data, None))
            intervals.append(got.reshape(-1, 2))
        intervals = np.concatenate(intervals) if intervals else np.zeros((0, 2), np.uint64)
    for b in (src, ws, receipt, token):
        b.free()
    return out, intervals


def draft_sample(logits: np.ndarray, options: SamplerOptions, word: int, history=()) -> DraftReceipt:
    """Runs the drafter's device sampler on one row of logits and returns the receipt."""
    L = load()
    logits = np.ascontiguousarray(logits, np.float32)
    history = np.ascontiguousarray(np.array(history, np.uint32))
    src = lib.DeviceBuffer.from_numpy(logits)
    ws = lib.DeviceBuffer(L.gf_draft_sample_workspace_bytes(logits.size))
    receipt = lib.DeviceBuffer(C.sizeof(DraftReceipt))
    token = lib.DeviceBuffer(16)
    check(L.gf_draft_sample(src.ptr, logits.size, options.temperature, options.top_k, options.top_p, options.min_p,
                            options.repetition_penalty, history.ctypes.data if history.size else None, history.size,
                            word, ws.ptr, receipt.ptr, token.ptr, None))
    out = DraftReceipt.from_buffer_copy(receipt.download(np.uint8).tobytes())
    for b in (src, ws, receipt, token):
        b.free()
    return out


class H1:
    """The speculative (or ordinary) generation engine over a target plan and a drafter plan."""

    def __init__(self, target: Model, draft: Model | None, options: H1Options):
        self.L = load()
        self.target, self.draft = target, draft
        handle = vp()
        check(self.L.gf_h1_create(target.handle, draft.handle if draft else None, C.byref(options), C.byref(handle)))
        self.handle = handle.value

    def prefill(self, tokens) -> None:
        tokens = np.ascontiguousarray(tokens, np.uint32)
        check(self.L.gf_h1_prefill(self.handle, tokens.ctypes.data, tokens.size))

    def generate(self, max_tokens: int) -> np.ndarray:
        out = np.zeros(max_tokens, np.uint32)
        count = u32()
        check(self.L.gf_h1_generate(self.handle, max_tokens, out.ctypes.data, C.byref(count)))
        return out[:count.value]

    def generate_steps(self, steps: int, max_tokens: int | None = None) -> np.ndarray:
        max_tokens = max_tokens or 2 * steps + 2
        out = np.zeros(max_tokens, np.uint32)
        count = u32()
        check(self.L.gf_h1_generate_steps(self.handle, steps, max_tokens, out.ctypes.data, C.byref(count)))
        return out[:count.value]

    def stats(self) -> H1Stats:
        stats = H1Stats()
        check(self.L.gf_h1_stats_read(self.handle, C.byref(stats)))
        return stats

    def reseed_schedule(self, seed: int) -> None:
        check(self.L.gf_h1_reseed_schedule(self.handle, seed))

    def records(self):
        out = []
        for i in range(self.L.gf_h1_cycle_record_count(self.handle)):
            record = CycleRecord()
            check(self.L.gf_h1_cycle_record_read(self.handle, i, C.byref(record)))
            out.append(record)
        return out

    def close(self):
        if getattr(self, "handle", None):
            self.L.gf_h1_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def verification_schedule(horizon: int, conditional: bool) -> list:
    """(drafts, rows) of every verification pass of a cycle with `horizon` drafts."""
    drafts, rows, tiles = (u32 * 4)(), (u32 * 4)(), u32()
    check(lib.load().gf_h1_verification_schedule(horizon, int(conditional), drafts, rows, C.byref(tiles)))
    return [(drafts[t], rows[t]) for t in range(tiles.value)]
