"""Host-side handoff coordinator (``tkv_coordinator_*``): routing of new requests to prefill workers, admission of
finished prefills to decode workers against their pools' free pages, overdue handoffs and the fallback to
re-prefill.  No CUDA, no torch: it only keeps the books the device calls report into."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

from . import _native as N
from ._native import TkvError, lib


def _check(rc: int) -> None:
    if rc != 0:
        buf = C.create_string_buffer(512)
        lib().tkv_last_error(buf, 512)
        raise TkvError(rc, buf.value.decode())


class Coordinator:
    def __init__(self, n_prefill: int, n_decode: int, block_size: int = 16, max_inflight_per_decode: int = 0, max_retries: int = 1,
                 headroom_blocks: int = 0, handoff_timeout: int = 0):
        cfg = N.TkvCoordinatorConfig(n_prefill, n_decode, block_size, max_inflight_per_decode, max_retries, headroom_blocks, handoff_timeout)
        self._h = lib().tkv_coordinator_new(C.byref(cfg))
        if not self._h:
            _check(N.ERR_INVALID_CONFIG)

    def close(self) -> None:
        if self._h:
            lib().tkv_coordinator_delete(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_headroom(self, decode_worker: int, free_blocks: int) -> None:
        _check(lib().tkv_coordinator_set_headroom(self._h, decode_worker, free_blocks))

    def submit(self, request_id: int, n_tokens: int, max_new_tokens: int = 0, priority: int = 5) -> int:
        w = C.c_uint32()
        _check(lib().tkv_coordinator_submit(self._h, request_id, n_tokens, max_new_tokens, priority, C.byref(w)))
        return int(w.value)

    def next_prefill(self, prefill_worker: int) -> Optional[int]:
        rid = C.c_uint64()
        rc = lib().tkv_coordinator_next_prefill(self._h, prefill_worker, C.byref(rid))
        if rc < 0:
            _check(N.ERR_INVALID_CONFIG)
        return int(rid.value) if rc == 1 else None

    def prefill_done(self, request_id: int, prefix_tokens_resident: int = 0) -> None:
        _check(lib().tkv_coordinator_prefill_done(self._h, request_id, prefix_tokens_resident))

    def admit(self, cap: int = 64) -> List[N.TkvAdmission]:
        out = (N.TkvAdmission * cap)()
        n = lib().tkv_coordinator_admit(self._h, out, cap)
        return [out[i] for i in range(n)]

    def handoff_started(self, request_id: int, now: int = 0) -> None:
        _check(lib().tkv_coordinator_handoff_started(self._h, request_id, now))

    def handoff_complete(self, request_id: int) -> None:
        _check(lib().tkv_coordinator_handoff_complete(self._h, request_id))

    def handoff_failed(self, request_id: int) -> int:
        action = C.c_uint32()
        _check(lib().tkv_coordinator_handoff_failed(self._h, request_id, C.byref(action)))
        return int(action.value)

    def timed_out(self, now: int, cap: int = 64) -> List[int]:
        ids = (C.c_uint64 * cap)()
        n = lib().tkv_coordinator_timed_out(self._h, now, ids, cap)
        return [int(ids[i]) for i in range(n)]

    def reprefill_done(self, request_id: int) -> None:
        _check(lib().tkv_coordinator_reprefill_done(self._h, request_id))

    def finish(self, request_id: int) -> None:
        _check(lib().tkv_coordinator_finish(self._h, request_id))

    def request(self, request_id: int) -> Optional[N.TkvRequestInfo]:
        info = N.TkvRequestInfo()
        return info if lib().tkv_coordinator_request(self._h, request_id, C.byref(info)) == 1 else None

    def stats(self) -> N.TkvCoordinatorStats:
        st = N.TkvCoordinatorStats()
        _check(lib().tkv_coordinator_stats(self._h, C.byref(st)))
        return st
