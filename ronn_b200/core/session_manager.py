"""Session manager: admission control and per-session statistics
(crates/ronn-core/src/session.rs:17-550).  ``max_sessions`` (100), per-session
``max_concurrent_inferences`` (10), ``timeout_seconds`` (30), 1-hour expiry sweep, statistics
(count / avg / min / max ms / errors), ``destroy_session`` waits up to 5 s for running inferences.
Inference runs a real ``InferenceSession`` (the reference's ``execute_inference`` returns ones[1,10])."""
from __future__ import annotations

import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..api.errors import SessionError


@dataclass
class SessionConfig:
    max_concurrent_inferences: int = 10
    timeout_seconds: float = 30.0
    memory_limit: Optional[int] = None
    expiry_seconds: float = 3600.0


@dataclass
class SessionStatistics:
    inference_count: int = 0
    total_time_ms: float = 0.0
    min_time_ms: float = 0.0
    max_time_ms: float = 0.0
    error_count: int = 0
    created_at: float = field(default_factory=time.time)
    last_used: float = field(default_factory=time.time)

    @property
    def average_time_ms(self) -> float:
        return self.total_time_ms / self.inference_count if self.inference_count else 0.0


@dataclass
class GlobalStatistics:
    session_count: int
    total_inferences: int
    total_errors: int
    average_time_ms: float


class _Managed:
    def __init__(self, session, config: SessionConfig):
        self.session = session
        self.config = config
        self.stats = SessionStatistics()
        self.active = 0
        self.lock = threading.Lock()
        self.idle = threading.Condition(self.lock)


class SessionManager:
    def __init__(self, max_sessions: int = 100):
        self.max_sessions = max_sessions
        self._sessions: Dict[str, _Managed] = {}
        self._lock = threading.Lock()

    def create_session(self, model, options=None, config: Optional[SessionConfig] = None) -> str:
        config = config or SessionConfig()
        with self._lock:
            self._sweep_locked()
            if len(self._sessions) >= self.max_sessions:
                raise SessionError(f"maximum number of sessions ({self.max_sessions}) reached")
        model.graph.validate()            # cyclic / dangling graphs are rejected at creation
        sess = model.create_session(options) if options is not None else model.create_session_default()
        sid = str(uuid.uuid4())
        with self._lock:
            if len(self._sessions) >= self.max_sessions:
                raise SessionError(f"maximum number of sessions ({self.max_sessions}) reached")
            self._sessions[sid] = _Managed(sess, config)
        return sid

    def _get(self, sid: str) -> _Managed:
        with self._lock:
            m = self._sessions.get(sid)
        if m is None:
            raise SessionError(f"session {sid} not found")
        return m

    def run_inference(self, sid: str, inputs):
        m = self._get(sid)
        with m.lock:
            if m.active >= m.config.max_concurrent_inferences:
                raise SessionError("too many concurrent inferences for this session")
            m.active += 1
        t0 = time.perf_counter()
        try:
            out = m.session.run(inputs)
            ms = (time.perf_counter() - t0) * 1e3
            if ms > m.config.timeout_seconds * 1e3:
                raise SessionError(f"inference exceeded the session timeout ({m.config.timeout_seconds} s)")
            with m.lock:
                s = m.stats
                s.min_time_ms = ms if s.inference_count == 0 else min(s.min_time_ms, ms)
                s.max_time_ms = max(s.max_time_ms, ms)
                s.inference_count += 1
                s.total_time_ms += ms
                s.last_used = time.time()
            return out
        except Exception:
            with m.lock:
                m.stats.error_count += 1
            raise
        finally:
            with m.lock:
                m.active -= 1
                m.idle.notify_all()

    def get_session_statistics(self, sid: str) -> SessionStatistics:
        return self._get(sid).stats

    def list_sessions(self) -> List[str]:
        with self._lock:
            return list(self._sessions)

    def session_count(self) -> int:
        with self._lock:
            return len(self._sessions)

    def destroy_session(self, sid: str, wait_seconds: float = 5.0) -> None:
        m = self._get(sid)
        deadline = time.time() + wait_seconds
        with m.lock:
            while m.active > 0 and time.time() < deadline:
                m.idle.wait(timeout=max(deadline - time.time(), 0.01))
        with self._lock:
            self._sessions.pop(sid, None)

    def _sweep_locked(self) -> None:
        now = time.time()
        for sid in [s for s, m in self._sessions.items() if now - m.stats.last_used > m.config.expiry_seconds and m.active == 0]:
            del self._sessions[sid]

    def cleanup_expired(self) -> None:
        with self._lock:
            self._sweep_locked()

    def global_statistics(self) -> GlobalStatistics:
        with self._lock:
            ms = list(self._sessions.values())
        n = sum(m.stats.inference_count for m in ms)
        t = sum(m.stats.total_time_ms for m in ms)
        return GlobalStatistics(len(ms), n, sum(m.stats.error_count for m in ms), t / n if n else 0.0)

    def shutdown(self) -> None:
        for sid in self.list_sessions():
            self.destroy_session(sid)


@dataclass
class AdmissionTicket:
    client: str
    admitted_at: float
    deadline: float


class RequestAdmission:
    """Admission control of the serving front end with the SessionManager's vocabulary: ``max_in_flight`` plays the
    role of ``max_sessions`` (requests admitted and not yet answered), ``max_per_client`` that of a session's
    ``max_concurrent_inferences``, ``timeout_seconds`` that of its inference timeout.  ``acquire`` returns a ticket or
    None (refused); ``release`` returns it and feeds the statistics (count, average / min / max ms, errors)."""

    def __init__(self, max_in_flight: int = 1024, max_per_client: int = 256, timeout_seconds: float = 600.0):
        self.max_in_flight = max_in_flight
        self.max_per_client = max_per_client
        self.timeout_seconds = timeout_seconds
        self._lock = threading.Lock()
        self._per_client: Dict[str, int] = {}
        self._in_flight = 0
        self.refused = 0
        self.stats = SessionStatistics()

    def acquire(self, client: str = "local") -> Optional[AdmissionTicket]:
        now = time.time()
        with self._lock:
            if self._in_flight >= self.max_in_flight or self._per_client.get(client, 0) >= self.max_per_client:
                self.refused += 1
                return None
            self._in_flight += 1
            self._per_client[client] = self._per_client.get(client, 0) + 1
        return AdmissionTicket(client, now, now + self.timeout_seconds)

    def expired(self, ticket: AdmissionTicket) -> bool:
        return time.time() > ticket.deadline

    def release(self, ticket: AdmissionTicket, error: bool = False) -> None:
        ms = (time.time() - ticket.admitted_at) * 1e3
        with self._lock:
            if ticket.deadline < 0:
                return                                  # already released
            ticket.deadline = -1.0
            self._in_flight -= 1
            left = self._per_client.get(ticket.client, 1) - 1
            if left <= 0:
                self._per_client.pop(ticket.client, None)
            else:
                self._per_client[ticket.client] = left
            s = self.stats
            if error:
                s.error_count += 1
            else:
                s.min_time_ms = ms if s.inference_count == 0 else min(s.min_time_ms, ms)
                s.max_time_ms = max(s.max_time_ms, ms)
                s.inference_count += 1
                s.total_time_ms += ms
            s.last_used = time.time()

    def snapshot(self) -> Dict[str, float]:
        with self._lock:
            return {"in_flight": self._in_flight, "clients": len(self._per_client), "refused": self.refused,
                    "answered": self.stats.inference_count, "errors": self.stats.error_count,
                    "average_ms": round(self.stats.average_time_ms, 3)}
