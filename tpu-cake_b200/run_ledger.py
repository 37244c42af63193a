"""Append-only run ledger (SQLite): one row per (run, state), legal transitions only.

Same state machine and guarantees as the reference's ``ExperimentLedger``
(src/tpu_cake/ledger.py:29-41 transitions, :59-183 append rules): a run is created once, moves
CREATED -> VERIFIED -> LOWERED -> COMPILED -> CORRECT -> {TIMED | TRACED | COUNTERED | VALIDATED}
-> ACCEPTED, may be REJECTED from any non-terminal state, and repeating a completed state is
accepted only with a byte-identical payload (idempotent completion).
"""

from __future__ import annotations

import hashlib
import json
import sqlite3
import time
from dataclasses import dataclass
from enum import StrEnum
from pathlib import Path
from typing import Callable, Mapping


class RunState(StrEnum):
    CREATED = "created"
    VERIFIED = "verified"
    LOWERED = "lowered"
    COMPILED = "compiled"
    CORRECT = "correct"
    TIMED = "timed"
    TRACED = "traced"
    COUNTERED = "countered"
    VALIDATED = "validated"
    ACCEPTED = "accepted"
    REJECTED = "rejected"


_MEASURED = (RunState.TIMED, RunState.TRACED, RunState.COUNTERED, RunState.VALIDATED)
_SUCCESSORS: dict[RunState, tuple[RunState, ...]] = {
    RunState.CREATED: (RunState.VERIFIED,),
    RunState.VERIFIED: (RunState.LOWERED,),
    RunState.LOWERED: (RunState.COMPILED,),
    RunState.COMPILED: (RunState.CORRECT,),
    RunState.CORRECT: _MEASURED,
    **{state: (RunState.ACCEPTED,) for state in _MEASURED},
}
_TERMINAL = (RunState.ACCEPTED, RunState.REJECTED)


def payload_sha256(payload: Mapping[str, object]) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


@dataclass(frozen=True)
class LedgerEvent:
    sequence: int
    run_id: str
    state: RunState
    timestamp_ns: int
    payload_sha256: str


class RunLedger:
    def __init__(self, path: Path, *, clock_ns: Callable[[], int] = time.time_ns):
        self.path = Path(path)
        self._clock_ns = clock_ns
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self._db = sqlite3.connect(self.path)
        self._db.execute("PRAGMA journal_mode=WAL")
        self._db.execute("PRAGMA synchronous=FULL")
        self._db.execute(
            "CREATE TABLE IF NOT EXISTS events (sequence INTEGER PRIMARY KEY AUTOINCREMENT, run_id TEXT NOT NULL, "
            "state TEXT NOT NULL, timestamp_ns INTEGER NOT NULL, payload_sha256 TEXT NOT NULL, UNIQUE(run_id, state))"
        )
        self._db.commit()

    def __enter__(self) -> "RunLedger":
        return self

    def __exit__(self, *_exc) -> None:
        self.close()

    def close(self) -> None:
        self._db.execute("PRAGMA wal_checkpoint(TRUNCATE)")
        self._db.close()

    def history(self, run_id: str) -> list[LedgerEvent]:
        rows = self._db.execute(
            "SELECT sequence, run_id, state, timestamp_ns, payload_sha256 FROM events WHERE run_id = ? ORDER BY sequence", (run_id,)
        ).fetchall()
        return [LedgerEvent(r[0], r[1], RunState(r[2]), r[3], r[4]) for r in rows]

    def current_state(self, run_id: str) -> RunState | None:
        events = self.history(run_id)
        return events[-1].state if events else None

    def create(self, run_id: str, payload: Mapping[str, object]) -> LedgerEvent:
        if self.current_state(run_id) not in (None, RunState.CREATED):
            raise ValueError(f"run {run_id} already exists")
        return self._append(run_id, RunState.CREATED, payload)

    def transition(self, run_id: str, state: RunState, payload: Mapping[str, object]) -> LedgerEvent:
        previous = self.current_state(run_id)
        if previous is None:
            raise ValueError(f"run {run_id} does not exist")
        if previous is not state:
            if previous in _TERMINAL:
                raise ValueError(f"run {run_id} is already terminal at {previous.value}")
            if state is not RunState.REJECTED and state not in _SUCCESSORS.get(previous, ()):
                raise ValueError(f"invalid run transition {previous.value} -> {state.value}")
        return self._append(run_id, state, payload)

    def _append(self, run_id: str, state: RunState, payload: Mapping[str, object]) -> LedgerEvent:
        digest = payload_sha256(payload)
        with self._db:
            row = self._db.execute(
                "SELECT sequence, timestamp_ns, payload_sha256 FROM events WHERE run_id = ? AND state = ?", (run_id, state.value)
            ).fetchone()
            if row is not None:
                if row[2] != digest:
                    raise ValueError(f"conflicting duplicate completion for {run_id} at {state.value}")
                return LedgerEvent(row[0], run_id, state, row[1], digest)
            stamp = self._clock_ns()
            cursor = self._db.execute(
                "INSERT INTO events (run_id, state, timestamp_ns, payload_sha256) VALUES (?, ?, ?, ?)", (run_id, state.value, stamp, digest)
            )
            return LedgerEvent(cursor.lastrowid, run_id, state, stamp, digest)
