"""Append-only JSONL event log with an FNV-1a hash chain: every line carries the previous line's hash and the hash of
(prev_hash + its own canonical payload), so an edit or a dropped line anywhere breaks the chain at that point.  A partial
last line (crash in mid-write) is tolerated and reported.  ``report()`` summarises a log for the ``gle_report`` tool.

Reference counterparts: src/gle/gle_telemetry.h:17-93, gle_telemetry.cpp, tools/gle_report.cpp."""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import List

EVENT_TYPES = ["UNKNOWN", "RUN_STARTED", "BAR_FROZEN", "UNIT_SPLIT", "BUILD_DONE", "CRITIC_VERDICT", "ARBITER_RULING",
               "ANTICHEAT_SWEEP", "BUILD_RESULT", "TEST_RESULT", "BENCH_SNAPSHOT", "REGRESSION_CHECK", "CLAIM_VERIFIED",
               "PHASE_EXIT", "PANIC_STOP", "RUN_ENDED", "AGENT_STARTED", "INVALID_ROUND"]


def fnv1a64(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


@dataclass
class Event:
    run_id: str = ""
    phase: str = ""
    task: str = ""
    type: str = "UNKNOWN"
    actor: str = ""
    verdict: str = "-"
    evidence: str = ""
    numbers: dict = field(default_factory=dict)
    ts: str = ""
    prev_hash: str = "0"
    hash: str = ""

    def payload(self) -> str:
        d = asdict(self)
        d.pop("hash"), d.pop("prev_hash")
        return json.dumps(d, sort_keys=True, separators=(",", ":"))

    def compute_hash(self) -> str:
        return format(fnv1a64((self.prev_hash + self.payload()).encode()), "016x")


def to_json_line(e: Event) -> str:
    return json.dumps(asdict(e), sort_keys=True, separators=(",", ":"))


@dataclass
class ChainReport:
    lines_read: int = 0
    events_parsed: int = 0
    skipped_lines: int = 0
    truncated_tail: bool = False
    first_bad_line: int = 0
    chain_valid: bool = True


class TelemetryReader:
    def __init__(self, path):
        self.events: List[Event] = []
        self.lines: List[int] = []
        self.rep = ChainReport()
        if not os.path.exists(path):
            return
        raw = open(path, "r", encoding="utf-8", errors="replace").read().split("\n")
        nonempty = [(i + 1, l) for i, l in enumerate(raw) if l.strip()]
        for k, (ln, l) in enumerate(nonempty):
            self.rep.lines_read += 1
            try:
                d = json.loads(l)
                self.events.append(Event(**d))
                self.lines.append(ln)
                self.rep.events_parsed += 1
            except (ValueError, TypeError):
                self.rep.skipped_lines += 1
                if k == len(nonempty) - 1:
                    self.rep.truncated_tail = True
        self.rep = self.verify_chain()

    def report(self) -> ChainReport:
        return self.rep

    def verify_chain(self) -> ChainReport:
        r = ChainReport(**asdict(self.rep))
        prev = "0"
        r.chain_valid, r.first_bad_line = True, 0
        for e, ln in zip(self.events, self.lines):
            if e.prev_hash != prev or e.compute_hash() != e.hash:
                r.chain_valid, r.first_bad_line = False, ln
                break
            prev = e.hash
        if r.skipped_lines and not (r.skipped_lines == 1 and r.truncated_tail):
            r.chain_valid = False
            r.first_bad_line = r.first_bad_line or -1
        return r

    def last_hash(self) -> str:
        return self.events[-1].hash if self.events else "0"


class TelemetryWriter:
    def __init__(self, path):
        self.path = path
        self.prev = TelemetryReader(path).last_hash()
        self.f = open(path, "a", encoding="utf-8")

    def append(self, e: Event) -> str:
        if e.type not in EVENT_TYPES:
            e.type = "UNKNOWN"
        e.ts = e.ts or time.strftime("%Y-%m-%dT%H:%M:%S%z")
        e.prev_hash = self.prev
        e.hash = e.compute_hash()
        self.f.write(to_json_line(e) + "\n")
        self.f.flush()
        self.prev = e.hash
        return e.hash

    def close(self):
        self.f.close()


def report(path) -> str:
    r = TelemetryReader(path)
    rep = r.report()
    by_type, verdicts = {}, {}
    for e in r.events:
        by_type[e.type] = by_type.get(e.type, 0) + 1
        if e.verdict not in ("", "-"):
            verdicts[e.verdict] = verdicts.get(e.verdict, 0) + 1
    lines = [f"GLE log: {path}", f"events: {rep.events_parsed} (lines {rep.lines_read}, skipped {rep.skipped_lines})",
             f"chain: {'VALID' if rep.chain_valid else 'BROKEN at line %d' % rep.first_bad_line}"
             + (" (partial last line)" if rep.truncated_tail else "")]
    lines += [f"  {t}: {n}" for t, n in sorted(by_type.items())]
    if verdicts:
        lines.append("verdicts: " + ", ".join(f"{k}={v}" for k, v in sorted(verdicts.items())))
    return "\n".join(lines) + "\n"
