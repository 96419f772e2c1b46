"""Structured event lines on stderr and the byte totals behind them.

Line format of the reference (crates/kf-core/src/event.rs:31-72): `kungfu event=<name> k=v ...`; a value with a
space, a quote or an equals sign travels as a JSON string, compact JSON objects and arrays travel as they are.
Events of this engine: `plan` (the cache plan before anything is allocated), `alloc` (pool, kind, bytes; totals are
kept, event.rs:74-100), `ready`, `request`, `error`.  Nothing is printed unless `enabled` is set (the engine's
`events` option and the command line's `--events`); the totals and counters are kept either way.
"""
from __future__ import annotations

import json
import sys
import threading

enabled = False
_lock = threading.Lock()
_totals: dict[str, int] = {}
counters: dict[str, int] = {}


def quote(v) -> str:
    v = str(v)
    compact = not any(c.isspace() or ord(c) < 32 for c in v)
    is_json = compact and ((v.startswith("{") and v.endswith("}")) or (v.startswith("[") and v.endswith("]")))
    plain = bool(v) and compact and '"' not in v and "=" not in v
    return v if (plain or is_json) else json.dumps(v)


def emit(name: str, **fields) -> None:
    """One event line on stderr (when events are enabled)."""
    count(f"event.{name}")
    if not enabled:
        return
    line = " ".join([f"kungfu event={name}"] + [f"{k}={quote(v)}" for k, v in fields.items()])
    with _lock:
        print(line, file=sys.stderr, flush=True)


def alloc(pool: str, kind: str, nbytes: int) -> None:
    """Bytes taken from `pool` (a device, 'host') for `kind` ('weights', 'cache', 'state', 'workspace')."""
    with _lock:
        _totals[f"{pool}.{kind}"] = _totals.get(f"{pool}.{kind}", 0) + int(nbytes)
    emit("alloc", pool=pool, kind=kind, bytes=int(nbytes))


def release(pool: str, kind: str, nbytes: int) -> None:
    with _lock:
        key = f"{pool}.{kind}"
        _totals[key] = max(0, _totals.get(key, 0) - int(nbytes))


def totals() -> dict[str, int]:
    with _lock:
        return dict(_totals)


def error(code: str, **fields) -> None:
    emit("error", code=code, **fields)


def count(name: str, n: int = 1) -> None:
    counters[name] = counters.get(name, 0) + n
