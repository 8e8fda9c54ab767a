"""Local object store with resource versions and watches.

Stands in for the Kubernetes API server that the reference uses as its database (five custom
resource kinds under kubernetes/kustomize/cornserve/base/crds/).  Objects are JSON documents keyed by
(kind, name) in a SQLite file that every service process of one deployment opens; each write bumps a
global, monotonically increasing ``resourceVersion`` and appends an event row, so a watcher that
polls "events after version V" sees ADDED / MODIFIED / DELETED in commit order, can resume after a
restart and can tell when it has caught up with a writer (``sync``).
"""

from __future__ import annotations

import asyncio
import json
import os
import sqlite3
import threading
import time
from collections.abc import AsyncIterator
from dataclasses import dataclass
from typing import Any


class AlreadyExists(Exception):
    pass


class NotFound(Exception):
    pass


@dataclass
class StoredObject:
    kind: str
    name: str
    spec: dict[str, Any]
    resource_version: int


@dataclass
class WatchEvent:
    type: str  # ADDED | MODIFIED | DELETED
    object: StoredObject


class LocalStore:
    def __init__(self, path: str | None = None):
        if path is None:
            from ..constants import STATE_DIR

            path = os.path.join(STATE_DIR, "store.sqlite")
        if path != ":memory:":
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self.path = path
        self._lock = threading.Lock()
        self._db = sqlite3.connect(path, timeout=30.0, check_same_thread=False, isolation_level=None)
        self._db.execute("PRAGMA journal_mode=WAL")
        self._db.executescript(
            """
            CREATE TABLE IF NOT EXISTS meta (k TEXT PRIMARY KEY, v INTEGER);
            INSERT OR IGNORE INTO meta VALUES ('rv', 0);
            CREATE TABLE IF NOT EXISTS objects (kind TEXT, name TEXT, spec TEXT, rv INTEGER, PRIMARY KEY (kind, name));
            CREATE TABLE IF NOT EXISTS events (rv INTEGER PRIMARY KEY, type TEXT, kind TEXT, name TEXT, spec TEXT);
            """
        )

    # -- helpers --------------------------------------------------------------------------------------
    def _tx(self, fn):
        with self._lock:
            self._db.execute("BEGIN IMMEDIATE")
            try:
                out = fn()
                self._db.execute("COMMIT")
                return out
            except BaseException:
                self._db.execute("ROLLBACK")
                raise

    def _bump(self) -> int:
        self._db.execute("UPDATE meta SET v = v + 1 WHERE k = 'rv'")
        return self._db.execute("SELECT v FROM meta WHERE k = 'rv'").fetchone()[0]

    # -- synchronous API -----------------------------------------------------------------------------------
    def create(self, kind: str, name: str, spec: dict[str, Any]) -> StoredObject:
        def run():
            if self._db.execute("SELECT 1 FROM objects WHERE kind=? AND name=?", (kind, name)).fetchone():
                raise AlreadyExists(f"{kind}/{name}")
            rv = self._bump()
            blob = json.dumps(spec)
            self._db.execute("INSERT INTO objects VALUES (?,?,?,?)", (kind, name, blob, rv))
            self._db.execute("INSERT INTO events VALUES (?,?,?,?,?)", (rv, "ADDED", kind, name, blob))
            return StoredObject(kind, name, spec, rv)

        return self._tx(run)

    def update(self, kind: str, name: str, spec: dict[str, Any], create: bool = False) -> StoredObject:
        def run():
            exists = self._db.execute("SELECT 1 FROM objects WHERE kind=? AND name=?", (kind, name)).fetchone()
            if not exists and not create:
                raise NotFound(f"{kind}/{name}")
            rv = self._bump()
            blob = json.dumps(spec)
            self._db.execute("INSERT OR REPLACE INTO objects VALUES (?,?,?,?)", (kind, name, blob, rv))
            self._db.execute("INSERT INTO events VALUES (?,?,?,?,?)",
                             (rv, "MODIFIED" if exists else "ADDED", kind, name, blob))
            return StoredObject(kind, name, spec, rv)

        return self._tx(run)

    def get(self, kind: str, name: str) -> StoredObject:
        with self._lock:
            row = self._db.execute("SELECT spec, rv FROM objects WHERE kind=? AND name=?", (kind, name)).fetchone()
        if row is None:
            raise NotFound(f"{kind}/{name}")
        return StoredObject(kind, name, json.loads(row[0]), row[1])

    def list(self, kind: str, limit: int | None = None) -> list[StoredObject]:
        q = "SELECT name, spec, rv FROM objects WHERE kind=? ORDER BY rv"
        if limit:
            q += f" LIMIT {int(limit)}"
        with self._lock:
            rows = self._db.execute(q, (kind,)).fetchall()
        return [StoredObject(kind, n, json.loads(s), rv) for n, s, rv in rows]

    def delete(self, kind: str, name: str) -> None:
        def run():
            row = self._db.execute("SELECT spec FROM objects WHERE kind=? AND name=?", (kind, name)).fetchone()
            if row is None:
                raise NotFound(f"{kind}/{name}")
            rv = self._bump()
            self._db.execute("DELETE FROM objects WHERE kind=? AND name=?", (kind, name))
            self._db.execute("INSERT INTO events VALUES (?,?,?,?,?)", (rv, "DELETED", kind, name, row[0]))

        self._tx(run)

    def delete_all(self, kind: str) -> int:
        names = [o.name for o in self.list(kind)]
        for n in names:
            try:
                self.delete(kind, n)
            except NotFound:
                pass
        return len(names)

    def resource_version(self) -> int:
        with self._lock:
            return self._db.execute("SELECT v FROM meta WHERE k = 'rv'").fetchone()[0]

    def events_after(self, rv: int, kinds: tuple[str, ...] | None = None) -> list[WatchEvent]:
        with self._lock:
            rows = self._db.execute("SELECT rv, type, kind, name, spec FROM events WHERE rv > ? ORDER BY rv", (rv,)).fetchall()
        return [WatchEvent(t, StoredObject(k, n, json.loads(s), v)) for v, t, k, n, s in rows
                if kinds is None or k in kinds]

    # -- asynchronous watch -----------------------------------------------------------------------------------
    async def watch(self, kinds: tuple[str, ...] | None = None, since: int = 0, poll_s: float = 0.1) -> AsyncIterator[WatchEvent]:
        """Yield every event after ``since`` (0 = replay the whole history), then follow new ones."""
        cursor = since
        while True:
            events = await asyncio.to_thread(self.events_after, cursor, None)
            for ev in events:
                cursor = ev.object.resource_version
                if kinds is None or ev.object.kind in kinds:
                    yield ev
            if not events:
                await asyncio.sleep(poll_s)

    def close(self) -> None:
        with self._lock:
            self._db.close()


_default: LocalStore | None = None


def default_store() -> LocalStore:
    global _default
    if _default is None:
        _default = LocalStore(os.environ.get("CORNSERVE_STORE_PATH"))
    return _default


def wait_for(predicate, timeout_s: float, poll_s: float = 0.05) -> bool:
    end = time.monotonic() + timeout_s
    while time.monotonic() < end:
        if predicate():
            return True
        time.sleep(poll_s)
    return predicate()
