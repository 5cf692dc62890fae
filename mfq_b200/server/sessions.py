"""SQLite session store: chat sessions and their messages, as the control API of the server exposes them.

One file, two tables, WAL mode; every call opens a short transaction, so the store can be shared by the server's
worker threads.  Reference: ``mfq/server/state/session_store.py`` (sessions, messages, titles, ordering by update time).
"""

from __future__ import annotations

import json
import sqlite3
import threading
import time
import uuid
from pathlib import Path


class SessionStore:
    def __init__(self, path: str | Path = ":memory:") -> None:
        self._db = sqlite3.connect(str(path), check_same_thread=False)
        self._lock = threading.Lock()
        with self._db:
            if str(path) != ":memory:":
                self._db.execute("PRAGMA journal_mode=WAL")
            self._db.execute("CREATE TABLE IF NOT EXISTS sessions (id TEXT PRIMARY KEY, title TEXT, model TEXT, created REAL, "
                             "updated REAL, meta TEXT)")
            self._db.execute("CREATE TABLE IF NOT EXISTS messages (session_id TEXT, seq INTEGER, role TEXT, content TEXT, "
                             "created REAL, meta TEXT, PRIMARY KEY (session_id, seq))")

    def create(self, title: str = "", model: str | None = None, meta: dict | None = None) -> dict:
        sid, now = uuid.uuid4().hex, time.time()
        with self._lock, self._db:
            self._db.execute("INSERT INTO sessions VALUES (?,?,?,?,?,?)", (sid, title, model, now, now, json.dumps(meta or {})))
        return self.get(sid)

    def get(self, sid: str) -> dict | None:
        with self._lock:
            row = self._db.execute("SELECT id,title,model,created,updated,meta FROM sessions WHERE id=?", (sid,)).fetchone()
            if row is None:
                return None
            msgs = self._db.execute("SELECT seq,role,content,created,meta FROM messages WHERE session_id=? ORDER BY seq", (sid,)).fetchall()
        return {"id": row[0], "title": row[1], "model": row[2], "created": row[3], "updated": row[4], "meta": json.loads(row[5]),
                "messages": [{"seq": m[0], "role": m[1], "content": m[2], "created": m[3], "meta": json.loads(m[4])} for m in msgs]}

    def list(self, limit: int = 100) -> list[dict]:
        with self._lock:
            rows = self._db.execute("SELECT s.id,s.title,s.model,s.updated,(SELECT COUNT(*) FROM messages m WHERE m.session_id=s.id) "
                                    "FROM sessions s ORDER BY s.updated DESC LIMIT ?", (limit,)).fetchall()
        return [{"id": r[0], "title": r[1], "model": r[2], "updated": r[3], "messages": r[4]} for r in rows]

    def append(self, sid: str, role: str, content: str, meta: dict | None = None) -> int:
        now = time.time()
        with self._lock, self._db:
            if self._db.execute("SELECT 1 FROM sessions WHERE id=?", (sid,)).fetchone() is None:
                raise KeyError(sid)
            seq = self._db.execute("SELECT COALESCE(MAX(seq), -1) + 1 FROM messages WHERE session_id=?", (sid,)).fetchone()[0]
            self._db.execute("INSERT INTO messages VALUES (?,?,?,?,?,?)", (sid, seq, role, content, now, json.dumps(meta or {})))
            self._db.execute("UPDATE sessions SET updated=? WHERE id=?", (now, sid))
        return seq

    def rename(self, sid: str, title: str) -> bool:
        with self._lock, self._db:
            return self._db.execute("UPDATE sessions SET title=?, updated=? WHERE id=?", (title, time.time(), sid)).rowcount > 0

    def delete(self, sid: str) -> bool:
        with self._lock, self._db:
            self._db.execute("DELETE FROM messages WHERE session_id=?", (sid,))
            return self._db.execute("DELETE FROM sessions WHERE id=?", (sid,)).rowcount > 0
