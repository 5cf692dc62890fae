"""Model catalog: what the server can load, found on disk and remembered across restarts.

Artifacts are discovered by scanning root directories: packed checkpoints (``*.mfq``, sharded sets count once under the
name of their first shard), GGUF files, and Hugging Face directories (``config.json`` next to ``*.safetensors``).  Every
entry records id, path, kind, byte size, modification time and -- for packed checkpoints -- what the header says about
architecture and quantization, so a client can choose a model without opening files.  Aliases map public model names
to entries; :meth:`ModelCatalog.resolve` is what the model service calls for a name it has not loaded yet.  The catalog
persists as one JSON document (atomic replace), entries whose files vanished are dropped by the next scan.

Reference: ``mfq/server/state/catalog.py`` (catalog of local artifacts with aliases), ``mfq/server/api/routes`` model
management routes.
"""

from __future__ import annotations

import json
import os
import re
import threading
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

_SHARD_RE = re.compile(r"^(?P<stem>.+)-(?P<index>\d{5})-of-(?P<count>\d{5})\.mfq$")


class ArtifactNotFound(KeyError):
    pass


@dataclass
class Artifact:
    id: str
    path: str
    kind: str  # "mfq", "gguf" or "hf"
    bytes: int
    modified_at: float
    shards: int = 1
    arch: str | None = None
    quantization: dict = field(default_factory=dict)
    aliases: list[str] = field(default_factory=list)
    added_at: float = field(default_factory=time.time)


def _mfq_summary(path: Path) -> tuple[str | None, dict]:
    try:
        from ..formats import open_mfq
        with open_mfq(path) as store:
            extra = store.header.extra or {}
            kinds: dict[str, int] = {}
            for name in store.records:
                d = store.dtype(name)
                kinds[d] = kinds.get(d, 0) + 1
            return store.header.model_arch, {"tensor_dtypes": kinds, **({"recipe": extra["quantization"]} if "quantization" in extra else {})}
    except Exception as exc:  # an unreadable file is still listed, with the reason
        return None, {"error": f"{type(exc).__name__}: {exc}"}


def _dir_bytes(files) -> int:
    return sum(f.stat().st_size for f in files)


def discover(root: Path) -> list[Artifact]:
    """Artifacts below ``root`` (not following symlinked directories)."""
    out: list[Artifact] = []
    root = Path(root)
    if not root.exists():
        return out
    seen_sets: set[str] = set()
    for dirpath, dirnames, filenames in os.walk(root):
        d = Path(dirpath)
        names = sorted(filenames)
        if "config.json" in names and any(n.endswith(".safetensors") for n in names):
            files = [d / n for n in names if n.endswith((".safetensors", ".json", ".model", ".txt"))]
            out.append(Artifact(d.name, str(d), "hf", _dir_bytes(files), max(f.stat().st_mtime for f in files)))
        for n in names:
            p = d / n
            if n.endswith(".gguf"):
                out.append(Artifact(p.stem, str(p), "gguf", p.stat().st_size, p.stat().st_mtime))
            elif n.endswith(".mfq"):
                m = _SHARD_RE.match(n)
                if m:
                    key = str(d / m["stem"])
                    if key in seen_sets:
                        continue
                    seen_sets.add(key)
                    shards = sorted(d.glob(f"{m['stem']}-*-of-{m['count']}.mfq"))
                    arch, quant = _mfq_summary(shards[0])
                    out.append(Artifact(m["stem"], str(shards[0]), "mfq", _dir_bytes(shards), max(s.stat().st_mtime for s in shards),
                                        shards=len(shards), arch=arch, quantization=quant))
                else:
                    arch, quant = _mfq_summary(p)
                    out.append(Artifact(p.stem, str(p), "mfq", p.stat().st_size, p.stat().st_mtime, arch=arch, quantization=quant))
    return out


class ModelCatalog:
    def __init__(self, state_file: str | Path | None = None, roots: list[str | Path] | None = None) -> None:
        self.state_file = Path(state_file) if state_file else None
        self.roots = [str(Path(r)) for r in (roots or [])]
        self.entries: dict[str, Artifact] = {}
        self._lock = threading.RLock()
        if self.state_file and self.state_file.exists():
            doc = json.loads(self.state_file.read_text())
            self.roots = sorted(set(self.roots) | set(doc.get("roots", [])))
            self.entries = {e["id"]: Artifact(**e) for e in doc.get("entries", [])}

    def _save(self) -> None:
        if not self.state_file:
            return
        tmp = self.state_file.with_suffix(self.state_file.suffix + ".tmp")
        tmp.write_text(json.dumps({"format": "mfq.model-catalog.v1", "roots": self.roots,
                                   "entries": [asdict(e) for e in self.entries.values()]}, indent=1))
        os.replace(tmp, self.state_file)

    def add_root(self, root: str | Path) -> None:
        with self._lock:
            r = str(Path(root))
            if r not in self.roots:
                self.roots.append(r)
                self._save()

    def scan(self) -> dict:
        """Re-read every root: new artifacts are added, changed ones refreshed, vanished ones dropped (aliases of an id that
        comes back are kept)."""
        with self._lock:
            found: dict[str, Artifact] = {}
            for root in self.roots:
                for art in discover(Path(root)):
                    ident, n = art.id, 2
                    while ident in found and found[ident].path != art.path:  # same file name in two places
                        ident, n = f"{art.id}-{n}", n + 1
                    art.id = ident
                    found[ident] = art
            added = [i for i in found if i not in self.entries]
            removed = [i for i in self.entries if i not in found]
            for ident, art in found.items():
                old = self.entries.get(ident)
                if old is not None:
                    art.aliases, art.added_at = old.aliases, old.added_at
            self.entries = found
            self._save()
            return {"entries": len(found), "added": sorted(added), "removed": sorted(removed)}

    def alias(self, name: str, ident: str) -> None:
        with self._lock:
            if ident not in self.entries:
                raise ArtifactNotFound(ident)
            for e in self.entries.values():
                if name in e.aliases:
                    e.aliases.remove(name)
            self.entries[ident].aliases.append(name)
            self._save()

    def remove(self, ident: str) -> bool:
        """Forget an entry (the files stay; the next scan of its root finds it again)."""
        with self._lock:
            gone = self.entries.pop(ident, None) is not None
            if gone:
                self._save()
            return gone

    def purge(self, ident: str) -> int:
        """Delete the files of an entry and forget it; returns the bytes freed.  Only paths below one of the catalog's
        roots may be deleted (an entry added by hand from elsewhere is refused)."""
        import shutil
        art = self.resolve(ident)
        path = Path(art.path).resolve()
        if not any(path == Path(r).resolve() or Path(r).resolve() in path.parents for r in self.roots):
            raise PermissionError(f"{path} is not below a catalog root")
        freed = art.bytes
        if path.is_dir():
            shutil.rmtree(path)
        else:
            m = _SHARD_RE.match(path.name)
            files = sorted(path.parent.glob(f"{m.group('stem')}-*-of-{m.group('count')}.mfq")) if m else [path]
            for f in files:
                f.unlink(missing_ok=True)
        self.remove(art.id)
        return freed

    def resolve(self, name: str) -> Artifact:
        with self._lock:
            if name in self.entries:
                return self.entries[name]
            for e in self.entries.values():
                if name in e.aliases:
                    return e
        raise ArtifactNotFound(name)

    def listing(self) -> list[dict]:
        with self._lock:
            return [asdict(e) for e in sorted(self.entries.values(), key=lambda e: e.id)]
