"""Old artifacts that stored Hugging Face tensor paths: expose them under canonical names at the loader boundary.

Early ``.mfq`` files kept the source names (``model.layers.3.self_attn.q_proj.weight``); everything after the loader
works on canonical names only (``model.block.3.attention.query.weight``).  :func:`canonical_view` wraps an opened store
in a read-only mapping that answers canonical names and translates one-to-one; stores that already use canonical names
come back unchanged.  Per-expert matrices of such an artifact (``...mlp.experts.7.up_proj.weight``) cannot be aliased
one-to-one -- the runtime wants them stacked -- so they are refused with a message that names the fix (re-run
``mfq quantize`` on the file, which re-packs under canonical names).

Reference: ``mfq/compat/legacy_tensor_names.py`` (an adapter used once, at the container loader's boundary).
"""

from __future__ import annotations

from collections.abc import Mapping

from ..architectures import canonical_name

ASSET_PREFIX = "__mfq_asset__/"


class _View(Mapping):
    def __init__(self, store, alias: dict[str, str]) -> None:
        self._store, self._alias = store, alias  # canonical -> stored name

    def __getitem__(self, name: str):
        return self._store[self._alias.get(name, name)]

    def __iter__(self):
        back = {v: k for k, v in self._alias.items()}
        return (back.get(n, n) for n in self._store)

    def __len__(self) -> int:
        return len(self._store)

    def __contains__(self, name) -> bool:
        return self._alias.get(name, name) in self._store

    def __getattr__(self, name):  # assets(), dtype(), raw(), close() ... of the wrapped store
        return getattr(self._store, name)


def canonical_view(store):
    """``store`` itself when its records carry canonical names, else a translating view."""
    alias: dict[str, str] = {}
    for name in store:
        if name.startswith(ASSET_PREFIX) or not (name.startswith("model.layers.") or name in ("model.embed_tokens.weight", "model.norm.weight", "lm_head.weight")):
            continue
        mapped = canonical_name(name)
        if mapped is None:
            continue
        cname, expert = mapped
        if expert is not None:
            raise ValueError(f"{name}: this artifact stores per-expert matrices under source names; re-pack it with "
                             "`mfq quantize <file> <new file>` to get stacked canonical expert tensors")
        alias[cname] = name
    return _View(store, alias) if alias else store
