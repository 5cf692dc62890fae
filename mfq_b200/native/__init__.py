"""Python face of the host runtime library (C++): container reader, packed-row decoders, prefix cache, planners.

The library is built in-tree by :mod:`mfq_b200.native.build` (``g++``; no CUDA needed) on first use.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build as _build

_vp, _i, _i64, _d, _cp = C.c_void_p, C.c_int, C.c_int64, C.c_double, C.c_char_p
_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(str(_build.build()))
        sig = {
            "mfq_last_error": ([], _cp),
            "mfq_store_open": ([_cp], _vp), "mfq_store_close": ([_vp], None), "mfq_store_version": ([_vp], _i),
            "mfq_store_arch": ([_vp], _cp), "mfq_store_extra_count": ([_vp], _i), "mfq_store_extra_key": ([_vp, _i], _cp),
            "mfq_store_extra_json": ([_vp, _i], _cp), "mfq_store_tensor_count": ([_vp], _i64),
            "mfq_store_tensor_name": ([_vp, _i64], _cp), "mfq_store_tensor_dtype": ([_vp, _i64], _cp),
            "mfq_store_tensor_nbytes": ([_vp, _i64], _i64), "mfq_store_tensor_file": ([_vp, _i64], _i),
            "mfq_store_find": ([_vp, _cp], _i64), "mfq_store_tensor_data": ([_vp, _i64], _vp),
            "mfq_store_read": ([_vp, _i64, _i64, _i64, _vp, _i, _i], _i),
            "mfq_nint_open": ([_vp, _i64], _vp), "mfq_nint_close": ([_vp], None), "mfq_nint_rows": ([_vp], _i64),
            "mfq_nint_row_len": ([_vp], _i64), "mfq_nint_decode": ([_vp, _i64, _i64, _vp, _i], _i),
            "mfq_nint_row_bits": ([_vp, _i64, _vp, _vp], _i), "mfq_nint_gemv": ([_vp, _i64, _i64, _vp, _vp, _i], _i),
            "mfq_mxfp4_decode": ([_vp, _vp, _i64, _i64, _vp, _i], _i),
            "mfq_fp8_block_decode": ([_vp, _vp, _i64, _i64, _i, _vp, _i], _i), "mfq_f32_to_bf16": ([_vp, _vp, _i64], None),
            "mfq_prefix_open": ([_cp, _i64, _i64, _i], _vp), "mfq_prefix_close": ([_vp], None),
            "mfq_prefix_keys": ([_vp, _vp, _i64, _cp, _vp], _i), "mfq_prefix_put": ([_vp, _vp, _vp, _i64], _i),
            "mfq_prefix_get": ([_vp, _vp, _vp, _i64], _i64), "mfq_prefix_match": ([_vp, _vp, _i], _i),
            "mfq_prefix_pin": ([_vp, _vp, _i], _i), "mfq_prefix_flush": ([_vp], _i), "mfq_prefix_stats": ([_vp, _vp], _i),
            "mfq_tp_plan": ([_i64, _i, _vp, _i64, _vp, _vp], _i),
            "mfq_moe_rank_swaps": ([_vp, _vp, _i, _i, _d, _vp, _vp], _i),
            "mfq_moe_dispatch_plan": ([_vp, _vp, _i, _d, _d, _d, _d, _i, _vp], _i),
            "mfq_json_vocab_open": ([_vp, _vp, _i64], _vp), "mfq_json_vocab_close": ([_vp], None),
            "mfq_json_vocab_nodes": ([_vp], _i64), "mfq_json_state_init": ([_vp, _i], None),
            "mfq_json_state_feed": ([_vp, _vp, _i64], _i), "mfq_json_state_complete": ([_vp], _i),
            "mfq_json_mask": ([_vp, _vp, _vp], _i64),
            "mfq_slotbook_open": ([_i], _vp), "mfq_slotbook_close": ([_vp], None), "mfq_slotbook_lookup": ([_vp, _i64], _i),
            "mfq_slotbook_acquire": ([_vp, _i64, _vp], _i), "mfq_slotbook_pin": ([_vp, _i64, _i], _i),
        }
        for name, (args, res) in sig.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, res
        _lib = L
    return _lib


def _err() -> str:
    return (lib().mfq_last_error() or b"").decode()


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class NativeStore:
    """Memory-mapped ``.mfq`` checkpoint (one file or a shard set) read by the C++ parser."""

    def __init__(self, path) -> None:
        self._h = lib().mfq_store_open(str(path).encode())
        if not self._h:
            raise OSError(_err())
        L = lib()
        self.version, self.arch = L.mfq_store_version(self._h), L.mfq_store_arch(self._h).decode()
        self.extra = {L.mfq_store_extra_key(self._h, i).decode(): L.mfq_store_extra_json(self._h, i).decode()
                      for i in range(L.mfq_store_extra_count(self._h))}
        n = L.mfq_store_tensor_count(self._h)
        self.names = [L.mfq_store_tensor_name(self._h, i).decode() for i in range(n)]

    def close(self) -> None:
        if self._h:
            lib().mfq_store_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self) -> int:
        return len(self.names)

    def find(self, name: str) -> int:
        return lib().mfq_store_find(self._h, name.encode())

    def info(self, i: int) -> tuple[str, str, int, int]:
        L = lib()
        return (self.names[i], L.mfq_store_tensor_dtype(self._h, i).decode(), L.mfq_store_tensor_nbytes(self._h, i),
                L.mfq_store_tensor_file(self._h, i))

    def view(self, i: int) -> np.ndarray:
        """Zero-copy uint8 view of blob ``i`` (valid while the store is open)."""
        n = lib().mfq_store_tensor_nbytes(self._h, i)
        p = lib().mfq_store_tensor_data(self._h, i)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(n,))

    def read_into(self, i: int, dst: np.ndarray, offset: int = 0, threads: int = 8, drop_cache: bool = False) -> None:
        """Parallel copy of ``dst.nbytes`` bytes of blob ``i`` into ``dst`` (e.g. a pinned staging buffer)."""
        if lib().mfq_store_read(self._h, i, offset, dst.nbytes, _np_ptr(dst), threads, int(drop_cache)) != 0:
            raise ValueError(_err())


class NintRows:
    """Row-addressable decoder over a NINT v2 payload (no copy of the payload is made; keep it alive)."""

    def __init__(self, blob: np.ndarray) -> None:
        self._blob = np.ascontiguousarray(blob, dtype=np.uint8)
        self._h = lib().mfq_nint_open(_np_ptr(self._blob), self._blob.nbytes)
        if not self._h:
            raise ValueError(_err())
        self.rows, self.row_len = lib().mfq_nint_rows(self._h), lib().mfq_nint_row_len(self._h)

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals are already cleared at interpreter exit
            lib().mfq_nint_close(self._h)
            self._h = None

    def decode(self, begin: int = 0, end: int | None = None, threads: int = 8) -> np.ndarray:
        end = self.rows if end is None else end
        out = np.empty((end - begin, self.row_len), dtype=np.float32)
        if lib().mfq_nint_decode(self._h, begin, end, _np_ptr(out), threads) != 0:
            raise ValueError(_err())
        return out

    def gemv(self, x: np.ndarray, begin: int = 0, end: int | None = None, threads: int = 8) -> np.ndarray:
        end = self.rows if end is None else end
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(end - begin, dtype=np.float32)
        if lib().mfq_nint_gemv(self._h, begin, end, _np_ptr(x), _np_ptr(y), threads) != 0:
            raise ValueError(_err())
        return y

    def row_bits(self, row: int) -> tuple[int, int]:
        q, k = C.c_int(), C.c_int()
        if lib().mfq_nint_row_bits(self._h, row, C.byref(q), C.byref(k)) != 0:
            raise ValueError(_err())
        return q.value, k.value


def nvq_decode(t, threads: int = 8) -> np.ndarray:
    """Rows of a plain (non-JSC) :class:`~mfq_b200.formats.nvq.NvqTensor` as float32 ``[out, neuron_len]``."""
    from ..formats.nvq import codebook as lattice
    table = np.ascontiguousarray(lattice(t.spec) if t.codebook is None else t.codebook, dtype=np.float32)
    rows, n = int(t.neuron_scale.size), int(t.neuron_len)
    idx = np.ascontiguousarray(t.indices, dtype=np.uint16)
    sg, sub = np.ascontiguousarray(t.signs, dtype=np.uint8), np.ascontiguousarray(t.sub_scale, dtype=np.uint8)
    anchors = np.ascontiguousarray(t.neuron_scale, dtype=np.float32)
    out = np.empty((rows, n), dtype=np.float32)
    fn = lib().mfq_nvq_decode
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
    fn.restype = C.c_int
    rc = fn(_np_ptr(idx), _np_ptr(sg), _np_ptr(sub), _np_ptr(anchors), _np_ptr(table), rows, n, t.spec.groupsize,
            t.spec.vector_size, table.shape[0], int(t.spec.sign_mode == "index_parity"), _np_ptr(out), threads)
    if rc != 0:
        raise ValueError(_err())
    return out


def mxfp4_decode(codes: np.ndarray, scales: np.ndarray, rows: int, cols: int, threads: int = 8) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.float32)
    codes, scales = np.ascontiguousarray(codes, np.uint8), np.ascontiguousarray(scales, np.uint8)
    if lib().mfq_mxfp4_decode(_np_ptr(codes), _np_ptr(scales), rows, cols, _np_ptr(out), threads) != 0:
        raise ValueError(_err())
    return out


def fp8_block_decode(codes: np.ndarray, scales: np.ndarray, block: int = 128, threads: int = 8) -> np.ndarray:
    rows, cols = codes.shape
    out = np.empty((rows, cols), dtype=np.float32)
    codes, scales = np.ascontiguousarray(codes, np.uint8), np.ascontiguousarray(scales, np.float32)
    if lib().mfq_fp8_block_decode(_np_ptr(codes), _np_ptr(scales), rows, cols, block, _np_ptr(out), threads) != 0:
        raise ValueError(_err())
    return out


class PrefixCache:
    """Content-addressed KV block store: SHA-256 chained keys, RAM tier + optional file tier (write-behind)."""

    def __init__(self, directory: str | Path | None = None, ram_budget: int = 1 << 30, disk_budget: int = 0,
                 block_tokens: int = 256) -> None:
        self.block_tokens = block_tokens
        self._h = lib().mfq_prefix_open(str(directory).encode() if directory else None, ram_budget, disk_budget, block_tokens)
        if not self._h:
            raise ValueError(_err())

    def close(self) -> None:
        if self._h:
            lib().mfq_prefix_close(self._h)
            self._h = None

    def keys(self, tokens, salt: str = "") -> np.ndarray:
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty((len(t) // self.block_tokens, 32), dtype=np.uint8)
        lib().mfq_prefix_keys(self._h, _np_ptr(t), len(t), salt.encode(), _np_ptr(out))
        return out

    def put(self, key: np.ndarray, data: np.ndarray) -> None:
        data = np.ascontiguousarray(data)
        lib().mfq_prefix_put(self._h, _np_ptr(np.ascontiguousarray(key)), _np_ptr(data), data.nbytes)

    def get(self, key: np.ndarray, nbytes: int) -> np.ndarray | None:
        dst = np.empty(nbytes, dtype=np.uint8)
        n = lib().mfq_prefix_get(self._h, _np_ptr(np.ascontiguousarray(key)), _np_ptr(dst), nbytes)
        if n == -2:
            raise ValueError(_err())
        return None if n < 0 else dst[:n]

    def match(self, keys: np.ndarray) -> int:
        """Number of leading blocks of ``keys`` that are cached (RAM or file tier)."""
        keys = np.ascontiguousarray(keys, dtype=np.uint8)
        return lib().mfq_prefix_match(self._h, _np_ptr(keys), len(keys))

    def pin(self, key: np.ndarray, delta: int = 1) -> None:
        if lib().mfq_prefix_pin(self._h, _np_ptr(np.ascontiguousarray(key)), delta) < 0:
            raise KeyError(_err())

    def flush(self) -> None:
        lib().mfq_prefix_flush(self._h)

    def stats(self) -> dict:
        v = np.zeros(8, dtype=np.int64)
        lib().mfq_prefix_stats(self._h, _np_ptr(v))
        return dict(zip(("ram_bytes", "disk_bytes", "ram_entries", "disk_entries", "hits_ram", "hits_disk", "misses",
                         "evictions"), (int(x) for x in v)))


def tp_plan(total: int, ranks: int, weights=None, granularity: int = 1) -> list[tuple[int, int]]:
    """Contiguous ``[begin, end)`` slices of ``total`` units, proportional to ``weights``, aligned to ``granularity``."""
    b, e = np.zeros(ranks, dtype=np.int64), np.zeros(ranks, dtype=np.int64)
    w = None if weights is None else np.ascontiguousarray(weights, dtype=np.float64)
    if lib().mfq_tp_plan(total, ranks, None if w is None else _np_ptr(w), granularity, _np_ptr(b), _np_ptr(e)) != 0:
        raise ValueError(_err())
    return [(int(x), int(y)) for x, y in zip(b, e)]


def moe_rank_swaps(heat, resident, max_swaps: int, hysteresis: float = 0.1) -> list[tuple[int, int]]:
    """(evict, load) pairs that replace the coldest resident experts with hotter absent ones."""
    heat = np.ascontiguousarray(heat, dtype=np.float64)
    res = np.ascontiguousarray(resident, dtype=np.uint8)
    ev, ld = np.zeros(max(1, max_swaps), dtype=np.int32), np.zeros(max(1, max_swaps), dtype=np.int32)
    n = lib().mfq_moe_rank_swaps(_np_ptr(heat), _np_ptr(res), len(heat), max_swaps, hysteresis, _np_ptr(ev), _np_ptr(ld))
    if n < 0:
        raise ValueError(_err())
    return [(int(ev[i]), int(ld[i])) for i in range(n)]


TIER_INACTIVE, TIER_GPU_RESIDENT, TIER_GPU_TRANSFER, TIER_CPU = 0, 1, 2, 3


def moe_dispatch_plan(tokens_per_expert, resident, *, bytes_per_expert: float, h2d_gbs: float = 50.0, gpu_tok_us: float = 0.05,
                      cpu_tok_us: float = 20.0, cpu_available: bool = True) -> np.ndarray:
    tok = np.ascontiguousarray(tokens_per_expert, dtype=np.int32)
    res = np.ascontiguousarray(resident, dtype=np.uint8)
    out = np.zeros(len(tok), dtype=np.int32)
    if lib().mfq_moe_dispatch_plan(_np_ptr(tok), _np_ptr(res), len(tok), bytes_per_expert, h2d_gbs, gpu_tok_us, cpu_tok_us,
                                   int(cpu_available), _np_ptr(out)) != 0:
        raise ValueError(_err())
    return out


class SlotBook:
    """Fixed number of cache slots with LRU replacement and pinning (expert / block residency bookkeeping)."""

    def __init__(self, slots: int) -> None:
        self._h = lib().mfq_slotbook_open(slots)
        if not self._h:
            raise ValueError(_err())

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals are already cleared at interpreter exit
            lib().mfq_slotbook_close(self._h)
            self._h = None

    def lookup(self, key: int) -> int:
        return lib().mfq_slotbook_lookup(self._h, key)

    def acquire(self, key: int) -> tuple[int, int | None]:
        ev = C.c_int64(-1)
        slot = lib().mfq_slotbook_acquire(self._h, key, C.byref(ev))
        if slot < 0:
            raise MemoryError(_err())
        return slot, (None if ev.value < 0 else ev.value)

    def pin(self, key: int, delta: int = 1) -> int:
        n = lib().mfq_slotbook_pin(self._h, key, delta)
        if n < 0:
            raise KeyError(_err())
        return n


class JsonVocabulary:
    """Byte trie of a tokenizer's vocabulary for JSON-constrained decoding (``token_bytes[i]``: the bytes token ``i``
    adds to the text; empty for special tokens, which then never match)."""

    def __init__(self, token_bytes: list[bytes]) -> None:
        self.size = len(token_bytes)
        offsets = np.zeros(self.size + 1, dtype=np.int64)
        np.cumsum([len(b) for b in token_bytes], out=offsets[1:])
        blob = np.frombuffer(b"".join(token_bytes) or b"\0", dtype=np.uint8)
        self._h = lib().mfq_json_vocab_open(_np_ptr(blob), _np_ptr(offsets), self.size)
        if not self._h:
            raise ValueError(_err())
        self.token_bytes = token_bytes

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals are already cleared at interpreter exit
            lib().mfq_json_vocab_close(self._h)
            self._h = None

    @property
    def nodes(self) -> int:
        return int(lib().mfq_json_vocab_nodes(self._h))


class JsonState:
    """Position of a partly generated JSON document in the grammar."""

    def __init__(self, vocab: JsonVocabulary, need_object: bool = False) -> None:
        self.vocab = vocab
        self._s = np.zeros(16, dtype=np.uint8)
        lib().mfq_json_state_init(_np_ptr(self._s), int(need_object))

    def feed(self, data: bytes) -> bool:
        """Consume bytes; False (state unchanged) if the grammar refuses them."""
        if not data:
            return True
        buf = np.frombuffer(data, dtype=np.uint8)
        return lib().mfq_json_state_feed(_np_ptr(self._s), _np_ptr(buf), len(data)) == 0

    def feed_token(self, token: int) -> bool:
        return self.feed(self.vocab.token_bytes[token])

    @property
    def complete(self) -> bool:
        return bool(lib().mfq_json_state_complete(_np_ptr(self._s)))

    def mask(self) -> np.ndarray:
        """bool ``[vocab]``: tokens that keep the text a prefix of a valid document."""
        key = self.key
        cache = self.vocab.__dict__.setdefault("_mask_cache", {})
        hit = cache.get(key)
        if hit is not None:
            return hit.copy()
        words = np.zeros((self.vocab.size + 31) // 32, dtype=np.uint32)
        if lib().mfq_json_mask(self.vocab._h, _np_ptr(self._s), _np_ptr(words)) < 0:
            raise ValueError(_err())
        mask = np.unpackbits(words.view(np.uint8), bitorder="little")[: self.vocab.size].astype(bool)
        if len(cache) >= 256:  # the mask is a function of the 16 state bytes alone; text inside a string keeps one state
            cache.pop(next(iter(cache)))
        cache[key] = mask
        return mask.copy()

    @property
    def key(self) -> bytes:
        """The grammar position as bytes: equal keys have equal masks."""
        return self._s.tobytes()
