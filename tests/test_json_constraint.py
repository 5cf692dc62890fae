"""JSON token constraint (native): the automaton against Python's json module, and the vocabulary mask."""

import json
import random

import numpy as np

from mfq_b200 import native


def _vocab():
    # single bytes + some multi-byte tokens as a BPE vocabulary would have them
    toks = [bytes([b]) for b in range(256)]
    toks += [b'{"', b'":', b'", "', b'"}', b"true", b"false", b"null", b"tru", b"123", b"-0.5e+3", b"],[", b"  ", b"\n\n\n",
             b'{"a": 1}', b"}}", b"{]", b'"\\u00', b"e9", b"", b"\xc3\xa9"]
    return native.JsonVocabulary(toks), toks


def test_accepts_valid_documents_and_refuses_invalid_prefixes():
    v, _ = _vocab()
    good = ['{"a": [1, 2.5e-3, true, null, {"b": "x\\n\\u00e9 é"}], "c": {}}', "[]", '"s"', "0", "-12.50", "[[], [[]]]", '{"k":"v"}\n']
    for doc in good:
        s = native.JsonState(v)
        assert s.feed(doc.encode()) and s.complete, doc
        json.loads(doc)
    bad = ['{"a" 1}', "[1,]", "{,}", "01", "1.e3", '{"a":}', "tru e", '"\n"', "[1 2]", '{"a":1,}', "nul!", "+1", "]"]
    for doc in bad:
        s = native.JsonState(v)
        assert not s.feed(doc.encode()), doc
    s = native.JsonState(v)
    assert s.feed(b'{"a": [1, 2') and not s.complete
    assert not s.feed(b"}") and s.feed(b"]}") and s.complete  # a refused chunk leaves the state where it was
    assert not s.feed(b"x")
    obj = native.JsonState(v, need_object=True)
    assert not obj.feed(b"[1]") and not obj.feed(b"3") and obj.feed(b' {"x": 3}') and obj.complete
    ws = native.JsonState(v)
    assert ws.feed(b"[" + b" " * 8) and not ws.feed(b" ")  # whitespace runs are bounded


def test_mask_matches_brute_force_over_the_vocabulary():
    v, toks = _vocab()
    prefixes = [b"", b"{", b'{"ke', b'{"k":', b'{"k": 1', b"[1, ", b"[tr", b'{"a": "x\\', b'"\\u0', b"[1.5", b'{"a": 1}', b"12"]
    for prefix in prefixes:
        s = native.JsonState(v)
        assert s.feed(prefix), prefix
        got = s.mask()
        for t, b in enumerate(toks):
            probe = native.JsonState(v)
            probe.feed(prefix)
            want = bool(b) and probe.feed(b)
            assert got[t] == want, (prefix, b)
    s = native.JsonState(v)
    s.feed(b'{"a": 1}')
    m = s.mask()
    assert s.complete and m[ord("\n")] and not m[ord("}")] and not m[toks.index(b"true")]
    assert v.nodes > 256


def test_random_walk_through_the_mask_always_yields_valid_json():
    v, toks = _vocab()
    rng = random.Random(5)
    for trial in range(20):
        s = native.JsonState(v, need_object=True)
        text = b""
        for _ in range(400):
            if s.complete and (rng.random() < 0.3 or len(text) > 300):
                break
            allowed = np.flatnonzero(s.mask())
            if not len(allowed):  # only the end of the sequence may follow
                assert s.complete
                break
            # steer towards closing once the text is long: prefer structural closers when they are allowed
            closers = [t for t in allowed if toks[t] in (b"}", b"]", b'"', b'"}', b"}}")]
            pick = rng.choice(closers) if closers and len(text) > 120 and rng.random() < 0.7 else int(rng.choice(list(allowed)))
            assert s.feed_token(int(pick))
            text += toks[int(pick)]
        if s.complete:
            assert isinstance(json.loads(text.decode("utf-8", errors="replace")), dict)
