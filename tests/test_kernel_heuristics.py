"""Launch-shape rules of the GPU operators (pure Python: which kernel, how many splits)."""

import math

from mfq_b200.ops import kernels as K


def test_decode_attention_splits_fill_one_wave():
    # a batch that fills the GPU by itself is not split; small batches split until one wave (592 CTAs at D <= 128) is full
    assert K.attn_splits_for(64, 8, 4096, 128, rows=4) == 1
    assert K.attn_splits_for(128, 8, 4096, 128, rows=4) == 1
    for batch, heads, ctx, d in ((1, 8, 4096, 128), (8, 8, 4096, 128), (64, 2, 4096, 128), (32, 2, 16384, 128), (64, 2, 4096, 256)):
        s = K.attn_splits_for(batch, heads, ctx, d, rows=4)
        slots = 148 * (4 if d <= 128 else 2)
        assert 1 <= s <= 32 and batch * heads * s <= slots and ctx // s >= 256
        more = s + 1
        assert batch * heads * more > slots or ctx // more < 256 or more > 32  # and it is the largest such count
    # windows wider than 8 (row, head) pairs run the 16-row kernel, which keeps its own rule
    assert K.attn_splits_for(64, 8, 4096, 128, rows=16) == 3
    assert K.attn_splits_for(1, 8, 512, 128, rows=4) == 2


def test_split_k_choice():
    for m in (1, 16, 64):
        for n, k in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096), (1536, 4096), (3584, 4096), (4096, 512)):
            s = K.pick_splits(m, n, k)
            tiles, kb = math.ceil(n / 128), k // 128
            assert 1 <= s <= 8, "decode tiles never leave the cluster path"
            assert s == 1 or math.ceil(kb / s) >= 2
            ctas = tiles * math.ceil(kb / math.ceil(kb / s))
            assert s == 1 or not 128 < ctas <= 148 or (tiles, kb) in K._MEASURED_SPLITS, (m, n, k, s, ctas)
    assert K.pick_splits(64, 28672, 4096) == 1 and K.pick_splits(64, 128256, 4096) == 1  # enough tiles already
    assert K.pick_splits(64, 6144, 4096) == 4  # measured override of the wave model's 3
    assert K.pick_splits(64, 1536, 4096) == 8  # 11 would leave the cluster path
    assert K.pick_splits(4096, 4096, 4096) == 1


def test_kernel_choice_by_rows():
    assert K.use_gemv(1, 28672, 4096) and K.use_gemv(8, 128256, 4096)
    assert K.use_gemv(16, 4096, 4096) and not K.use_gemv(16, 28672, 4096) and not K.use_gemv(12, 4096, 14336)
    assert K.use_gemv(64, 768, 4096) and not K.use_gemv(64, 3072, 4096)
    assert not K.use_gemv(4, 100, 4096)  # rows of 16 only
    assert K.act_gemv_ok(4, 4096, 4096) and not K.act_gemv_ok(5, 4096, 4096) and not K.act_gemv_ok(1, 4096, 32768)
    assert not K.act_gemv_pays(1, 4096, 4096)  # measured slower: off unless asked for
