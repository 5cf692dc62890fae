"""tcgen05 prefill attention against the fp32 reference."""

import math

import pytest
import torch

from mfq_b200 import ops
from mfq_b200.ops import reference as ref
from gpu_common import assert_close, check_status, require_gpu_lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,hq,hk", [(128, 4, 2), (300, 8, 2), (1024, 4, 4), (1, 4, 1), (129, 2, 1)])
def test_prefill_attention_matches_reference(t, hq, hk):
    require_gpu_lib()
    g = torch.Generator(device="cuda").manual_seed(t)
    q = torch.randn((t, hq, 128), generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn((t, hk, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((t, hk, 128), generator=g, device="cuda").to(torch.bfloat16)
    scale = 1 / math.sqrt(128)
    got = ops.kernels.attn_prefill_bf16(q, k, v, scale)
    check_status()
    want = ref.attention(q, k, v, scale, causal_offset=0)
    assert_close(got, want, rel=2e-2, what=f"prefill attention T={t}")


def test_packed_sequences_do_not_mix():
    require_gpu_lib()
    q = torch.randn((200, 4, 128), device="cuda").to(torch.bfloat16)
    k = torch.randn((200, 2, 128), device="cuda").to(torch.bfloat16)
    v = torch.randn((200, 2, 128), device="cuda").to(torch.bfloat16)
    got = ops.attn_prefill(q, k, v, [0, 70, 200], 0.09)
    want = torch.cat([ref.attention(q[:70], k[:70], v[:70], 0.09, 0), ref.attention(q[70:], k[70:], v[70:], 0.09, 0)])
    assert_close(got, want, rel=2e-2)
    check_status()
