"""GPU: the allocation-free attention entry point (scratch in a fixed array inside the
library) against the allocating one. Collected last on purpose: a run that stops at the first
failure has then already run every other test.

Some hosts cannot let a library allocate: all free device memory already belongs to their own
pool, or their token loop must not hit the device-wide stall of cudaMalloc / cudaFree. They
call mlb_op_attn_decode_static with buffers they own. Two calls in a row are checked because
the array keeps the previous call's contents (arrival counters, partial sums)."""
import numpy as np
import pytest

from test_gpu_ops import call_attention, make_attention_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api(built_lib):
    from mini_llm_cuda_b200 import api as _api
    return _api


def test_static_scratch_attention_matches_allocating_entry_point_twice(api):
    import torch
    shapes = [
        # batch, heads, kv_heads, hd, splits, dtype, contexts
        (4, 8, 2, 64, 6, torch.bfloat16, [300, 1, 33, 128]),
        (3, 4, 4, 128, 4, torch.float32, [17, 90, 64]),      # second call: other shape, same array
    ]
    for i, (B, H, Hkv, hd, S, dt, ctx) in enumerate(shapes):
        case = make_attention_case(torch, B, H, Hkv, hd, ctx, dt, 10 + i, with_gate=True)
        rc_a, want = call_attention(api, torch, "mlb_op_attn_decode", case, B, H, Hkv, hd, S, dt)
        rc_s, got = call_attention(api, torch, "mlb_op_attn_decode_static", case, B, H, Hkv, hd, S, dt)
        assert rc_a == 0 and rc_s == 0, api.lib().mlb_last_error()
        assert torch.isfinite(got).all()
        # same kernel, same inputs: equal to the tolerance the operator test uses
        assert (got.double() - want.double()).abs().max().item() < 2e-5
        assert (got.cpu().double() - case["want"]).abs().max().item() < 2e-5
        assert api.lib().mlb_op_attn_decode_static_status(None) == 0
    # the call allocates nothing: free device memory is the same before and after it (the first call above
    # placed the library's array)
    out = torch.empty(B, H * hd, device="cuda:0")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    rc_s = api.lib().mlb_op_attn_decode_static(
        case["kpool"].data_ptr(), case["vpool"].data_ptr(), api.DT_BF16 if dt == torch.bfloat16 else api.DT_F32,
        case["table"].data_ptr(), case["pt_stride"], case["n_pages"], case["pos"].data_ptr(), case["q"].data_ptr(),
        case["gate"].data_ptr(), out.data_ptr(), B, H, Hkv, hd, S, None)
    torch.cuda.synchronize()
    assert rc_s == 0 and torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(out, got)
    # same shape again right away: stale partials / counters from the call before must not leak
    rc_s, again = call_attention(api, torch, "mlb_op_attn_decode_static", case, B, H, Hkv, hd, S, dt)
    assert rc_s == 0 and torch.equal(again, got)


def test_static_scratch_attention_refuses_oversized_shapes(api):
    import torch
    cap = api.lib().mlb_op_attn_decode_static_capacity()
    assert cap == 4 << 20
    B, H, Hkv, hd, S = 64, 16, 4, 128, 8                      # 64*16*8*130*4 bytes > 4 MiB
    case = make_attention_case(torch, B, H, Hkv, hd, [20] * B, torch.bfloat16, 2, with_gate=False)
    rc, _ = call_attention(api, torch, "mlb_op_attn_decode_static", case, B, H, Hkv, hd, S, torch.bfloat16)
    assert rc == api.MLB_E_UNSUPPORTED
    assert b"built-in array" in api.lib().mlb_last_error()
    rc, out = call_attention(api, torch, "mlb_op_attn_decode_static", case, B, H, Hkv, hd, 2, torch.bfloat16)
    assert rc == 0
    assert (out.cpu().double() - case["want"]).abs().max().item() < 2e-5
