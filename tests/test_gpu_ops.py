"""GPU: kernel-level parity of the stand-alone operator entry points (device pointers)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api(built_lib):
    from mini_llm_cuda_b200 import api as _api
    return _api


def make_attention_case(torch, batch, heads, kv_heads, hd, ctx_list, dtype, seed, with_gate):
    """Random paged KV cache with shuffled page assignment; returns device tensors + fp64 answer."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    block = 16
    pages_per_seq = [(c + block - 1) // block for c in ctx_list]
    pt_stride = max(pages_per_seq) + 1
    n_pages = sum(pages_per_seq) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(batch, pt_stride, dtype=torch.int32)
    it = iter(perm)
    for b in range(batch):
        for p in range(pages_per_seq[b]):
            table[b, p] = next(it)
    kpool = torch.randn(n_pages, kv_heads, block, hd, generator=g).to(dtype)
    vpool = torch.randn(n_pages, kv_heads, block, hd, generator=g).to(dtype)
    q = torch.randn(batch, heads * hd, generator=g)
    gate = torch.rand(batch, heads * hd, generator=g) if with_gate else None
    want = torch.zeros(batch, heads * hd, dtype=torch.float64)
    group = heads // kv_heads
    for b in range(batch):
        ctx = ctx_list[b]
        idx = table[b, :pages_per_seq[b]].long()
        K = kpool[idx].double().permute(1, 0, 2, 3).reshape(kv_heads, -1, hd)[:, :ctx]
        V = vpool[idx].double().permute(1, 0, 2, 3).reshape(kv_heads, -1, hd)[:, :ctx]
        for h in range(heads):
            qh = q[b, h * hd:(h + 1) * hd].double()
            s = (K[h // group] @ qh) / np.sqrt(hd)
            p = torch.softmax(s, dim=0)
            want[b, h * hd:(h + 1) * hd] = p @ V[h // group]
        if with_gate:
            want[b] *= gate[b].double()
    dev = "cuda:0"
    pos = torch.tensor([c - 1 for c in ctx_list], dtype=torch.int32)
    return dict(kpool=kpool.to(dev), vpool=vpool.to(dev), table=table.to(dev), pos=pos.to(dev), q=q.to(dev),
                gate=gate.to(dev) if with_gate else None, want=want, pt_stride=pt_stride, n_pages=n_pages)


def call_attention(api, torch, fn_name, case, batch, heads, kv_heads, hd, splits, dtype):
    out = torch.full((batch, heads * hd), float("nan"), device="cuda:0")
    kv_dt = api.DT_BF16 if dtype == torch.bfloat16 else api.DT_F32
    fn = getattr(api.lib(), fn_name)
    rc = fn(case["kpool"].data_ptr(), case["vpool"].data_ptr(), kv_dt, case["table"].data_ptr(), case["pt_stride"],
            case["n_pages"], case["pos"].data_ptr(), case["q"].data_ptr(), case["gate"].data_ptr() if case["gate"] is not None else None,
            out.data_ptr(), batch, heads, kv_heads, hd, splits, None)
    torch.cuda.synchronize()
    return rc, out


@pytest.mark.parametrize("heads,kv_heads,hd,dtype_name,splits,with_gate", [
    (4, 4, 64, "float32", 1, False),
    (4, 4, 64, "bfloat16", 5, True),
    (8, 2, 128, "bfloat16", 8, True),
    (8, 1, 64, "float32", 3, False),
    (4, 2, 128, "float32", 16, True),
])
def test_attention_op_matches_fp64(api, heads, kv_heads, hd, dtype_name, splits, with_gate):
    import torch
    dtype = getattr(torch, dtype_name)
    ctx_list = [1, 16, 17, 250, 77]          # one position, page edges, more splits than pages
    case = make_attention_case(torch, 5, heads, kv_heads, hd, ctx_list, dtype, 3, with_gate)
    rc, out = call_attention(api, torch, "mlb_op_attn_decode", case, 5, heads, kv_heads, hd, splits, dtype)
    assert rc == 0, api.lib().mlb_last_error()
    err = (out.cpu().double() - case["want"]).abs().max().item()
    assert err < 2e-5, err


def test_attention_op_rejects_bad_arguments(api):
    import torch
    case = make_attention_case(torch, 1, 4, 4, 64, [5], torch.float32, 1, False)
    L = api.lib()
    args = lambda **kw: None
    out = torch.zeros(1, 256, device="cuda:0")
    base = [case["kpool"].data_ptr(), case["vpool"].data_ptr(), api.DT_F32, case["table"].data_ptr(), case["pt_stride"],
            case["n_pages"], case["pos"].data_ptr(), case["q"].data_ptr(), None, out.data_ptr(), 1, 4, 4, 64, 4, None]
    bad = list(base); bad[13] = 96
    assert L.mlb_op_attn_decode(*bad) == api.MLB_E_UNSUPPORTED
    bad = list(base); bad[12] = 3
    assert L.mlb_op_attn_decode(*bad) == api.MLB_E_INVALID
    bad = list(base); bad[7] = None
    assert L.mlb_op_attn_decode(*bad) == api.MLB_E_INVALID
    bad = list(base); bad[2] = api.DT_FP8
    assert L.mlb_op_attn_decode(*bad) == api.MLB_E_INVALID
    bad = list(base); bad[4] = 0
    assert L.mlb_op_attn_decode(*bad) == api.MLB_E_INVALID
    assert L.mlb_op_attn_decode(*base) == 0


def test_attention_op_skips_what_the_page_table_does_not_cover(api):
    """A caller-owned page table is checked on the device. A position that needs more pages than
    pt_stride: that sequence is skipped (its output row keeps what it held), the others are
    computed. A page id outside the pool: page 0 is read instead. Either way the call returns
    MLB_E_INVALID and nothing outside the caller's buffers is touched."""
    import torch
    L = api.lib()
    B, H, hd = 3, 4, 64
    case = make_attention_case(torch, B, H, H, hd, [40, 20, 33], torch.float32, 7, False)
    # (a) sequence 1 claims a position far beyond its page-table row
    pos = case["pos"].clone()
    pos[1] = 16 * case["pt_stride"] + 5
    out = torch.full((B, H * hd), 123.0, device="cuda:0")
    rc = L.mlb_op_attn_decode(case["kpool"].data_ptr(), case["vpool"].data_ptr(), api.DT_F32, case["table"].data_ptr(),
                              case["pt_stride"], case["n_pages"], pos.data_ptr(), case["q"].data_ptr(), None, out.data_ptr(),
                              B, H, H, hd, 2, None)
    assert rc == api.MLB_E_INVALID and b"more pages than pt_stride" in L.mlb_last_error()
    assert (out[1] == 123.0).all()                                      # skipped, not dereferenced
    for b in (0, 2):
        assert (out[b].cpu().double() - case["want"][b]).abs().max().item() < 2e-5
    # (b) a stale page id in the table
    table = case["table"].clone()
    table[2, 1] = case["n_pages"] + 1000
    rc = L.mlb_op_attn_decode(case["kpool"].data_ptr(), case["vpool"].data_ptr(), api.DT_F32, table.data_ptr(),
                              case["pt_stride"], case["n_pages"], case["pos"].data_ptr(), case["q"].data_ptr(), None,
                              out.data_ptr(), B, H, H, hd, 2, None)
    assert rc == api.MLB_E_INVALID and b"outside [0, num_pages)" in L.mlb_last_error()
    # the allocation-free entry point reports the same through its status call
    rc = L.mlb_op_attn_decode_static(case["kpool"].data_ptr(), case["vpool"].data_ptr(), api.DT_F32, table.data_ptr(),
                                     case["pt_stride"], case["n_pages"], case["pos"].data_ptr(), case["q"].data_ptr(), None,
                                     out.data_ptr(), B, H, H, hd, 2, None)
    assert rc == 0
    assert L.mlb_op_attn_decode_static_status(None) == api.MLB_E_INVALID
    rc = L.mlb_op_attn_decode_static(case["kpool"].data_ptr(), case["vpool"].data_ptr(), api.DT_F32, case["table"].data_ptr(),
                                     case["pt_stride"], case["n_pages"], case["pos"].data_ptr(), case["q"].data_ptr(), None,
                                     out.data_ptr(), B, H, H, hd, 2, None)
    assert rc == 0 and L.mlb_op_attn_decode_static_status(None) == 0
    assert (out.cpu().double() - case["want"]).abs().max().item() < 2e-5


@pytest.mark.parametrize("N,K,batch", [(128, 64, 16), (256, 512, 32), (1408, 512, 256), (512, 1408, 100), (1552, 512, 20),
                                       (8192, 512, 300)])
def test_tcgen05_gemm_matches_fp32_matmul(api, N, K, batch):
    """Plain / residual / gate-up forms of the tensor-core projection against torch.matmul on the
    same bf16 values in fp32 (only the accumulation order differs): ragged N and batch tails,
    several k-blocks, two batch tiles."""
    import torch
    g = torch.Generator(device="cpu").manual_seed(N + K + batch)
    W = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    W2 = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    X = torch.randn(batch, K, generator=g).to(torch.bfloat16).cuda()
    R = torch.randn(batch, N, generator=g).cuda()
    want = X.float() @ W.float().T
    L = api.lib()
    out = torch.full((batch, N), float("nan"), device="cuda")
    assert L.mlb_op_gemm_bf16(W.data_ptr(), None, X.data_ptr(), None, out.data_ptr(), N, K, batch, None) == 0, L.mlb_last_error()
    scale = want.abs().max().item()
    assert (out - want).abs().max().item() < 2e-5 * max(scale, 1.0) + 1e-5
    out2 = R.clone()
    assert L.mlb_op_gemm_bf16(W.data_ptr(), None, X.data_ptr(), out2.data_ptr(), out2.data_ptr(), N, K, batch, None) == 0
    assert (out2 - (want + R)).abs().max().item() < 2e-5 * max(scale, 1.0) + 1e-5
    up = X.float() @ W2.float().T
    h_want = (want / (1.0 + torch.exp(-want))) * up
    h = torch.zeros(batch, N, dtype=torch.bfloat16, device="cuda")
    assert L.mlb_op_gemm_bf16(W.data_ptr(), W2.data_ptr(), X.data_ptr(), None, h.data_ptr(), N, K, batch, None) == 0
    assert (h.float() - h_want).abs().max().item() < 1e-2 * max(h_want.abs().max().item(), 1e-3)


def test_bounded_wait_runs_out_and_context_stays_usable(api):
    """The wait routine of the streaming kernels, on a barrier that nothing completes: the kernel
    ends by itself, the call reports MLB_E_TIMEOUT, and the next operator call on the same
    context works (no trap, no fault, no endless loop)."""
    lib = api.lib()
    rc = lib.mlb_op_wait_probe(0, 20000)
    assert rc == api.MLB_E_TIMEOUT
    assert b"bounded device-side wait ran out" in lib.mlb_last_error()
    assert lib.mlb_op_wait_probe(0, 0) == api.MLB_E_INVALID
    # the context is intact: a tcgen05 GEMM right after it still matches torch
    test_tcgen05_gemm_matches_fp32_matmul(api, 256, 512, 32)
