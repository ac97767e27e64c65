"""jl_decode_static: the decode entry point for callers that may not allocate device memory
(a server whose memory arena is fixed at start-up, a plug-in that owns no allocator).  Its split-KV
scratch is an array inside the library, so the test drives it through the raw C ABI with
preallocated inputs and outputs only, twice in a row (the second call finds the first call's
leftovers in the scratch), and compares with the regular jl_decode entry point, which gets a
caller-allocated workspace.  Collected last on purpose: a failure here cannot hide another test's."""
import ctypes as C

import pytest
import torch

import jetlong_oracle as orc

pytestmark = pytest.mark.gpu


def _args(n, q_ops, k, v, boundary, out, lse, splits):
    """DecodeArgs for contiguous (B,1,H,D) queries and a contiguous (B,S,Hk,D) cache split at `boundary`."""
    B, _, H, D = q_ops[0].shape
    S, Hk = k.shape[1], k.shape[2]
    a = n.DecodeArgs()
    for c, q in enumerate(q_ops):
        a.q[c] = q.data_ptr()
    a.q_stride_b, a.q_stride_h = H * D, D
    for i, (lo, hi, cls) in enumerate(((0, boundary, 1), (boundary, S, 0))):
        g = a.seg[i]
        g.k = k.data_ptr() + lo * Hk * D * 2
        g.v = v.data_ptr() + lo * Hk * D * 2
        g.k_stride_b = g.v_stride_b = S * Hk * D
        g.k_stride_s = g.v_stride_s = Hk * D
        g.k_stride_h = g.v_stride_h = D
        g.len, g.q_class = hi - lo, cls
    a.n_segments, a.batch, a.heads, a.kv_heads, a.head_dim = 2, B, H, Hk, D
    a.num_splits, a.softmax_scale, a.group_size = splits, D ** -0.5, 1
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.o_stride_b, a.o_stride_h = H * D, D
    return a


def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    from jetlm.kernels import _native as n
    lib = n.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.jl_decode_static_scratch_bytes() == 4 << 20
    for trial, (B, H, Hk, S, boundary, splits) in enumerate(((2, 16, 8, 3000, 2100, 0), (1, 32, 8, 9001, 5000, 7))):
        torch.manual_seed(100 + trial)
        q = [torch.randn(B, 1, H, 128, device="cuda").bfloat16() for _ in range(2)]
        k = torch.randn(B, S, Hk, 128, device="cuda").bfloat16()
        v = torch.randn(B, S, Hk, 128, device="cuda").bfloat16()
        out_ws, out_st = (torch.zeros(B, 1, H, 128, device="cuda", dtype=torch.bfloat16) for _ in range(2))
        lse_ws, lse_st = (torch.zeros(B, H, device="cuda") for _ in range(2))
        ws = torch.zeros(lib.jl_decode_workspace_bytes(B, H, 128, 0), dtype=torch.uint8, device="cuda")   # counters start at zero
        a = _args(n, q, k, v, boundary, out_ws, lse_ws, splits)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        n.check("jl_decode", lib.jl_decode(C.byref(a), stream))
        b = _args(n, q, k, v, boundary, out_st, lse_st, splits)          # no workspace at all
        for call in range(2):
            out_st.zero_(); lse_st.zero_()
            n.check("jl_decode_static", lib.jl_decode_static(C.byref(b), stream))
            torch.cuda.synchronize()
            # same kernels, same split count, same arithmetic: identical results, well inside the 2e-2 / 1e-3 parity bars
            assert float((out_st.float() - out_ws.float()).abs().max()) <= 2e-2, (trial, call)
            assert float((lse_st - lse_ws).abs().max()) <= 1e-3, (trial, call)
            assert torch.equal(out_st, out_ws) and torch.equal(lse_st, lse_ws), (trial, call)
        # and directly against the CPU oracle, at the parity bars of every other kernel test
        eo, el = orc.jetlong_decode(q[0].cpu(), q[1].cpu(), k[:, boundary:].cpu(), v[:, boundary:].cpu(),
                                    k[:, :boundary].cpu(), v[:, :boundary].cpu())
        d, cos = orc.compare(out_st.float().cpu(), eo)
        dl, _ = orc.compare(lse_st.cpu().view(B, H, 1), el)
        assert d <= 2e-2 and cos >= 0.9999 and dl <= 1e-3, (trial, d, cos, dl)


def test_static_scratch_decode_refuses_requests_beyond_its_array():
    from jetlm.kernels import _native as n
    lib = n.lib()
    B, H, Hk, S = 16, 32, 8, 70000
    q = [torch.randn(B, 1, H, 128, device="cuda").bfloat16() for _ in range(2)]
    k = torch.randn(B, S, Hk, 128, device="cuda").bfloat16()
    out = torch.zeros(B, 1, H, 128, device="cuda", dtype=torch.bfloat16)
    lse = torch.zeros(B, H, device="cuda")
    a = _args(n, q, k, k, S // 2, out, lse, 32)       # 16 * 32 * 32 * 129 * 4 bytes = 8.1 MiB > 4 MiB
    rc = lib.jl_decode_static(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == n.JL_ERR_WORKSPACE
    msg = lib.jl_last_error().decode()
    assert "built-in array" in msg and str(4 << 20) in msg
    torch.cuda.synchronize()
    assert torch.all(out == 0)                          # nothing was launched
