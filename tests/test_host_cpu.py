"""CPU-only checks: the C-ABI library loads and exports every declared symbol, ctypes structures
match the header's layout, and the host-side argument validation raises the reference's error types
before any kernel is reached."""
import ctypes as C
import os
import re
import subprocess

import pytest
import torch

from conftest import ROOT


def _native():
    from jetlm.kernels import _native
    return _native


def test_library_exports_every_declared_symbol():
    n = _native()
    lib = n.lib()
    header = open(os.path.join(ROOT, "include", "jetlong_b200.h")).read()
    declared = set(re.findall(r"\b(jl_[a-z0-9_]+)\s*\(", header))
    bound = {name for name, _, _ in n.EXPORTS}
    assert declared == bound, (declared ^ bound)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.jl_version() >= 100
    assert lib.jl_status_string(0) == b"ok"
    assert b"workspace" in lib.jl_status_string(n.JL_ERR_WORKSPACE)


def test_struct_layout_matches_header(tmp_path):
    """sizeof of every argument structure of the header == its ctypes mirror (a stub that is one field short
    makes the library read past the caller's struct)."""
    n = _native()
    pairs = [("jl_posmap", n.PosMap), ("jl_prefill_args", n.PrefillArgs), ("jl_kv_segment", n.KvSegment),
             ("jl_decode_args", n.DecodeArgs), ("jl_merge_args", n.MergeArgs), ("jl_rotate_args", n.RotateArgs),
             ("jl_norm_rope_args", n.NormRopeArgs), ("jl_rmsnorm_args", n.RmsNormArgs), ("jl_silu_mul_args", n.SiluMulArgs),
             ("jl_step_advance_args", n.StepAdvanceArgs), ("jl_decode_append_args", n.DecodeAppendArgs),
             ("jl_peer_merge_args", n.PeerMergeArgs)]
    header = open(os.path.join(ROOT, "include", "jetlong_b200.h")).read()
    declared = set(re.findall(r"}\s*(jl_[a-z0-9_]+)\s*;", header))
    assert declared == {name for name, _ in pairs}, declared ^ {name for name, _ in pairs}
    src = tmp_path / "sz.c"
    body = "".join(f'printf("%zu\\n", sizeof({name}));' for name, _ in pairs)
    src.write_text('#include <stdio.h>\n#include "jetlong_b200.h"\nint main(){' + body + "return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)])
    sizes = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    assert sizes == [C.sizeof(t) for _, t in pairs], list(zip([p[0] for p in pairs], sizes, [C.sizeof(t) for _, t in pairs]))
    # and the last fields sit where the header puts them (a missing trailing field shows up here)
    assert n.PrefillArgs.q_pos0_batch_step.offset + 8 == C.sizeof(n.PrefillArgs)
    assert n.PeerMergeArgs.status.offset + 8 == C.sizeof(n.PeerMergeArgs)


def test_host_only_entry_points():
    lib = _native().lib()
    assert lib.jl_decode_workspace_bytes(1, 32, 128, 4) == 16384 + 1 * 32 * 4 * 129 * 4      # arrival counters + partials
    assert lib.jl_decode_workspace_bytes(0, 32, 128, 4) == 0
    s = lib.jl_decode_auto_splits(1, 8, 131072)
    assert 1 <= s and s * 8 <= 296
    assert lib.jl_decode_auto_splits(1, 8, 10) == 1
    assert lib.jl_decode_auto_splits(8, 8, 131072) == 4


def test_null_args_are_rejected_without_a_gpu():
    n = _native()
    lib = n.lib()
    assert lib.jl_merge(None, None) == n.JL_ERR_BAD_ARG
    assert lib.jl_decode(None, None) == n.JL_ERR_BAD_ARG
    assert lib.jl_rotate(None, None) == n.JL_ERR_BAD_ARG
    assert lib.jl_prefill(None, None) == n.JL_ERR_BAD_ARG
    assert b"NULL" in lib.jl_last_error()
    a = n.PrefillArgs()
    a.head_dim = 64
    assert lib.jl_prefill(C.byref(a), None) == n.JL_ERR_UNSUPPORTED
    # stripe batching: the argument checks come before anything touches a device
    a = n.PrefillArgs()
    a.head_dim, a.batch, a.heads, a.kv_heads, a.seqlen_q, a.seqlen_k = 128, 3, 4, 2, 256, 256
    a.map.kind, a.map.n_classes, a.map.near_span = n.JL_MAP_BAND, 2, 10
    a.q_batch_wrap, a.q_batch_first = 2, 0                  # more stripes asked for than the tensors hold
    assert lib.jl_prefill(C.byref(a), None) == n.JL_ERR_BAD_ARG
    assert b"stripe batching" in lib.jl_last_error()
    a.batch, a.q_batch_first = 2, 2                         # first stripe out of range
    assert lib.jl_prefill(C.byref(a), None) == n.JL_ERR_BAD_ARG
    a.q_batch_first, a.impl = 1, 1                          # the cross-check kernel has no stripe batching
    assert lib.jl_prefill(C.byref(a), None) == n.JL_ERR_UNSUPPORTED


def test_backend_guards_match_reference_behaviour():
    from jetlm.kernels import cute_jetlong_backend as be
    x = torch.zeros(1, 2, 4, 128, dtype=torch.bfloat16)
    kw = dict(seqstart_q=0, window_size_left=2, softmax_scale=1.0)
    with pytest.raises(RuntimeError, match="inference-only"):
        be.fused_jetlong_prefill(x, x, x, x, x, has_any_pad=False, training=True, **kw)
    with pytest.raises(RuntimeError, match="left-padded prefill"):
        be.fused_jetlong_prefill(x, x, x, x, x, has_any_pad=True, training=False, **kw)
    inv = torch.ones(64)
    with pytest.raises(RuntimeError, match="inference-only"):
        be.fused_jetlong_decode(x, x, x, x, x, x, inv_freq=inv, group_size=2, has_any_pad=False, training=True)
    with pytest.raises(RuntimeError, match="left-padded decode"):
        be.fused_jetlong_decode(x, x, x, x, x, x, inv_freq=inv, group_size=2, has_any_pad=True, training=False)
    with pytest.raises(RuntimeError, match="non-empty distant decode region"):
        be.fused_jetlong_decode(x, x, x, x, x[:, :0], x[:, :0], inv_freq=inv, group_size=2, has_any_pad=False, training=False)


def test_ops_reject_cpu_tensors_and_bad_metadata():
    from jetlm.kernels import jetlong_ops as ops
    x = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16)
    ss = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(ValueError, match="unsupported metadata arguments.*seqused_q"):
        ops.jetlong_prefill(x, x, x, x, x, seqstart_q=ss, window_size_left=1, seqused_q=ss)
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        ops.jetlong_prefill(x, x, x, x, x, seqstart_q=ss, window_size_left=1)
    with pytest.raises(ValueError, match="requires CUDA tensors"):
        ops.merge_partials([x, x], [torch.zeros(1, 2, 4), torch.zeros(1, 2, 4)])
    with pytest.raises(ValueError, match="CUDA Q/K/V"):
        ops.jetlong_decode(x[:, :1], x[:, :1], x, x, x, x, seqused_near=ss, seqused_distant=ss,
                           inv_freq=torch.ones(64), group_size=2)


def test_position_map_constructors():
    from jetlm.kernels import jetlong_ops as ops
    n = _native()
    m = ops.PositionMap.jetlong(2048)
    assert (m.kind, m.n_classes, m.near_span) == (n.JL_MAP_BAND, 2, 2048)
    m = ops.PositionMap.selfext(1024)
    assert (m.kind, m.n_classes, m.near_span) == (n.JL_MAP_BAND, 2, 1023)
    m = ops.PositionMap.dca(20480)
    assert (m.kind, m.n_classes, m.chunk) == (n.JL_MAP_CHUNK, 3, 20480)
