"""KV-sequence sharding on CPU ranks (gloo, world size 2 and 3): stripe geometry, the one all-gather
and the N-way merge reproduce attention over the whole key sequence.  The local attention and the
merge are the CPU oracle here; on GPUs the same driver runs the CUDA kernels."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, block, results):
    sys.path[:0] = [PKG, os.path.join(ROOT, "oracle")]
    import jetlong_oracle as orc
    from jetlm.kernels.sequence_parallel import SequenceShard, sharded_attention
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(7)                                   # same tensors on every rank
        B, S, H, Hk, D, w0, ss = 1, 300, 4, 2, 128, 70, 37     # 37 keys were already cached: chunked prefill
        Skv = S + ss
        qb, qg = torch.randn(B, S, H, D), torch.randn(B, S, H, D)
        kb, kg, v = (torch.randn(B, Skv, Hk, D) for _ in range(3))
        shard = SequenceShard(rank, world, block=block)
        rows = shard.owned_rows(Skv)
        assert rows.numel() == shard.n_owned(Skv)
        pos0, blk, stride = shard.geometry()
        j = torch.arange(rows.numel())
        assert torch.equal(rows, pos0 + (j // blk) * stride + j % blk)      # the kernels' key-position map

        def local():                                           # attention of all queries over this rank's keys only
            near, far = orc.bifocal_masks(S, Skv, ss, w0)
            on, ln = orc.attention(qb, kb[:, rows], v[:, rows], near[:, :, rows])
            of, lf = orc.attention(qg, kg[:, rows], v[:, rows], far[:, :, rows])
            return orc.merge2(on, ln, of, lf)

        merge = lambda outs, lses: orc.merge_partials(torch.stack(outs), torch.stack(lses))
        out, lse = sharded_attention(local, merge, shard)
        eo, el = orc.jetlong_prefill(qb, qg, kb, kg, v, seqstart=ss, w0=w0)
        d, cos = orc.compare(out, eo)
        dl, _ = orc.compare(lse, el)
        # decode: contiguous ranges
        lo, hi = shard.contiguous_range(Skv)
        boundary = Skv - 1 - w0
        q1, q1g = qb[:, -1:], qg[:, -1:]

        def local_dec():
            kn, vn = kb[:, max(lo, boundary):hi], v[:, max(lo, boundary):hi]
            kf, vf = kg[:, lo:min(hi, boundary)], v[:, lo:min(hi, boundary)]
            on, ln = orc.attention(q1, kn, vn) if kn.shape[1] else (torch.zeros(B, 1, H, D), torch.full((B, H, 1), -float("inf")))
            of, lf = orc.attention(q1g, kf, vf) if kf.shape[1] else (torch.zeros(B, 1, H, D), torch.full((B, H, 1), -float("inf")))
            return orc.merge2(on, ln, of, lf)

        from jetlm.kernels.sequence_parallel import PartialBuffer
        buf = PartialBuffer(shard, (B, 1, H, D), (B, H, 1), torch.float32, "cpu")      # in-place gather path

        def local_dec_into(out, lse):
            o, l = local_dec()
            out.copy_(o); lse.copy_(l)

        od, ld = sharded_attention(local_dec_into, merge, shard, buf)
        od2, ld2 = sharded_attention(local_dec, merge, shard)
        assert torch.equal(od, od2) and torch.equal(ld, ld2)
        eod, eld = orc.jetlong_decode(q1, q1g, kb[:, boundary:], v[:, boundary:], kg[:, :boundary], v[:, :boundary])
        dd, _ = orc.compare(od, eod)
        dld, _ = orc.compare(ld, eld)
        # the peer-memory exchange cannot be set up on CPU ranks: every rank must learn that (one all-reduce)
        # and take the collective path together, whatever the environment asks for
        import warnings
        from jetlm.kernels.sequence_parallel import make_peer_exchange
        for mode in ("", "0", "1"):
            os.environ["JETLONG_PEER_EXCHANGE"] = mode
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                assert make_peer_exchange(shard, 1, H, D, torch.device("cpu")) is None
        os.environ.pop("JETLONG_PEER_EXCHANGE")
        # the K/V-gather form of the token-sharded prefill: every rank contributes its block-cyclic stripe of the
        # keys and values, one all-gather, one strided copy -> the whole sequence in position order on every rank
        from jetlm.kernels.sequence_parallel import interleave_stripes
        n_full = 2 * world * block                              # two whole blocks per rank
        seq = torch.randn(2, B, n_full, Hk, 8)                  # [K / V], same on every rank (seeded)
        mine = shard.owned_rows(n_full)
        stage = torch.empty(world, 2, B, mine.numel(), Hk, 8)
        stage[rank] = seq[:, :, mine]
        dist.all_gather_into_tensor(stage.view(-1), stage[rank].clone().view(-1))
        full = interleave_stripes(stage, block, torch.empty(2, B, n_full, Hk, 8))
        assert torch.equal(full, seq)
        results[rank] = (d, cos, dl, dd, dld)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,block", [(2, 128), (3, 64)])
def test_sharded_attention_equals_full_attention(world, block):
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, block, results), nprocs=world, join=True)
        assert len(results) == world
        for rank, (d, cos, dl, dd, dld) in results.items():
            assert d < 1e-5 and cos > 0.99999 and dl < 1e-5 and dd < 1e-5 and dld < 1e-5, (rank, d, cos, dl, dd, dld)


def test_stripe_geometry_partitions_the_keys():
    sys.path[:0] = [PKG]
    from jetlm.kernels.sequence_parallel import SequenceShard
    for n_keys in (1, 127, 128, 1000, 4097):
        for world in (1, 2, 4, 8):
            rows = [SequenceShard(r, world, block=128).owned_rows(n_keys) for r in range(world)]
            allrows = torch.cat(rows).sort().values
            assert torch.equal(allrows, torch.arange(n_keys))
            ranges = [SequenceShard(r, world).contiguous_range(n_keys) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n_keys
            assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))


def test_token_sharded_prefill_picks_the_smaller_exchange(monkeypatch):
    """K/V gather while the cache is at most H/Hk times longer than the chunk (its bytes are then the smaller ones),
    Q exchange for the late chunks of a long chunked prefill; the environment variable overrides."""
    sys.path[:0] = [PKG]
    from jetlm.kernels.cute_jetlong_backend import token_sharded_prefill_mode as mode
    monkeypatch.delenv("JETLONG_SP_PREFILL", raising=False)
    assert mode(8, 131072, 131072, 32, 8) == "kv_gather"            # a fresh prompt
    assert mode(8, 4 * 32768, 32768, 32, 8) == "kv_gather"          # cache = 4 chunks at 32 / 8 heads: the break-even
    assert mode(8, 5 * 32768, 32768, 32, 8) == "q_exchange"
    assert mode(8, 1048576, 32768, 32, 8) == "q_exchange"           # the last chunk of a 1M-token prompt
    assert mode(2, 65536, 65536, 16, 16) == "kv_gather"             # no grouped-query advantage, still no return trip
    monkeypatch.setenv("JETLONG_SP_PREFILL", "q")
    assert mode(8, 131072, 131072, 32, 8) == "q_exchange"
    monkeypatch.setenv("JETLONG_SP_PREFILL", "kv")
    assert mode(8, 1048576, 32768, 32, 8) == "kv_gather"


def _token_sharded_worker(rank, world, port, block, mode, results):
    """The token-sharded prefill drivers - "q_exchange" (stripe batching, own stripe in the first launch, exchange,
    N-way merge) and "kv_gather" (all-gather, stripe interleave, local regroup, one launch) - with the CPU oracle
    standing in for the kernels and point-to-point sends standing in for the all-to-all (gloo has none); symmetric
    memory does not exist on CPU ranks, so the Q exchange takes its collective path."""
    sys.path[:0] = [PKG, os.path.join(ROOT, "oracle")]
    import types
    import jetlong_oracle as orc
    from jetlm.kernels import cute_jetlong_backend as be
    from jetlm.kernels.sequence_parallel import SequenceShard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), JETLONG_PREFILL_PEER_COPY="0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(11)                                  # same tensors on every rank
        B, H, Hk, D, w0, G = 1, 4, 2, 128, 90, 3
        n_blocks_q, n_blocks_cached = 2, 1                     # per rank: the chunk holds 2 blocks, 1 block was cached before
        S_loc = n_blocks_q * block
        S, cached = S_loc * world, n_blocks_cached * block * world
        Skv = cached + S
        inv = orc.default_inv_freq()
        pos = torch.arange(Skv)
        q = torch.randn(B, S, H, D)
        k, v = torch.randn(B, Skv, Hk, D), torch.randn(B, Skv, Hk, D)
        regroup = lambda x, p: orc.rotate_bshd(x, orc.regroup_delta(p.view(1, -1), G), inv)
        kg = regroup(k, pos)
        expect, _ = orc.jetlong_prefill(q, regroup(q, pos[cached:]), k, kg, v, seqstart=cached, w0=w0)

        def positions(n, pos0, blk, stride):
            i = torch.arange(n)
            return pos0 + i if blk <= 0 else pos0 + (i // blk) * stride + i % blk

        calls = []

        def rope_regroup(x, inv_freq, *, group_size, pos0=0, pos_block=0, pos_block_stride=0, out=None):
            r = regroup(x, positions(x.shape[1], pos0, pos_block, pos_block_stride))
            return r if out is None else out.copy_(r)

        def posmap_prefill(q_ops, k_ops, value, *, pmap, q_pos0, k_pos0=0, q_block=0, q_block_stride=0, k_block=0,
                           k_block_stride=0, softmax_scale=None, out=None, lse=None, stripes=None, return_lse=True):
            out = torch.empty_like(q_ops[0]) if out is None else out
            lse = torch.empty(q_ops[0].shape[0], q_ops[0].shape[2], q_ops[0].shape[1]) if lse is None else lse
            first, count, step = stripes if stripes is not None else (0, q_ops[0].shape[0], 0)
            wrap = q_ops[0].shape[0]
            calls.append((first, count))
            pk = positions(k_ops[0].shape[1], k_pos0, k_block, k_block_stride).view(1, 1, -1)
            for i in range(count):
                e = (first + i) % wrap if stripes is not None else i
                pq = positions(q_ops[0].shape[1], q_pos0 + e * step, q_block, q_block_stride).view(1, -1, 1)
                near, far = (pk <= pq) & (pk >= pq - pmap), pk < pq - pmap
                on, ln = orc.attention(q_ops[0][e:e + 1], k_ops[0], value, near, softmax_scale)
                of, lf = orc.attention(q_ops[1][e:e + 1], k_ops[1], value, far, softmax_scale)
                o, l = orc.merge2(on, ln, of, lf)
                out[e:e + 1].copy_(o)
                lse[e:e + 1].copy_(l)
            return (out, lse) if return_lse else out

        def merge_partials(outs, lses, return_lse=True):
            o, l = orc.merge_partials(torch.stack(list(outs)), torch.stack(list(lses)))
            return (o, l) if return_lse else o

        be.ops = types.SimpleNamespace(PositionMap=types.SimpleNamespace(jetlong=lambda w: w), rope_regroup=rope_regroup,
                                       posmap_prefill=posmap_prefill, merge_partials=merge_partials)

        def all_to_all(outs, ins, group=None, async_op=False):
            works = [dist.isend(t.contiguous(), d) for d, t in enumerate(ins) if t.numel()]
            works += [dist.irecv(t, s) for s, t in enumerate(outs) if t.numel()]
            for w in works:
                w.wait()
            return types.SimpleNamespace(wait=lambda: None)

        dist.all_to_all = all_to_all
        shard = SequenceShard(rank, world, block=block)
        be.configure_sequence_sharding(shard)
        mine_q = shard.owned_rows(S)                            # rows of the chunk, relative to its start
        mine_k = shard.owned_rows(Skv)
        out = be.fused_jetlong_prefill_token_sharded(
            q[:, mine_q].contiguous(), k[:, mine_k].contiguous(), kg[:, mine_k].contiguous(), v[:, mine_k].contiguous(),
            q_start=cached, inv_freq=inv, group_size=G, window_size_left=w0, softmax_scale=D ** -0.5, mode=mode)
        d, cos = orc.compare(out, expect[:, mine_q])
        if mode == "q_exchange":       # one batched launch for my own stripe and the first half of the others, one for the rest
            first = (world - 1 + 1) // 2
            want = [(rank, 1 + first)] + ([((rank + 1 + first) % world, world - 1 - first)] if world - 1 - first else [])
        else:                           # one launch of my query stripe against all the gathered keys
            want = [(0, 1)]
        results[rank] = (d, cos, calls == want)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["q_exchange", "kv_gather"])
@pytest.mark.parametrize("world,block", [(2, 64), (3, 32)])
def test_token_sharded_prefill_drivers(world, block, mode):
    port = _free_port()
    results = mp.Manager().dict()
    mp.spawn(_token_sharded_worker, args=(world, port, block, mode, results), nprocs=world, join=True)
    assert len(results) == world
    for r in range(world):
        d, cos, launches_as_planned = results[r]
        assert d <= 2e-5 and cos >= 0.99999, (r, d, cos)
        assert launches_as_planned, r
