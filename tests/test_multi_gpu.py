"""KV-sequence-sharded prefill and decode on 2+ GPUs (NCCL): every rank must end with the result of
the unsharded kernels.  Skipped unless at least two CUDA devices are visible."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from conftest import PKG, ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    sys.path[:0] = [PKG, os.path.join(ROOT, "oracle")]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    import jetlong_oracle as orc
    from jetlm.kernels import cute_jetlong_backend as be
    from jetlm.kernels.sequence_parallel import SequenceShard
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        torch.manual_seed(5)
        B, S, Skv, H, Hk, D, w0, G = 1, 1500, 2300, 8, 4, 128, 300, 3
        inv = orc.default_inv_freq().cuda()
        mk = lambda *shape: torch.randn(*shape, device="cuda").bfloat16()
        qb, qg = mk(B, H, S, D), mk(B, H, S, D)                     # (B,H,S,D) as the modeling file hands over
        kb, kg, v = mk(B, Hk, Skv, D), mk(B, Hk, Skv, D), mk(B, Hk, Skv, D)
        kw = dict(seqstart_q=Skv - S, window_size_left=w0, softmax_scale=D ** -0.5, has_any_pad=False, training=False)
        ref = be.fused_jetlong_prefill(qb, qg, kb, kg, v, **kw)
        be.configure_sequence_sharding(SequenceShard(rank, world, block=256))
        got = be.fused_jetlong_prefill(qb, qg, kb, kg, v, **kw)
        d_pre, cos_pre = orc.compare(got.float().cpu(), ref.float().cpu())
        # decode off the cache with in-kernel regroup
        q1, q1g = mk(B, 1, H, D), mk(B, 1, H, D)
        dk = dict(boundary=Skv - 1 - w0, inv_freq=inv, group_size=G, has_any_pad=False, training=False, return_lse=True)
        o_sh, l_sh = be.fused_jetlong_decode_cache(q1, q1g, kb, v, **dk)
        # the same decode from block-cyclic cache stripes (what the token-sharded prefill leaves behind)
        sh = SequenceShard(rank, world, block=256)
        o_st, l_st = be.fused_jetlong_decode_cache_stripe(q1, q1g, sh.take_stripe(kb, dim=2), sh.take_stripe(v, dim=2),
                                                           boundary=Skv - 1 - w0, inv_freq=inv, group_size=G, return_lse=True)
        be.configure_sequence_sharding(None)
        o_1, l_1 = be.fused_jetlong_decode_cache(q1, q1g, kb, v, **dk)
        d_st, cos_st = orc.compare(o_st.float().cpu(), o_1.float().cpu())
        d_lst, _ = orc.compare(l_st.cpu(), l_1.cpu())
        assert d_st <= 2e-2 and cos_st >= 0.9999 and d_lst <= 1e-3, (rank, d_st, cos_st, d_lst)
        d_dec, cos_dec = orc.compare(o_sh.float().cpu(), o_1.float().cpu())
        d_lse, _ = orc.compare(l_sh.cpu(), l_1.cpu())
        # token-sharded (sequence-parallel) model forward vs the unsharded forward of the same weights
        import json
        from transformers.models.qwen3.configuration_qwen3 import Qwen3Config
        from jetlm.modeling.jetlong_fused import Qwen3JetLongFusedForCausalLM
        with open(os.path.join(PKG, "model_configs", "Qwen3-1.7B-Base-jetlong_fused", "config.json")) as f:
            d = json.load(f)
        d.pop("auto_map"); d.pop("architectures")
        d.update(dict(num_hidden_layers=2, vocab_size=256, hidden_size=256, intermediate_size=512,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_window_layers=2))
        cfg = Qwen3Config(**d)
        cfg.jetlong["w"], cfg.jetlong["w_0"] = 300, 130
        cfg._attn_implementation = "sdpa"
        torch.manual_seed(11)
        model = Qwen3JetLongFusedForCausalLM(cfg).eval().to("cuda", torch.bfloat16)
        model.model.rotary_emb.inv_freq = orc.default_inv_freq().cuda()
        ids = torch.randint(0, 256, (1, 256 * world * 3), device="cuda")
        with torch.inference_mode():
            full = model(input_ids=ids).logits.float()
            shard = SequenceShard(rank, world, block=256)
            be.configure_sequence_sharding(shard)
            model.model.token_sharded = True
            rows = shard.owned_rows(ids.shape[1]).cuda()
            d_tok, cos_tok = 0.0, 1.0
            for forced in ("kv", "q"):          # both exchanges: gathered K / V, and gathered Q + returned partials
                os.environ["JETLONG_SP_PREFILL"] = forced
                local = model(input_ids=ids).logits.float()
                assert be.LAST_TOKEN_SHARDED_MODE == ("kv_gather" if forced == "kv" else "q_exchange")
                d, c = orc.compare(local.cpu(), full[:, rows].cpu())
                d_tok, cos_tok = max(d_tok, d), min(cos_tok, c)
            os.environ.pop("JETLONG_SP_PREFILL")
            be.configure_sequence_sharding(None)
            model.model.token_sharded = False
        # chunked prefill (first chunk inside the window) + decode steps on a striped static cache vs the
        # same schedule on one GPU; then the greedy driver, which must return the same tokens on every rank
        from jetlm.kernels.kv_cache import BifocalKVCache
        chunk, n_dec = 256 * world, 6
        model.model.rotary_emb.jetlong_w = chunk + 44          # chunk 1 inside the window (G=1), then G = 2, 3
        ids2 = torch.randint(0, 256, (1, 3 * chunk + n_dec), device="cuda")

        def drive(cache):
            outs = [model(input_ids=ids2[:, c * chunk: (c + 1) * chunk], past_key_values=cache, use_cache=True).logits.float()
                    for c in range(3)]
            steps = [model(input_ids=ids2[:, t: t + 1], past_key_values=cache, use_cache=True).logits.float()
                     for t in range(3 * chunk, 3 * chunk + n_dec)]
            return torch.cat(outs, 1), torch.cat(steps, 1)

        with torch.inference_mode():
            model.model.kernels_within_window = True
            pre_1, dec_1 = drive(BifocalKVCache(cfg, ids2.shape[1], device="cuda", dtype=torch.bfloat16))
            toks_1 = model.generate_long(ids2[:, : 3 * chunk], max_new_tokens=4, chunk_tokens=chunk)
            be.configure_sequence_sharding(shard)
            model.model.token_sharded = True
            cache = BifocalKVCache(cfg, ids2.shape[1], device="cuda", dtype=torch.bfloat16, shard=shard)
            pre_n, dec_n = drive(cache)
            toks_n = model.generate_long(ids2[:, : 3 * chunk], max_new_tokens=4, chunk_tokens=chunk)
            toks_g = model.generate_long(ids2[:, : 3 * chunk], max_new_tokens=4, chunk_tokens=chunk, cuda_graph=True)
            assert toks_g.tolist() == toks_n.tolist(), (rank, toks_g.tolist(), toks_n.tolist())
            os.environ["JETLONG_PEER_EXCHANGE"] = "0"       # the same graph decode with NCCL all-gather + jl_merge instead of jl_peer_merge
            toks_c = model.generate_long(ids2[:, : 3 * chunk], max_new_tokens=4, chunk_tokens=chunk, cuda_graph=True)
            os.environ.pop("JETLONG_PEER_EXCHANGE")
            assert toks_c.tolist() == toks_n.tolist(), (rank, toks_c.tolist(), toks_n.tolist())
            # jl_peer_merge alone: five exchanges of fresh random partials against all-gather + jl_merge
            from jetlm.kernels import jetlong_ops as jops
            from jetlm.kernels.sequence_parallel import PeerExchange
            ex = PeerExchange(shard, 2, 8, 128, torch.device("cuda", rank))
            epoch = torch.zeros(1, dtype=torch.int64, device="cuda")
            for it in range(1, 6):
                gen = torch.Generator(device="cuda").manual_seed(1000 * it + rank)
                po = torch.randn(2, 1, 8, 128, device="cuda", generator=gen).bfloat16()
                pl = torch.randn(2, 8, 1, device="cuda", generator=gen) * 3
                if it == 3 and rank == 0:
                    pl.fill_(float("-inf"))                 # a rank without keys contributes nothing
                epoch.fill_(it)
                got_o, got_l = jops.peer_merge(po, pl, ex, epoch_base=epoch, epoch_stride=1, epoch_offset=0, return_lse=True)
                all_o = [torch.empty_like(po) for _ in range(world)]
                all_l = [torch.empty_like(pl) for _ in range(world)]
                dist.all_gather(all_o, po)
                dist.all_gather(all_l, pl)
                want_o, want_l = jops.merge_partials(all_o, all_l)
                assert torch.equal(got_o, want_o), (rank, it, (got_o.float() - want_o.float()).abs().max())
                assert torch.allclose(got_l, want_l, atol=1e-5), (rank, it)
            assert not ex.failed()
            gathered = [torch.empty_like(toks_n) for _ in range(world)]
            dist.all_gather(gathered, toks_n)
            be.configure_sequence_sharding(None)
            model.model.token_sharded = False
        assert cache.get_seq_length() == ids2.shape[1]
        assert cache.layers[0].rows == shard.n_owned(ids2.shape[1])
        assert all(torch.equal(t, toks_n) for t in gathered)
        rows_c = torch.cat([shard.owned_rows(chunk) + c * chunk for c in range(3)]).cuda()
        d_cpre, cos_cpre = orc.compare(pre_n.cpu(), pre_1[:, rows_c].cpu())
        d_cdec, cos_cdec = orc.compare(dec_n.cpu(), dec_1.cpu())
        assert cos_cpre >= 0.999 and d_cpre <= 0.15, (rank, d_cpre, cos_cpre)
        assert cos_cdec >= 0.999 and d_cdec <= 0.15, (rank, d_cdec, cos_cdec)
        results[rank] = (d_pre, cos_pre, d_dec, cos_dec, d_lse, d_tok, cos_tok)
    finally:
        dist.destroy_process_group()


def test_sharded_kernels_match_unsharded():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    port = _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert len(results) == world
        for rank, (d_pre, cos_pre, d_dec, cos_dec, d_lse, d_tok, cos_tok) in results.items():
            assert cos_tok >= 0.999 and d_tok <= 0.15, (rank, d_tok, cos_tok)     # logits after 2 bf16 layers
            # partials are rounded to bf16 before the merge: one extra rounding step
            assert d_pre <= 2e-2 and cos_pre >= 0.9999, (rank, d_pre, cos_pre)
            assert d_dec <= 2e-2 and cos_dec >= 0.9999 and d_lse <= 1e-3, (rank, d_dec, cos_dec, d_lse)
